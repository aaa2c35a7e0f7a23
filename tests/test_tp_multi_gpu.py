"""GPU, two or more devices: the column-sharded tensor-parallel paths on real peers (one process per
GPU, NCCL for the rendezvous, NVLink peer stores for the data).  Skipped with fewer than two
visible GPUs; the single-GPU emulation of the same kernels is in test_gpu_parity.py.

What is asserted on EVERY rank, for the slices that arrive from the other GPUs as much as for
its own: the gathered result equals the unsharded single-GPU result -- bit for bit for the
decode GEMV (rows are independent and the per-row arithmetic does not depend on the sharding),
within fp32-reordering noise for the tensor-core GEMM (a different split of K may apply)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out_dir):
    for p in (str(ROOT), str(ROOT / "vllm-gguf-plugin-prism_b200"), str(ROOT / "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from gguf_b200 import capi, synth, tp
        from helpers import rel_l2

        def weight(t, n, k, seed):
            return torch.from_numpy(synth.make_weight(t, n, k, seed=seed)).to(dev)

        def act(m, k, seed, dtype=torch.float16):
            return torch.from_numpy(synth.make_activation(m, k, seed=seed, dtype=np.float32)).to(dev).to(dtype)

        # ---- decode: packets over NVLink, chained through the quantizer ------------------------
        n_up = 2048                                       # up: K=1024 -> N=2048 ; down: K=2048 -> N=1024
        fused = tp.FusedGatherGemv(n_up, 6, torch.float16, dev, reduce_n=1024)
        for name, t in (("Q4_K", 12), ("IQ2_XXS", 16), ("Q8_0", 8)):
            w_up, w_dn = weight(t, n_up, 1024, 1), weight(t, 1024, n_up, 2)
            x = act(1, 1024, 3)
            s = 2.0 ** -10
            for rep in range(3):
                fused(0, tp.shard_rows(w_up, rank, world), x, t)                                  # y0 = W_up x
                fused(1, tp.shard_rows(w_dn, rank, world), None, t, add_slot=0, add_scale=s)       # y1 = W_dn (s * y0)
                fused(2, tp.shard_rows(w_up, rank, world), x, t, add_slot=1, add_scale=s)          # y2 = W_up (x + s * y1)
                got = [fused.gathered(0), fused.gathered(1, n=1024), fused.gathered(2)]
                y0 = capi.mul_mat_vec_a8(w_up, x, t, n_up)
                x1 = (s * y0.float()).half()
                y1 = capi.mul_mat_vec_a8(w_dn, x1, t, 1024)
                x2 = (x.float() + s * y1.float()).half()
                y2 = capi.mul_mat_vec_a8(w_up, x2, t, n_up)
                torch.cuda.synchronize()
                assert capi.last_status() == 0
                assert torch.equal(got[0], y0), f"{name}: gathered GEMV differs from the unsharded one (rank {rank})"
                assert torch.equal(got[1], y1), f"{name}: chained call 1 differs (rank {rank})"
                assert torch.equal(got[2], y2), f"{name}: chained call 2 differs (rank {rank})"
                dist.barrier()   # nobody rewrites slot 0 while a slower rank still unpacks it
        # ---- row-parallel decode: K-shards, fp32 partial sums to every rank, summed in rank order ---
        # (the pairing of a tensor-parallel MLP: up = column-parallel, down = row-parallel on this
        #  rank's slice of the up result, ONE reduction per pair)
        for name, t in (("Q4_K", 12), ("Q8_0", 8)):
            w_up, w_dn = weight(t, n_up, 1024, 11), weight(t, 1024, n_up, 12)
            x = act(1, 1024, 13)
            s = 2.0 ** -10
            for rep in range(2):
                fused(3, tp.shard_rows(w_up, rank, world), x, t)                                       # y0 = W_up x          (gathered)
                fused.rowpar(4, tp.shard_cols(w_dn, t, rank, world), None, t, add_slot=3, add_scale=s)  # y1 = W_dn (s * y0)   (reduced)
                fused(5, tp.shard_rows(w_up, rank, world), x, t, add_slot=4, add_scale=s, add_parts=world)   # y2 = W_up (x + s * y1)
                got1, got2 = fused.reduced(4, 1024), fused.gathered(5)
                y0 = capi.mul_mat_vec_a8(w_up, x, t, n_up)
                x1 = (s * y0.float()).half()
                kl = n_up // world
                parts = [capi.mul_mat_vec_a8(tp.shard_cols(w_dn, t, r, world), x1[:, r * kl:(r + 1) * kl].contiguous().float(), t, 1024)
                         for r in range(world)]
                acc = parts[0].clone()
                for p_ in parts[1:]:
                    acc += p_
                y1 = acc.half()
                y2 = capi.mul_mat_vec_a8(w_up, (x.float() + s * y1.float()).half(), t, n_up)
                torch.cuda.synchronize()
                assert capi.last_status() == 0
                assert torch.equal(got1.view(1, -1), y1), f"{name}: reduced row-parallel GEMV differs (rank {rank})"
                assert torch.equal(got2, y2), f"{name}: call after the reduction differs (rank {rank})"
                full = capi.mul_mat_vec_a8(w_dn, x1, t, 1024)
                assert rel_l2(got1.float().cpu().view(1, -1), full.float().cpu()) <= 1e-3
                dist.barrier()
            y_nccl = tp.RowParallelGGUFLinear(w_dn, t, matmul=lambda xx, ww, tt: capi.mul_mat_vec_a8(ww, xx, tt, ww.shape[0]))(
                x1[:, rank * kl:(rank + 1) * kl].contiguous())
            assert rel_l2(y_nccl.float().cpu(), full.float().cpu()) <= 2e-3
        # ---- decode through NCCL (the plain collective, for reference) -------------------------
        w = weight(12, 1024, 2048, 5)
        x = act(1, 2048, 6)
        layer = tp.ColumnParallelGGUFLinear(w, 12, matmul=lambda xx, ww, tt: capi.mul_mat_vec_a8(ww, xx, tt, ww.shape[0]))
        assert torch.equal(layer(x), capi.mul_mat_vec_a8(w, x, 12, 1024))
        # ---- prefill: tiles stored into every rank's output, per-call flags --------------------
        mm = tp.FusedGatherMatmul(130, 2048, 2, torch.float16, dev)
        for name, t, op, n, k, m in (("Q4_K", 12, capi.OP_MMQ, 2048, 2048, 130), ("IQ2_XXS", 16, capi.OP_DEQUANT_MATMUL, 1024, 4096, 128),
                                     ("Q6_K", 14, capi.OP_MMQ, 1024, 8192, 64)):
            w, x = weight(t, n, k, 7), act(m, k, 8)
            want = capi.mul_mat_a8(w, x, t, n) if op == capi.OP_MMQ else capi.dequant_matmul(w, x, t, n)
            for rep in range(2):
                y = mm(rep, op, tp.shard_rows(w, rank, world), x, t)
                torch.cuda.synchronize()
                assert capi.last_status() == 0
                assert rel_l2(y.float().cpu(), want.float().cpu()) <= 3e-4, f"{name}: gathered GEMM differs (rank {rank})"
            dist.barrier()
            y_nccl = tp.ColumnParallelGGUFLinear(w, t, matmul=lambda xx, ww, tt: (capi.mul_mat_a8 if op == capi.OP_MMQ else capi.dequant_matmul)(ww, xx, tt, ww.shape[0]))(x)
            assert rel_l2(y_nccl.float().cpu(), want.float().cpu()) <= 3e-4
        torch.cuda.synchronize()
        dist.barrier()
        (Path(out_dir) / f"ok{rank}").write_text("ok")
        dist.destroy_process_group()
    except BaseException:
        # leave at once, idle (every wait of the kernels is bounded), without a collective that
        # the other ranks may never join
        import traceback

        traceback.print_exc()
        torch.cuda.synchronize()
        os._exit(1)


def test_tensor_parallel_on_real_peers(native_libs, tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    port = 29700 + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
