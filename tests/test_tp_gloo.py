"""CPU: the column-sharded tensor-parallel wrapper on 2 gloo ranks.  The local matmul is replaced by
the CPU oracle (test infrastructure), so this covers the host logic: row slicing of the packed
weight, the all-gather and the reassembly of the output columns."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, qtype, n, k, m, out_dir):
    for p in (str(ROOT), str(ROOT / "vllm-gguf-plugin-prism_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gguf_b200 import synth, tp
        from oracle import cpu

        def oracle_matmul(x, w, t):
            y64, _ = cpu.matmul_a8(w.numpy(), t, x.numpy(), "float16", mmq=False)
            return torch.from_numpy(y64.astype(np.float32))

        w = torch.from_numpy(synth.make_weight(qtype, n, k, seed=3))
        x = torch.from_numpy(synth.make_activation(m, k, seed=4))
        layer = tp.ColumnParallelGGUFLinear(w, qtype, matmul=oracle_matmul)
        assert layer.weight.shape[0] == n // world
        assert torch.equal(layer.weight, w[rank * n // world:(rank + 1) * n // world])
        y = layer(x)
        full = oracle_matmul(x, w, qtype)
        assert y.shape == (m, n)
        assert torch.equal(y, full), "sharded result must equal the unsharded one exactly"
        with pytest.raises(ValueError):
            tp.shard_rows(w[:n - 1], rank, world)
        # row-parallel: whole blocks of every row per rank, this rank's K/g activations, all-reduce
        if (k // synth.QUANT_SIZES[qtype][0]) % world == 0:
            row = tp.RowParallelGGUFLinear(w, qtype, matmul=oracle_matmul)
            bw = w.shape[1] // world
            assert torch.equal(row.weight, w[:, rank * bw:(rank + 1) * bw])
            y_row = row(x[:, rank * k // world:(rank + 1) * k // world].contiguous())
            assert y_row.shape == (m, n)
            err = float(torch.linalg.norm(y_row - full) / torch.linalg.norm(full))
            assert err <= 1e-5, err   # (same products, summed in two halves)
        with pytest.raises(ValueError):
            tp.shard_cols(w[:, : synth.QUANT_SIZES[qtype][1]], qtype, rank, world)   # one block per row cannot be split in two
        (Path(out_dir) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", [(16, 64, 8192 // 16, 1), (8, 30, 1024, 3)])
def test_column_parallel_two_ranks(tmp_path, case):
    qtype, n, k, m = case
    port = 29500 + (os.getpid() % 500) + qtype
    mp.spawn(_worker, args=(2, port, qtype, n, k, m, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_moe_weight_sharding_follows_the_row_dim():
    sys.path.insert(0, str(ROOT / "vllm-gguf-plugin-prism_b200"))
    from gguf_b200 import tp

    w = torch.arange(4 * 6 * 5, dtype=torch.uint8).reshape(4, 6, 5)
    s = tp.shard_rows(w, 1, 3)
    assert s.shape == (4, 2, 5) and torch.equal(s, w[:, 2:4])
