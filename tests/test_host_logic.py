"""CPU: host-side logic of the drop-in layer -- dispatcher routing against the table recorded
from the reference's own dispatcher, the routing/alignment restatements, the linear method's
shard handling.  No kernel runs: the operator functions are replaced by recorders."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from gguf_b200 import synth

ROUTING = json.loads((Path(__file__).parent / "golden" / "golden_routing.json").read_text())


@pytest.fixture()
def recorded_ops(monkeypatch, native_libs):
    from vllm_gguf_plugin import ops
    from vllm_gguf_plugin.quantization import linear

    calls = []

    def rec(name, fn):
        def f(*a, **kw):
            calls.append(name)
            return fn(*a)
        return f

    monkeypatch.setattr(ops, "ggml_mul_mat_vec_a8", rec("ggml_mul_mat_vec_a8", lambda W, X, t, row: torch.zeros(X.shape[0], row)))
    monkeypatch.setattr(ops, "ggml_mul_mat_a8", rec("ggml_mul_mat_a8", lambda W, X, t, row: torch.zeros(X.shape[0], row)))
    monkeypatch.setattr(ops, "ggml_dequantize", rec("ggml_dequantize", lambda W, t, m, n, dt: torch.zeros(m, n, dtype=dt)))
    # the fused IQ route stands where the reference calls ggml_dequantize and then matmuls
    monkeypatch.setattr(ops, "ggml_dequant_matmul", rec("ggml_dequantize", lambda W, X, t, row: torch.zeros(X.shape[0], row)))
    return calls, linear


def test_dispatcher_routes_like_the_reference(recorded_ops):
    calls, linear = recorded_ops
    assert len(ROUTING) == 528
    for case in ROUTING:
        t, rows, m = case["type"], case["rows"], case["m"]
        bs, ts = synth.QUANT_SIZES[t]
        calls.clear()
        w = torch.zeros(rows, 256 // bs * ts, dtype=torch.uint8)
        x = torch.zeros(m, 256, dtype=torch.float16)
        y = linear._fused_mul_mat_gguf(x, w, t)
        assert list(y.shape) == [m, rows]
        assert calls == case["calls"], (case, calls)


def test_dispatcher_rejects_unknown_type(recorded_ops):
    _, linear = recorded_ops
    with pytest.raises(NotImplementedError):
        linear._fused_mul_mat_gguf(torch.zeros(1, 256, dtype=torch.float16), torch.zeros(4, 10, dtype=torch.uint8), 99)


def test_moe_align_restatements_agree(native_libs):
    from vllm_gguf_plugin.quantization.fused_moe import moe_align_block_size_torch

    for (T, E, k, blk) in [(50, 8, 2, 4), (256, 64, 8, 64), (3, 16, 4, 64), (70, 5, 1, 32)]:
        _, ids = synth.make_routing(T, E, k, T)
        s0, e0, n0 = synth.moe_align_block_size(ids, blk, E)
        s1, e1, n1 = moe_align_block_size_torch(torch.from_numpy(ids), blk, E)
        n = int(n0[0])
        assert n == int(n1[0]) and n % blk == 0
        assert np.array_equal(s0[:n], s1[:n].numpy())
        assert np.array_equal(e0[:n // blk], e1[:n // blk].numpy())
        slots = np.sort(s0[:n][s0[:n] < T * k])
        assert np.array_equal(slots, np.arange(T * k))           # every slot exactly once
        for b in range(n // blk):                                 # a block holds one expert's slots
            blk_ids = s0[b * blk:(b + 1) * blk]
            real = blk_ids[blk_ids < T * k]
            assert (ids.reshape(-1)[real] == e0[b]).all()


def test_linear_method_merges_same_type_shards_into_one_call(recorded_ops):
    calls, linear = recorded_ops
    m = linear.GGUFLinearMethod(quant_config=None)
    layer = torch.nn.Module()
    m.create_weights(layer, 256, [8, 4, 4], 256, 16, torch.float16)
    for sid, rows in (("q", 8), ("k", 4), ("v", 4)):
        layer.weight.weight_loader(layer.weight, torch.zeros(rows, 144, dtype=torch.uint8), sid)
        layer.weight_type.weight_loader(layer.weight_type, torch.tensor(12), sid)
    m.process_weights_after_loading(layer)
    assert tuple(layer.weight.shape) == (16, 144)
    assert layer.weight.shard_offset_map == {"q": (0, 8, 144), "k": (8, 12, 144), "v": (12, 16, 144)}
    calls.clear()
    y = m.apply(layer, torch.zeros(1, 256, dtype=torch.float16), bias=torch.ones(16))
    assert calls == ["ggml_mul_mat_vec_a8"] and tuple(y.shape) == (1, 16) and float(y.sum()) == 16.0


def test_linear_method_mixed_type_shards_call_per_shard(recorded_ops):
    calls, linear = recorded_ops
    m = linear.GGUFLinearMethod(quant_config=None)
    layer = torch.nn.Module()
    m.create_weights(layer, 256, [8, 8], 256, 16, torch.float16)
    layer.weight.weight_loader(layer.weight, torch.zeros(8, 144, dtype=torch.uint8), 0)
    layer.weight.weight_loader(layer.weight, torch.zeros(8, 210, dtype=torch.uint8), 1)
    layer.weight_type.weight_loader(layer.weight_type, torch.tensor(12), 0)
    layer.weight_type.weight_loader(layer.weight_type, torch.tensor(14), 1)
    m.process_weights_after_loading(layer)
    assert tuple(layer.weight.shape) == (16, 210)
    calls.clear()
    y = m.apply(layer, torch.zeros(9, 256, dtype=torch.float16))
    assert calls == ["ggml_mul_mat_a8", "ggml_mul_mat_a8"] and tuple(y.shape) == (9, 16)


def _strict_set_weight_attrs(weight, attrs):
    """vLLM's set_weight_attrs: refuses to overwrite an attribute that is already there."""
    for k, v in (attrs or {}).items():
        assert not hasattr(weight, k), f"Overwriting existing tensor attribute: {k}"
        setattr(weight, k, v)


def test_create_weights_accepts_vllm_weight_loader_extra(recorded_ops, monkeypatch):
    """vLLM's LinearBase / FusedMoE always pass `weight_loader` among the extras and its
    set_weight_attrs asserts on overwrite: both create_weights must pop it first."""
    _, linear = recorded_ops
    from vllm_gguf_plugin.quantization import fused_moe

    monkeypatch.setattr(linear, "set_weight_attrs", _strict_set_weight_attrs)
    monkeypatch.setattr(fused_moe, "set_weight_attrs", _strict_set_weight_attrs)
    theirs = lambda *a, **k: None
    layer = torch.nn.Module()
    linear.GGUFLinearMethod(None).create_weights(layer, 256, [16], 256, 16, torch.float16, weight_loader=theirs)
    assert layer.weight.fallback_weight_loader is theirs and layer.weight.weight_loader is not theirs
    moe = torch.nn.Module()
    fused_moe.GGUFMoEMethod(None).create_weights(moe, 4, 256, 128, torch.float16, weight_loader=theirs)
    assert moe.w13_weight.base_weight_loader is theirs and callable(moe.w2_weight.weight_loader)


@pytest.mark.parametrize("rank", [0, 1])
def test_linear_loader_slices_for_tensor_parallel_ranks(recorded_ops, monkeypatch, rank):
    """Column-parallel layers keep rows [r*N/g, ...) (reference params.py:227-236), row-parallel
    layers keep whole blocks [r*bytes/g, ...) of every row (params.py:259-264)."""
    _, linear = recorded_ops
    monkeypatch.setattr(linear, "tensor_parallel_rank_and_size", lambda: (rank, 2))
    full = torch.arange(16 * 288, dtype=torch.int64).remainder(251).to(torch.uint8).reshape(16, 288)   # 2 Q4_K blocks per row
    m = linear.GGUFLinearMethod(None)
    col = torch.nn.Module()
    m.create_weights(col, 512, [8], 512, 16, torch.float16)          # 8 of 16 output rows per rank
    col.weight.weight_loader(col.weight, full)
    col.weight_type.weight_loader(col.weight_type, torch.tensor(12))
    m.process_weights_after_loading(col)
    assert torch.equal(col.weight.data, full[rank * 8:(rank + 1) * 8])
    row = torch.nn.Module()
    m.create_weights(row, 256, [16], 512, 16, torch.float16)         # 256 of 512 input values per rank
    row.weight.weight_loader(row.weight, full)
    m.process_weights_after_loading(row)
    assert torch.equal(row.weight.data, full[:, rank * 144:(rank + 1) * 144])
    merged = torch.nn.Module()
    m.create_weights(merged, 512, [4, 4], 512, 16, torch.float16)    # gate / up, each 8 rows in the file
    for sid in (0, 1):
        merged.weight.weight_loader(merged.weight, full[sid * 8:(sid + 1) * 8], sid)
        merged.weight_type.weight_loader(merged.weight_type, torch.tensor(12), sid)
    m.process_weights_after_loading(merged)
    want = torch.cat([full[rank * 4:rank * 4 + 4], full[8 + rank * 4:8 + rank * 4 + 4]])
    assert torch.equal(merged.weight.data, want)


@pytest.mark.parametrize("size", [1, 2])
def test_moe_loader_honours_expert_and_shard_ids(recorded_ops, monkeypatch, size):
    _, linear = recorded_ops
    from vllm_gguf_plugin.quantization import fused_moe

    rank = size - 1
    monkeypatch.setattr(linear, "tensor_parallel_rank_and_size", lambda: (rank, size))
    E, I, H = 3, 8, 64                          # Q4_0: 18 bytes per 32 values -> rows of 36 (w13) / 18*I/32.. bytes
    w1 = torch.randint(0, 255, (E, I, 36), dtype=torch.uint8)
    w3 = torch.randint(0, 255, (E, I, 36), dtype=torch.uint8)
    w2 = torch.randint(0, 255, (E, H, 72), dtype=torch.uint8)
    layer = torch.nn.Module()
    meth = fused_moe.GGUFMoEMethod(None)
    meth.create_weights(layer, E, H, I // size, torch.float16, weight_loader=lambda *a, **k: None)
    # stacked tensors for w1 / w3, one expert at a time for w2
    layer.w13_weight.weight_loader(layer.w13_weight, w1, "experts.gate", shard_id="w1", expert_id=0)
    layer.w13_weight.weight_loader(layer.w13_weight, w3, "experts.up", shard_id="w3", expert_id=0)
    for e in range(E):
        assert layer.w2_weight.weight_loader(layer.w2_weight, w2[e], "experts.down", shard_id="w2", expert_id=e, return_success=True)
    n = I // size
    assert tuple(layer.w13_weight.shape) == (E, 2 * n, 36)
    assert torch.equal(layer.w13_weight.data[:, :n], w1[:, rank * n:(rank + 1) * n])
    assert torch.equal(layer.w13_weight.data[:, n:], w3[:, rank * n:(rank + 1) * n])
    b = 72 // size
    assert torch.equal(layer.w2_weight.data, w2[:, :, rank * b:(rank + 1) * b])
    layer.w13_weight_type.weight_loader(layer.w13_weight_type, torch.tensor(2), "x", shard_id="w1", expert_id=0)
    assert layer.w13_weight_type.weight_type == 2
