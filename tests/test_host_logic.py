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
    assert len(ROUTING) == 288
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
