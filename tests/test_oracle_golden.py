"""CPU: the oracle against the committed golden fixtures (gguf-py outputs) and its own invariants."""
import re
import os
from pathlib import Path

import numpy as np
import pytest

from helpers import DEQUANT_ONLY_TYPES, REL_L2_TOL, ROOT, TYPES, rel_l2

from gguf_b200 import synth
from oracle import cpu

GOLD = np.load(Path(__file__).parent / "golden" / "golden_gguf_py.npz")


@pytest.mark.parametrize("name", list(TYPES) + list(DEQUANT_ONLY_TYPES))
def test_dequantize_matches_gguf_py_fixture(name):
    t = {**TYPES, **DEQUANT_ONLY_TYPES}[name]
    w, want = GOLD[f"w_{name}"], GOLD[f"dq_{name}"]
    n = want.size
    got32 = cpu.as_float(cpu.dequantize(w, t, n, "float32"), "float32").reshape(want.shape)
    if name in ("IQ2_XXS", "IQ4_XS", "IQ4_NL"):
        # fp32 decoders: the reference kernel and gguf-py do the same fp32 multiplies
        assert np.array_equal(got32, want)
    else:
        # half-arithmetic decoders round to fp16 where gguf-py keeps fp32: same tolerance as the
        # reference's own test (tests/test_kernels.py:99)
        np.testing.assert_allclose(got32, want, atol=1e-2, rtol=4e-2)
        assert rel_l2(got32, want) < 5e-4
    got16 = cpu.as_float(cpu.dequantize(w, t, n, "float16"), "float16").reshape(want.shape)
    np.testing.assert_allclose(got16, want, atol=1e-2, rtol=4e-2)
    gotbf = cpu.as_float(cpu.dequantize(w, t, n, "bfloat16"), "bfloat16").reshape(want.shape)
    np.testing.assert_allclose(gotbf, want, atol=1e-2, rtol=4e-2)


@pytest.mark.parametrize("name", TYPES)
def test_matmul_matches_cpu_route_fixture(name):
    """a8 results differ from the unquantized CPU route only by the q8_1 activation noise (~5e-3)."""
    t = TYPES[name]
    w, x, y = GOLD[f"w_{name}"], GOLD[f"x_{name}"], GOLD[f"y_{name}"]
    for mmq in (False, True):
        y64, out = cpu.matmul_a8(w, t, x, "float16", mmq=mmq)
        assert rel_l2(y64, y) < 2.5e-2
        assert rel_l2(cpu.as_float(out, "float16"), y64) < 1e-3
    dense = cpu.dense_matmul(GOLD[f"dq_{name}"], x, "float16")
    assert rel_l2(dense, y) < 1e-12


def test_q4k_tiled_formula_differs_from_gemv_formula():
    w = synth.make_weight(12, 16, 1024, seed=5)
    x = synth.make_activation(4, 1024, seed=5)
    a, _ = cpu.matmul_a8(w, 12, x, "float16", mmq=False)
    b, _ = cpu.matmul_a8(w, 12, x, "float16", mmq=True)
    r = rel_l2(a, b)
    assert 0 < r < REL_L2_TOL


def test_q4k_contraction_modes_differ_only_in_last_bit():
    w = synth.make_weight(12, 8, 1024, seed=6)
    a = cpu.dequantize(w, 12, 8 * 1024, "float16", q4k_contract=0).view(np.int16).astype(np.int32)
    b = cpu.dequantize(w, 12, 8 * 1024, "float16", q4k_contract=1).view(np.int16).astype(np.int32)
    assert (a != b).any()
    fa = cpu.as_float(a.astype(np.int16).view(np.uint16), "float16")
    fb = cpu.as_float(b.astype(np.int16).view(np.uint16), "float16")
    assert rel_l2(fa, fb) < 5e-4


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_q8_1_invariants(dtype):
    rng = np.random.default_rng(0)
    x32 = rng.standard_normal((5, 800)).astype(np.float32)
    x32[1] = 0.0                      # all-zero row: d = 0, q = 0
    x32[2, :32] = 3.0                 # all-equal block: q = 127 everywhere
    x = {"float32": x32, "float16": x32.astype(np.float16), "bfloat16": synth.to_bf16_bits(x32)}[dtype]
    xf = {"float32": x32, "float16": x32.astype(np.float16).astype(np.float32),
          "bfloat16": (synth.to_bf16_bits(x32).astype(np.uint32) << 16).view(np.float32)}[dtype]
    q = cpu.quantize_q8_1(x, dtype)
    kpad = 1024
    assert q.shape == (5, kpad // 32 * 36)
    blocks = q.reshape(5, kpad // 32, 36)
    d = blocks[:, :, 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    s = blocks[:, :, 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    qs = blocks[:, :, 4:].view(np.int8).astype(np.int32)
    xp = np.zeros((5, kpad), np.float32)
    xp[:, :800] = xf
    xb = xp.reshape(5, kpad // 32, 32)
    amax = np.abs(xb).max(axis=2)
    np.testing.assert_allclose(d, (amax / 127).astype(np.float16).astype(np.float32), rtol=1e-3, atol=1e-8)
    np.testing.assert_allclose(s, xb.sum(axis=2), rtol=2e-3, atol=2e-3)
    assert np.abs(qs).max() <= 127
    assert (qs[1] == 0).all() and (d[1] == 0).all()
    assert (qs[2, 0] == 127).all()
    assert (qs[:, 25:] == 0).all()    # zero padding beyond K = 800
    recon = qs * d[..., None]
    assert np.abs(recon - xb).max() <= (amax.max() / 127) * 0.51 + 1e-3


def test_moe_oracle_equals_per_slot_matmul():
    E, N, K, T, top_k, blk = 4, 32, 256, 10, 2, 4
    w = np.stack([synth.make_weight(2, N, K, seed=e) for e in range(E)])
    x = synth.make_activation(T, K, seed=3)
    _, ids = synth.make_routing(T, E, top_k, 0)
    s, e, n = synth.moe_align_block_size(ids, blk, E)
    y64, _ = cpu.moe_a8(w, 2, x, s, e, int(n[0]), blk, top_k, T)
    for tok in range(T):
        for j in range(top_k):
            ref, _ = cpu.matmul_a8(w[ids[tok, j]], 2, x[tok:tok + 1], "float16", mmq=True)
            assert np.allclose(y64[tok * top_k + j], ref[0], rtol=1e-12, atol=1e-12)
    yv, _ = cpu.moe_a8_vec(w, 2, x, ids, top_k, T)
    assert rel_l2(yv, y64) < 1e-12  # Q4_0: tiled and GEMV formulas coincide


def test_iq_tables_match_reference_header_when_present():
    from oracle import reference_root

    if reference_root() is None:
        pytest.skip("reference checkout absent")
    hdr = reference_root() / "vllm_gguf_plugin/csrc/gguf/ggml-common.h"
    import sys

    sys.path.insert(0, str(ROOT / "include"))
    from gen_iq_tables import more_tables, render, tables

    src = hdr.read_text()

    def arr(name):
        m = re.search(name + r"\[[^\]]*\]\s*=\s*\{(.*?)\};", src, re.S)
        return [int(v, 0) for v in re.findall(r"-?0x[0-9a-fA-F]+|-?\d+", m.group(1))]

    grid, ksigns, kvalues = tables()
    assert arr("iq2xxs_grid") == grid and arr("ksigns_iq2xs") == ksigns and arr("kvalues_iq4nl") == kvalues
    iq2xs, iq2s, iq3xxs, iq3s, iq1s = more_tables()
    assert arr("iq2xs_grid") == iq2xs and arr("iq2s_grid") == iq2s
    assert arr("iq3xxs_grid") == iq3xxs and arr("iq3xs_grid") == iq3s   # (the IQ3_S code book is called iq3xs_grid there)
    assert arr("iq1s_grid_gpu") == iq1s
    assert (ROOT / "include" / "gguf_b200_iq_tables.h").read_text() == render()
