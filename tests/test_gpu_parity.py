"""GPU parity tests: every kernel through the C-ABI (gguf_b200.capi -> libgguf_b200.so)
against the CPU oracle, and -- when oracle/_ref/_C_gguf_ref.so was built -- against the
reference plugin's own CUDA kernels on the same inputs.

Bars: dequantize and q8_1 quantization bit-exact; matmul outputs within relative L2 2e-3
(REL_L2_TOL) of the reference kernel of the same entry point."""
import numpy as np
import pytest
import torch

from helpers import DEQUANT_ONLY_TYPES, MMQ_TYPES, REL_L2_TOL, TYPES, RefCuda, bits, np_act, rel_l2

from gguf_b200 import capi, synth
from oracle import cpu

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ref(native_libs):
    return RefCuda()


def dev_w(t, n, k, seed):
    w = synth.make_weight(t, n, k, seed=seed)
    return w, torch.from_numpy(w).to(DEV)


def dev_x(m, k, seed, dtype=torch.float16):
    x = torch.from_numpy(synth.make_activation(m, k, seed=seed, dtype=np.float32)).to(DEV).to(dtype)
    return x


# ---------------------------------------------------------------- q8_1 quantization ----------

@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 1024), (3, 4096), (7, 800), (64, 14336)])
def test_quantize_q8_1_bit_exact(ref, dtype, shape):
    M, K = shape
    x = dev_x(M, K, seed=M, dtype=dtype)
    if M >= 3:
        x[1] = 0                    # all-zero blocks
        x[2, :64] = 1.5             # all-equal blocks
    got = capi.quantize_q8_1(x)
    torch.cuda.synchronize()
    if ref.available:
        assert torch.equal(got, ref.quantize_q8_1(x)), "differs from the reference kernel"
    # CPU oracle: IEEE division where the GPU build uses the fast-math approximation, so codes may
    # differ by one step at exact ties and d by one fp16 ulp; anything else is a bug.
    xa, dn = np_act(x)
    want = cpu.quantize_q8_1(xa, dn).reshape(M, -1, 36)
    g = got.cpu().numpy().reshape(M, -1, 36)
    dq = g[..., 4:].view(np.int8).astype(np.int32) - want[..., 4:].view(np.int8).astype(np.int32)
    assert np.abs(dq).max() <= 1
    assert (dq != 0).mean() < 2e-3
    dd = g[..., 0:2].copy().view(np.int16).astype(np.int32) - want[..., 0:2].copy().view(np.int16).astype(np.int32)
    assert np.abs(dd).max() <= 1
    assert np.array_equal(g[..., 2:4], want[..., 2:4]), "block sums must match exactly (same butterfly order)"


# ---------------------------------------------------------------- dequantize -----------------

@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("name", TYPES)
def test_dequantize_bit_exact(ref, name, dtype):
    t = TYPES[name]
    N, K = 96, 2048
    wn, w = dev_w(t, N, K, seed=t)
    got = capi.dequantize(w, t, N, K, dtype)
    torch.cuda.synchronize()
    dn = str(dtype).split(".")[1]
    want = cpu.dequantize(wn, t, N * K, dn)
    want_t = torch.from_numpy(want.view(np.int32) if dn == "float32" else want.view(np.int16)).reshape(N, K)
    assert torch.equal(bits(got).cpu(), want_t), "differs from the CPU oracle"
    if ref.available:
        r = ref.ops.ggml_dequantize(w, t, N, K, dtype)
        assert torch.equal(bits(got), bits(r)), "differs from the reference kernel"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("name", DEQUANT_ONLY_TYPES)
def test_dequantize_more_types_bit_exact(ref, name, dtype):
    """Block types that only the standalone dequantize serves."""
    t = DEQUANT_ONLY_TYPES[name]
    N, K = 40, 2048
    wn, w = dev_w(t, N, K, seed=t)
    got = capi.dequantize(w, t, N, K, dtype)
    torch.cuda.synchronize()
    dn = str(dtype).split(".")[1]
    want = cpu.dequantize(wn, t, N * K, dn)
    want_t = torch.from_numpy(want.view(np.int32) if dn == "float32" else want.view(np.int16)).reshape(N, K)
    assert torch.equal(bits(got).cpu(), want_t), "differs from the CPU oracle"
    if ref.available:
        r = ref.ops.ggml_dequantize(w, t, N, K, dtype)
        assert torch.equal(bits(got), bits(r)), "differs from the reference kernel"


def test_dequantize_full_matrices_bit_exact_on_device(ref):
    """One full benchmark matrix per type, compared on the device with the reference kernel."""
    if not ref.available:
        pytest.skip("reference kernels not built")
    for name, (N, K) in {"Q4_K": (14336, 4096), "Q6_K": (37888, 3584), "IQ4_XS": (37888, 3584), "IQ2_XXS": (28672, 8192),
                         "Q8_0": (3072, 1024), "Q4_0": (2048, 2048)}.items():
        t = TYPES[name]
        w = torch.from_numpy(synth.make_weight(t, N, K, seed=7)).to(DEV)
        got = capi.dequantize(w, t, N, K, torch.float16)
        want = ref.ops.ggml_dequantize(w, t, N, K, torch.float16)
        assert torch.equal(bits(got), bits(want)), name
        del w, got, want
        torch.cuda.empty_cache()


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K", "Q8_0", "IQ2_XXS", "Q5_K", "Q3_K", "IQ4_NL", "IQ3_S", "IQ1_M"])
def test_embedding_row_gather_equals_index_select_then_dequantize(ref, name):
    """The embedding caller: rows picked inside the dequantize kernel, bit for bit what the
    reference's two steps (index_select, ggml_dequantize) give; an id outside the table gives zeros."""
    from vllm_gguf_plugin.quantization import vocal_embeds

    t = {**TYPES, **DEQUANT_ONLY_TYPES}[name]
    V, H = 300, 1024
    wn, w = dev_w(t, V, H, seed=3)
    ids = torch.tensor([[5, 299, 0], [17, 17, 123]], device=DEV)
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        got = vocal_embeds._apply_gguf_embedding(ids, w, t, H, dtype)
        assert got.shape == (2, 3, H) and got.dtype == dtype
        quant = torch.index_select(w, 0, ids.flatten())
        want = capi.dequantize(quant, t, ids.numel(), H, dtype)
        assert torch.equal(bits(got.view(-1, H)), bits(want))
        if ref.available:
            r = ref.ops.ggml_dequantize(quant, t, H, ids.numel(), dtype)
            assert torch.equal(bits(got.view(-1, H)), bits(r.view(-1, H)))
    bad = capi.dequantize_rows(w, torch.tensor([1, V + 5, -1], device=DEV), t)
    assert torch.equal(bad[0], capi.dequantize(w[1:2].clone(), t, 1, H)[0]) and float(bad[1:].abs().sum()) == 0.0


def test_dequantize_ragged_counts(ref):
    """Element counts that are not a multiple of the 256-value warp step (32-value blocks)."""
    for name in ("Q4_0", "Q8_0"):
        t = TYPES[name]
        wn, w = dev_w(t, 1, 32 * 11, seed=3)
        got = capi.dequantize(w, t, 1, 32 * 11, torch.float16)
        want = cpu.dequantize(wn, t, 32 * 11, "float16")
        assert np.array_equal(got.cpu().numpy().view(np.uint16).reshape(-1), want)
    with pytest.raises(capi.GgufB200Error):
        capi.dequantize(w, 12, 1, 100, torch.float16)


def test_q4k_contraction_knob_selects_oracle_mode():
    wn, w = dev_w(12, 16, 1024, seed=9)
    try:
        for mode in (0, 1):
            capi.lib().gguf_b200_set_q4k_contract(mode)
            got = capi.dequantize(w, 12, 16, 1024, torch.float16).cpu().numpy().view(np.uint16).reshape(-1)
            assert np.array_equal(got, cpu.dequantize(wn, 12, 16 * 1024, "float16", q4k_contract=mode))
    finally:
        capi.lib().gguf_b200_set_q4k_contract(1)


# ---------------------------------------------------------------- GEMV -----------------------

GEMV_SHAPES = [(3072, 1024, 1), (520, 4096, 1), (257, 2048, 3), (128, 14336, 2), (1001, 4096, 2), (300, 1024, 2), (96, 28672, 1), (64, 3584, 8), (40, 4096, 11),
               # K whose blocks do not divide evenly into the K-slices of the two-vector kernel
               (300, 8960, 2), (70, 8448, 2), (33, 12544, 2), (50, 10752, 1), (7, 18944, 1), (5000, 512, 1)]


@pytest.mark.parametrize("shape", GEMV_SHAPES)
@pytest.mark.parametrize("name", TYPES)
def test_gemv_parity(ref, name, shape):
    t = TYPES[name]
    N, K, M = shape
    if K % synth.QUANT_SIZES[t][0]:
        pytest.skip("K not a multiple of the block size")
    wn, w = dev_w(t, N, K, seed=t + N)
    x = dev_x(M, K, seed=M)
    y = capi.mul_mat_vec_a8(w, x, t, N)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    if ref.available:
        r = ref.ops.ggml_mul_mat_vec_a8(w, x, t, N)
        assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL
        assert rel_l2(y.float().cpu(), r.float().cpu()) <= 1e-4   # in practice: same formulas, fp32 noise
    if N * K * M <= 16e6:
        y64, _ = cpu.matmul_a8(wn, t, x.cpu().numpy(), "float16", mmq=False)
        assert rel_l2(y.float().cpu().numpy(), y64) <= 1e-3       # fp16 output rounding + rare q8_1 tie flips


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemv_other_dtypes(ref, dtype):
    for name in ("Q4_K", "IQ2_XXS", "Q6_K"):
        t = TYPES[name]
        wn, w = dev_w(t, 300, 2048, seed=1)
        x = dev_x(2, 2048, seed=2, dtype=dtype)
        y = capi.mul_mat_vec_a8(w, x, t, 300)
        assert y.dtype == dtype
        xa, dn = np_act(x)
        y64, _ = cpu.matmul_a8(wn, t, xa, dn, mmq=False)
        tol = 1e-5 if dtype == torch.float32 else 5e-3
        # a q8_1 tie flip (fast-math division) moves one product term: allow it in the fp32 case
        assert rel_l2(y.float().cpu().numpy(), y64) <= max(tol, 2e-4)
        if ref.available:
            r = ref.ops.ggml_mul_mat_vec_a8(w, x, t, 300)
            assert rel_l2(y.float().cpu(), r.float().cpu()) <= (1e-5 if dtype == torch.float32 else REL_L2_TOL)


def test_gemv_empty_and_prepared_split():
    t = 12
    wn, w = dev_w(t, 64, 1024, seed=4)
    assert capi.mul_mat_vec_a8(w, torch.empty((0, 1024), dtype=torch.float16, device=DEV), t, 64).shape == (0, 64)
    x = dev_x(2, 1024, seed=4)
    ws = capi.gemv_prepare(x, t)
    a = capi.gemv_prepared(w, ws, t, 2, 64, 1024)
    b = capi.mul_mat_vec_a8(w, x, t, 64)
    assert torch.equal(a, b)


def test_gemv_is_deterministic_and_linear_at_full_size():
    """Full benchmark size (Q4_K 14336x4096): run twice -> identical bits; scaling the weight
    scales d by 2 (exact in fp16) must scale the output by exactly 2."""
    t, N, K = 12, 14336, 4096
    wn = synth.make_weight(t, N, K, seed=0)
    w = torch.from_numpy(wn).to(DEV)
    x = dev_x(1, K, seed=0, dtype=torch.float32)
    y1 = capi.mul_mat_vec_a8(w, x, t, N)
    y2 = capi.mul_mat_vec_a8(w, x, t, N)
    assert torch.equal(y1, y2)
    blocks = wn.reshape(-1, 144).copy()
    d = blocks[:, 0:4].copy().view(np.float16) * np.float16(2)
    blocks[:, 0:4] = d.view(np.uint8)
    y3 = capi.mul_mat_vec_a8(torch.from_numpy(blocks.reshape(N, -1)).to(DEV), x, t, N)
    assert torch.equal(y3, 2 * y1)


# ---------------------------------------------------------------- tensor-core GEMM -----------

MMQ_SHAPES = [(256, 1024, 16), (1000, 2048, 7), (384, 4096, 83), (512, 2048, 130), (300, 1024, 512), (128, 14336, 33)]


@pytest.mark.parametrize("shape", MMQ_SHAPES)
@pytest.mark.parametrize("name", MMQ_TYPES)
def test_mmq_parity(ref, name, shape):
    t = TYPES[name]
    N, K, M = shape
    wn, w = dev_w(t, N, K, seed=t + M)
    x = dev_x(M, K, seed=M)
    y = capi.mul_mat_a8(w, x, t, N)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert not torch.isnan(y).any()
    if ref.available:
        r = ref.ops.ggml_mul_mat_a8(w, x, t, N)
        assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL
    if N * K * M <= 2.2e8:
        y64, _ = cpu.matmul_a8(wn, t, x.cpu().numpy(), "float16", mmq=True)
        assert rel_l2(y.float().cpu().numpy(), y64) <= REL_L2_TOL


def test_mmq_block_multiple_of_32_but_not_64():
    """K = 32 * odd: the last 64-wide contraction slab is half padding."""
    for name in ("Q4_0", "Q8_0"):
        t = TYPES[name]
        wn, w = dev_w(t, 130, 32 * 37, seed=2)
        x = dev_x(20, 32 * 37, seed=2)
        y = capi.mul_mat_a8(w, x, t, 130)
        y64, _ = cpu.matmul_a8(wn, t, x.cpu().numpy(), "float16", mmq=True)
        assert rel_l2(y.float().cpu().numpy(), y64) <= REL_L2_TOL


@pytest.mark.parametrize("N", [264, 260])
@pytest.mark.parametrize("name", ["Q6_K", "Q3_K", "Q2_K", "Q5_0", "IQ2_XXS"])
def test_mmq_rows_of_every_alignment(ref, name, N):
    """K = 768: rows of 630 / 330 / 252 / 528 / 198 bytes, i.e. eight (or four, or one) alignment classes of rows.
    N = 264 is a multiple of eight (one TMA box per class), N = 260 is not (one bulk copy per row)."""
    t = TYPES[name]
    K, M = 768, 40
    wn, w = dev_w(t, N, K, seed=N)
    x = dev_x(M, K, seed=3)
    if name == "IQ2_XXS":
        y = capi.dequant_matmul(w, x, t, N)
        want = (x @ capi.dequantize(w, t, N, K, torch.float16).T).float().cpu().numpy()
    else:
        y = capi.mul_mat_a8(w, x, t, N)
        want, _ = cpu.matmul_a8(wn, t, x.cpu().numpy(), "float16", mmq=True)
        if ref.available:
            r = ref.ops.ggml_mul_mat_a8(w, x, t, N)
            assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert rel_l2(y.float().cpu().numpy(), want) <= REL_L2_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mmq_other_dtypes(dtype):
    t = 12
    wn, w = dev_w(t, 200, 1024, seed=8)
    x = dev_x(40, 1024, seed=8, dtype=dtype)
    y = capi.mul_mat_a8(w, x, t, 200)
    assert y.dtype == dtype
    xa, dn = np_act(x)
    y64, _ = cpu.matmul_a8(wn, t, xa, dn, mmq=True)
    assert rel_l2(y.float().cpu().numpy(), y64) <= (REL_L2_TOL if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("name", ["IQ2_XXS", "IQ4_XS", "IQ4_NL"])
def test_dequant_matmul_parity(ref, name, dtype):
    """IQ types above the GEMV threshold: the reference dequantizes and calls a dense matmul."""
    t = TYPES[name]
    for (N, K, M) in [(256, 1024, 16), (1000, 2048, 40), (384, 4096, 128), (264, 2048, 300)]:   # the last: 256-token tiles
        wn, w = dev_w(t, N, K, seed=N)
        x = dev_x(M, K, seed=M, dtype=dtype)
        y = capi.dequant_matmul(w, x, t, N)
        torch.cuda.synchronize()
        assert capi.last_status() == 0
        wd = capi.dequantize(w, t, N, K, dtype)
        want = x @ wd.T                                    # the reference's second step
        assert rel_l2(y.float().cpu(), want.float().cpu()) <= REL_L2_TOL
        if ref.available:
            r = x @ ref.ops.ggml_dequantize(w, t, N, K, dtype).T
            assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL
        dq = cpu.as_float(cpu.dequantize(wn, t, N * K, "float32"), "float32").reshape(N, K)
        xa, dn = np_act(x)
        y64 = cpu.dense_matmul(dq, xa, dn)
        assert rel_l2(y.float().cpu().numpy(), y64) <= (REL_L2_TOL if dtype == torch.float16 else 6e-3)


# ---------------------------------------------------------------- MoE ------------------------

def moe_case(t, E, N, K, T, top_k, seed):
    w = np.stack([synth.make_weight(t, N, K, seed=seed + e) for e in range(E)])
    x = synth.make_activation(T, K, seed=seed)
    tw, ids = synth.make_routing(T, E, top_k, seed)
    return w, x, tw, ids


@pytest.mark.parametrize("name", ["Q4_0", "Q4_K", "Q8_0", "Q2_K", "Q3_K"])
def test_moe_a8_parity(ref, name):
    t = TYPES[name]
    E, N, K, T, top_k = 8, 192, 1024, 70, 2
    wn, xn, _, ids = moe_case(t, E, N, K, T, top_k, seed=11)
    w, x = torch.from_numpy(wn).to(DEV), torch.from_numpy(xn).to(DEV)
    blk = capi.lib().gguf_b200_moe_block_size(t)
    s, e, n = synth.moe_align_block_size(ids, blk, E)
    y = capi.moe_a8(x, w, torch.from_numpy(s).to(DEV), torch.from_numpy(e).to(DEV), torch.from_numpy(n).to(DEV), t, N, top_k, T)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    y64, _ = cpu.moe_a8(wn, t, xn, s, e, int(n[0]), blk, top_k, T)
    assert rel_l2(y.float().cpu().numpy(), y64) <= REL_L2_TOL
    if ref.available:
        s4, e4, n4 = synth.moe_align_block_size(ids, 4, E)   # the reference's own block size
        r = ref.ops.ggml_moe_a8(x, w, torch.from_numpy(s4).to(DEV), torch.from_numpy(e4).to(DEV),
                                torch.from_numpy(n4).to(DEV), t, N, top_k, T)
        assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL


@pytest.mark.parametrize("name", ["Q6_K", "Q3_K"])
def test_moe_a8_whole_row_tiles_of_unaligned_rows(name):
    """N a multiple of 128 with rows that are not a multiple of 16 bytes: the experts' raw weights arrive as
    alignment-class TMA boxes over the stacked [E * N] rows."""
    t = TYPES[name]
    E, N, K, T, top_k = 6, 256, 1024, 50, 2
    wn, xn, _, ids = moe_case(t, E, N, K, T, top_k, seed=17)
    w, x = torch.from_numpy(wn).to(DEV), torch.from_numpy(xn).to(DEV)
    blk = capi.lib().gguf_b200_moe_block_size(t)
    s, e, n = synth.moe_align_block_size(ids, blk, E)
    y = capi.moe_a8(x, w, torch.from_numpy(s).to(DEV), torch.from_numpy(e).to(DEV), torch.from_numpy(n).to(DEV), t, N, top_k, T)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    y64, _ = cpu.moe_a8(wn, t, xn, s, e, int(n[0]), blk, top_k, T)
    assert rel_l2(y.float().cpu().numpy(), y64) <= REL_L2_TOL


def test_moe_a8_padding_rows_are_zero_and_bad_experts_skipped():
    t, E, N, K, T, top_k = 2, 4, 128, 512, 20, 2
    wn, xn, _, ids = moe_case(t, E, N, K, T, top_k, seed=5)
    w, x = torch.from_numpy(wn).to(DEV), torch.from_numpy(xn).to(DEV)
    blk = capi.lib().gguf_b200_moe_block_size(t)
    s, e, n = synth.moe_align_block_size(ids, blk, E)
    e_bad = e.copy()
    e_bad[0] = 300                                           # expert id outside [0, 255]: block skipped
    y = capi.moe_a8(x, w, torch.from_numpy(s).to(DEV), torch.from_numpy(e_bad).to(DEV), torch.from_numpy(n).to(DEV), t, N, top_k, T)
    y64, _ = cpu.moe_a8(wn, t, xn, s, e_bad, int(n[0]), blk, top_k, T)
    assert rel_l2(y.float().cpu().numpy(), y64) <= REL_L2_TOL
    skipped = s[:blk][s[:blk] < T * top_k]
    assert float(y[torch.from_numpy(skipped).long().to(DEV)].abs().sum()) == 0.0


@pytest.mark.parametrize("name", ["Q4_0", "Q6_K", "IQ4_XS"])
def test_moe_a8_vec_parity(ref, name):
    t = TYPES[name]
    E, N, K, T, top_k = 8, 160, 1024, 6, 3
    wn, xn, _, ids = moe_case(t, E, N, K, T, top_k, seed=21)
    w, x = torch.from_numpy(wn).to(DEV), torch.from_numpy(xn).to(DEV)
    idt = torch.from_numpy(ids).to(DEV).contiguous()
    y = capi.moe_a8_vec(x, w, idt, top_k, t, N, T)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    y64, _ = cpu.moe_a8_vec(wn, t, xn, ids, top_k, T)
    assert rel_l2(y.float().cpu().numpy(), y64) <= 1e-3
    if ref.available:
        r = ref.ops.ggml_moe_a8_vec(x, w, idt, top_k, t, N, T)
        assert rel_l2(y.float().cpu(), r.float().cpu()) <= 1e-4


# ---------------------------------------------------------------- operator API (torch library) --

def test_ops_api_equals_capi_and_dispatcher_end_to_end():
    from vllm_gguf_plugin import ops
    from vllm_gguf_plugin.quantization import linear

    for name, t in TYPES.items():
        wn, w = dev_w(t, 256, 1024, seed=t)
        x1, x64 = dev_x(1, 1024, seed=1), dev_x(64, 1024, seed=2)
        assert torch.equal(ops.ggml_mul_mat_vec_a8(w, x1, t, 256), capi.mul_mat_vec_a8(w, x1, t, 256))
        assert torch.equal(ops.ggml_dequantize(w, t, 256, 1024, torch.float16), capi.dequantize(w, t, 256, 1024))
        y = linear._fused_mul_mat_gguf(x64, w, t)
        if name in MMQ_TYPES:
            want = capi.mul_mat_a8(w, x64, t, 256)
        elif t in ops._DEQUANT_MATMUL_TYPES:
            want = capi.dequant_matmul(w, x64, t, 256)
        else:   # code-book types with a GEMV only: the reference's two steps (linear.py:50-54)
            want = x64 @ capi.dequantize(w, t, 256, 1024).T
        assert torch.equal(y, want)
    with pytest.raises(NotImplementedError):
        ops.ggml_mul_mat_vec_a8(w, x1, 9, 256)
    with pytest.raises(RuntimeError):
        ops.ggml_mul_mat_vec_a8(w[:, :-1].contiguous(), x1, 23, 256)      # not a whole number of blocks


def test_fused_moe_dispatcher_matches_dense_experts():
    from vllm_gguf_plugin.quantization import fused_moe

    t, E, H, I, T, top_k = 2, 8, 512, 256, 96, 2
    w13n = np.stack([synth.make_weight(t, 2 * I, H, seed=e) for e in range(E)])
    w2n = np.stack([synth.make_weight(t, H, I, seed=100 + e) for e in range(E)])
    x = dev_x(T, H, seed=3)
    tw, ids = synth.make_routing(T, E, top_k, 3)
    w13, w2 = torch.from_numpy(w13n).to(DEV), torch.from_numpy(w2n).to(DEV)
    out = fused_moe._fused_moe_gguf(x, w13, w2, torch.from_numpy(tw).to(DEV), torch.from_numpy(ids).to(DEV).int(), t, t, "silu")
    # dense restatement on dequantized weights (what the reference's test_moe compares with)
    d13 = torch.stack([capi.dequantize(w13[e], t, 2 * I, H) for e in range(E)]).float()
    d2 = torch.stack([capi.dequantize(w2[e], t, H, I) for e in range(E)]).float()
    want = torch.zeros(T, H, device=DEV)
    for tok in range(T):
        for j in range(top_k):
            e = int(ids[tok, j])
            h = x[tok].float() @ d13[e].T
            h = torch.nn.functional.silu(h[:I]) * h[I:]
            want[tok] += float(tw[tok, j]) * (h @ d2[e].T)
    # activations are q8_1-quantized twice on the kernel path: the reference's own tolerance class
    assert rel_l2(out.float().cpu(), want.cpu()) < 3e-2


def _reference_moe_sequence(ref, x, w13, w2, tw, ids, t13, t2):
    """The reference's tiled MoE branch (quantization/fused_moe.py:56-95) restated with the
    reference's own kernels: block-4 alignment, ggml_moe_a8, silu-and-mul in the activation type
    (silu rounded, then multiplied), ggml_moe_a8, routing weights, sum over top_k."""
    T, top_k = ids.shape
    E, N2, _ = w13.shape
    H = w2.shape[1]
    s4, e4, n4 = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(ids.cpu().numpy(), 4, E)]
    out = ref.ops.ggml_moe_a8(x, w13, s4, e4, n4, t13, N2, top_k, T)
    g, u = out[:, :N2 // 2].float(), out[:, N2 // 2:]
    act = (g / (1.0 + torch.exp(-g))).to(out.dtype) * u
    out = ref.ops.ggml_moe_a8(act.contiguous(), w2, s4, e4, n4, t2, H, 1, T * top_k)
    out = (out.view(T, top_k, H).float() * tw.view(T, top_k, 1).float()).to(x.dtype)
    return out.float().sum(dim=1).to(x.dtype)


# (name, gate/up type, down type, experts, H, I, tokens, top_k, activation scale: the synthetic K-quant
#  weights have a large scale, and silu(gate) * up has to stay inside fp16 as it does in a real model)
@pytest.mark.parametrize("case", [("Q4_0", 2, 2, 8, 512, 256, 96, 2, 1.0), ("Q4_K", 12, 14, 6, 1024, 512, 70, 3, 1 / 64), ("Q8_0", 8, 8, 4, 256, 256, 130, 1, 1.0),
                                  ("Q5_K", 13, 6, 5, 512, 256, 80, 2, 1 / 128)])
def test_fused_moe_step_matches_reference_sequence(ref, case):
    """gguf_b200_fused_moe (alignment + GEMM + activation-in-quantizer + GEMM with routing weights in
    the epilogue + sum) against the reference's sequence of separate ops on its own kernels."""
    name, t13, t2, E, H, I, T, top_k, x_scale = case
    w13 = torch.from_numpy(np.stack([synth.make_weight(t13, 2 * I, H, seed=e) for e in range(E)])).to(DEV)
    w2 = torch.from_numpy(np.stack([synth.make_weight(t2, H, I, seed=100 + e) for e in range(E)])).to(DEV)
    x = (dev_x(T, H, seed=3).float() * x_scale).half()
    twn, idn = synth.make_routing(T, E, top_k, 3)
    tw, ids = torch.from_numpy(twn).to(DEV), torch.from_numpy(idn).to(DEV)
    got = capi.fused_moe(x, w13, w2, ids, tw, t13, t2)
    torch.cuda.synchronize()
    assert capi.last_status() == 0 and bool(torch.isfinite(got).all())
    # the same library, op by op (separate alignment, activation, weighting and sum)
    blk = capi.lib().gguf_b200_moe_block_size(t13)
    s, e, n = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(idn, blk, E)]
    o1 = capi.moe_a8(x, w13, s, e, n, t13, 2 * I, top_k, T)
    a1 = (torch.nn.functional.silu(o1[:, :I].float()).half() * o1[:, I:]).contiguous()
    o2 = capi.moe_a8(a1, w2, s, e, n, t2, H, 1, T * top_k)
    stepwise = (o2.view(T, top_k, H).float() * tw.view(T, top_k, 1)).half().float().sum(1).half()
    assert rel_l2(got.float().cpu(), stepwise.float().cpu()) <= 5e-4
    if ref.available:
        # End to end the two pipelines cannot agree to the single-op tolerance: the second GEMM
        # re-quantizes the first one's output to q8_1, and a 4e-4 difference in that output (fp16
        # operands here, integer dot products there) flips a few per cent of the int8 codes, each
        # worth 1/127 of its block's range.  Every stage on IDENTICAL inputs stays within 2e-3
        # (test_moe_a8_parity, test_moe_full_size_close_to_reference and the check below, which feeds
        # the reference's own first-stage output to this library's second stage).
        want = _reference_moe_sequence(ref, x, w13, w2, tw, ids, t13, t2)
        assert rel_l2(got.float().cpu(), want.float().cpu()) <= 1e-2
        s4, e4, n4 = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(idn, 4, E)]
        r1 = ref.ops.ggml_moe_a8(x, w13, s4, e4, n4, t13, 2 * I, top_k, T)
        ra = ((r1[:, :I].float() / (1.0 + torch.exp(-r1[:, :I].float()))).half() * r1[:, I:]).contiguous()
        ours2 = capi.moe_a8(ra, w2, s, e, n, t2, H, 1, T * top_k)
        ref2 = ref.ops.ggml_moe_a8(ra, w2, s4, e4, n4, t2, H, 1, T * top_k)
        assert rel_l2(ours2.float().cpu(), ref2.float().cpu()) <= REL_L2_TOL
    # a slot routed to "no expert" (id -1, as expert-parallel masking does) contributes nothing
    ids2 = ids.clone()
    ids2[0, 0] = -1
    got2 = capi.fused_moe(x, w13, w2, ids2, tw, t13, t2)
    tw2 = tw.clone()
    tw2[0, 0] = 0.0
    want2 = capi.fused_moe(x, w13, w2, ids, tw2, t13, t2)
    assert rel_l2(got2.float().cpu(), want2.float().cpu()) <= 1e-3
    assert torch.equal(got2[1:], want2[1:])


def test_fused_moe_dispatcher_uses_the_fused_step(ref):
    """_fused_moe_gguf above 64 tokens = the fused call; gelu as well; bf16 activations."""
    from vllm_gguf_plugin.quantization import fused_moe

    t, E, H, I, T, top_k = 2, 8, 512, 256, 96, 2
    w13 = torch.from_numpy(np.stack([synth.make_weight(t, 2 * I, H, seed=e) for e in range(E)])).to(DEV)
    w2 = torch.from_numpy(np.stack([synth.make_weight(t, H, I, seed=100 + e) for e in range(E)])).to(DEV)
    twn, idn = synth.make_routing(T, E, top_k, 3)
    tw, ids = torch.from_numpy(twn).to(DEV), torch.from_numpy(idn).to(DEV).int()
    for dtype in (torch.float16, torch.bfloat16):
        x = dev_x(T, H, seed=3, dtype=dtype)
        for act, code in (("silu", capi.ACT_SILU), ("gelu", capi.ACT_GELU)):
            out = fused_moe._fused_moe_gguf(x, w13, w2, tw, ids, t, t, act)
            assert torch.equal(out, capi.fused_moe(x, w13, w2, ids, tw, t, t, code))
            assert out.dtype == dtype and bool(torch.isfinite(out).all())


def test_fused_moe_full_size_matches_reference_sequence(ref):
    """The MoE benchmark configuration end to end: 64 experts, top-8, hidden 2048, intermediate 1024, Q4_0, 256 tokens."""
    if not ref.available:
        pytest.skip("reference kernels not built")
    t, E, top_k, H, I, T = 2, 64, 8, 2048, 1024, 256
    w13 = torch.from_numpy(np.stack([synth.make_weight(t, 2 * I, H, seed=100 + e) for e in range(E)])).to(DEV)
    w2 = torch.from_numpy(np.stack([synth.make_weight(t, H, I, seed=300 + e) for e in range(E)])).to(DEV)
    x = torch.from_numpy(synth.make_activation(T, H, seed=1)).to(DEV)
    twn, idn = synth.make_routing(T, E, top_k, 0)
    tw, ids = torch.from_numpy(twn).to(DEV), torch.from_numpy(idn).to(DEV)
    got = capi.fused_moe(x, w13, w2, ids, tw, t, t)
    want = _reference_moe_sequence(ref, x, w13, w2, tw, ids, t, t)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    # (two chained q8_1 quantizations: see test_fused_moe_step_matches_reference_sequence)
    assert rel_l2(got.float().cpu(), want.float().cpu()) <= 1e-2


# ---------------------------------------------------------------- fused gather (tensor parallel) --
# Two ranks emulated on ONE GPU, one after the other on one stream, so nothing ever waits on a
# kernel that has not been launched.  The real 2/4/8-GPU runs are in tests/test_tp_multi_gpu.py.

@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("name", ["Q4_K", "Q8_0", "IQ4_XS", "IQ2_XXS"])
def test_tp_gemv_packets_one_gpu(name, dtype):
    """Each rank sends its row slice as tagged packets into both packet arenas; unpacking either
    arena gives the unsharded GEMV bit for bit.  A second call whose activations are
    x + s * (vector gathered by the first) reads the packets in its own quantizer."""
    t = TYPES[name]
    N, K, world = 2048, 1024, 2
    wn, w = dev_w(t, N, K, seed=5)
    x = dev_x(1, K, seed=5, dtype=dtype)
    want = capi.mul_mat_vec_a8(w, x, t, N)
    psz = 8 if dtype == torch.float32 else 4
    slots, slot_packets = 4, 2048
    arenas = [torch.zeros(slots * slot_packets * psz, dtype=torch.uint8, device=DEV) for _ in range(world)]
    epochs = [torch.zeros(slots, dtype=torch.int32, device=DEV) for _ in range(world)]
    ptrs = [a.data_ptr() for a in arenas]
    shards = [w[r * N // world:(r + 1) * N // world].contiguous() for r in range(world)]
    for rep in range(3):   # later rounds find the previous round's packets in place: only the tag tells them apart
        for r in range(world):
            capi.mul_mat_vec_a8_tp(shards[r], x, ptrs, epochs[r], 1, slot_packets, t, r)
        for r in range(world):
            got = capi.tp_unpack(arenas[r], epochs[r], 1, 1, slot_packets, N, dtype)
            assert torch.equal(got, want)
            assert int(epochs[r][1]) == rep + 1
    # chained call: x2 = x + s * y(slot 1)[:K], rounded to the activation type, into slot 2
    s = 2.0 ** -9
    x2 = (x.float() + s * want[:, :K].float()).to(dtype)
    want2 = capi.mul_mat_vec_a8(w, x2, t, N)
    for r in range(world):
        capi.mul_mat_vec_a8_tp(shards[r], x, ptrs, epochs[r], 2, slot_packets, t, r, add_slot=1, add_scale=s)
    for r in range(world):
        assert torch.equal(capi.tp_unpack(arenas[r], epochs[r], 2, 1, slot_packets, N, dtype), want2)
    # both slots at once
    both = capi.tp_unpack(arenas[0], epochs[0], 1, 2, slot_packets, N, dtype)
    assert torch.equal(both[0:1], want) and torch.equal(both[1:2], want2)
    torch.cuda.synchronize()
    assert capi.last_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("name", ["Q4_K", "Q8_0", "Q6_K", "IQ2_XXS"])
def test_tp_gemv_row_parallel_one_gpu(ref, name, dtype):
    """K-sharded decode, two emulated ranks: each sends the fp32 partial sums over its half of K to
    both arenas; their sum in rank order is the all-reduced vector -- the same bits on both ranks,
    equal to 'partial GEMVs in fp32, added, rounded once', and close to the unsharded GEMV and to
    the reference kernel.  A column-parallel call then consumes the reduced vector in its quantizer,
    and a row-parallel call consumes a gathered one (the two pairings of a tensor-parallel MLP)."""
    t = TYPES[name]
    N, K, world = 1024, 4096, 2
    wn, w = dev_w(t, N, K, seed=11)
    x = dev_x(1, K, seed=11, dtype=dtype)
    from gguf_b200 import tp as tpmod

    wk = [tpmod.shard_cols(w, t, r, world) for r in range(world)]
    xk = [x[:, r * K // world:(r + 1) * K // world].contiguous() for r in range(world)]
    parts = [capi.mul_mat_vec_a8(wk[r], xk[r].float(), t, N) for r in range(world)]      # fp32 partial GEMVs
    want = (parts[0] + parts[1]).to(dtype)
    psz = 8 if dtype == torch.float32 else 4
    slots, slot_packets = 4, world * N * 8 // psz
    arenas = [torch.zeros(slots * slot_packets * psz, dtype=torch.uint8, device=DEV) for _ in range(world)]
    epochs = [torch.zeros(slots, dtype=torch.int32, device=DEV) for _ in range(world)]
    ptrs = [a.data_ptr() for a in arenas]
    for rep in range(2):
        for r in range(world):
            capi.mul_mat_vec_a8_tp_rowpar(wk[r], xk[r], ptrs, epochs[r], 0, slot_packets, t, r)
        got = [capi.tp_unpack_sum(arenas[r], epochs[r], 0, slot_packets, N, world, dtype) for r in range(world)]
        assert torch.equal(got[0], got[1])
        assert torch.equal(got[0].view(1, N), want), "not the rank-ordered fp32 sum of the partial GEMVs"
    full = capi.mul_mat_vec_a8(w, x, t, N)
    assert rel_l2(got[0].float().cpu().view(1, N), full.float().cpu()) <= 1e-3   # (fp16 rounding of the result: 5e-4)
    if ref.available and name != "IQ2_XXS" or ref.available and K <= 4096:
        r_full = ref.ops.ggml_mul_mat_vec_a8(w, x, t, N)
        assert rel_l2(got[0].float().cpu().view(1, N), r_full.float().cpu()) <= 1e-3
    # column-parallel call on x2 = x[:N] + s * reduced(slot 0)  (rows of w2 split over the ranks)
    s = 2.0 ** -10
    _, w2 = dev_w(t, 512, N, seed=12)
    x2 = (x[:, :N].float() + s * want.float()).to(dtype)
    want2 = capi.mul_mat_vec_a8(w2, x2, t, 512)
    for r in range(world):
        capi.mul_mat_vec_a8_tp(w2[r * 256:(r + 1) * 256].contiguous(), x[:, :N].contiguous(), ptrs, epochs[r], 1, slot_packets, t, r,
                               add_slot=0, add_scale=s, add_parts=world)
    for r in range(world):
        assert torch.equal(capi.tp_unpack(arenas[r], epochs[r], 1, 1, slot_packets, 512, dtype), want2)
    # row-parallel call whose activations are this rank's slice of s * gathered(slot 1)  (no X at all)
    _, w3 = dev_w(t, 256, 512, seed=13)
    x3 = (s * want2.float()).to(dtype)
    w3k = [tpmod.shard_cols(w3, t, r, world) for r in range(world)]
    p3 = [capi.mul_mat_vec_a8(w3k[r], x3[:, r * 256:(r + 1) * 256].contiguous().float(), t, 256) for r in range(world)]
    want3 = (p3[0] + p3[1]).to(dtype)
    for r in range(world):
        capi.mul_mat_vec_a8_tp_rowpar(w3k[r], None, ptrs, epochs[r], 2, slot_packets, t, r, add_slot=1, add_scale=s, dtype=dtype)
    for r in range(world):
        assert torch.equal(capi.tp_unpack_sum(arenas[r], epochs[r], 2, slot_packets, 256, world, dtype).view(1, 256), want3)
    torch.cuda.synchronize()
    assert capi.last_status() == 0


@pytest.mark.parametrize("case", [("Q4_K", 12, 1, 512, 2048, 96), ("Q6_K", 14, 1, 256, 8192, 130), ("IQ2_XXS", 16, 4, 512, 4096, 128),
                                  ("IQ4_XS", 23, 4, 1024, 1024, 40)])
def test_tp_matmul_tiles_one_gpu(case):
    """Prefill GEMM, two emulated ranks: each stores its column block into both gathered outputs
    (tile epilogue, or the partial-tile adder when K is split) and raises both flags."""
    name, t, op, N, K, M = case
    world = 2
    wn, w = dev_w(t, N, K, seed=7)
    x = dev_x(M, K, seed=7)
    want = capi.mul_mat_a8(w, x, t, N) if op == capi.OP_MMQ else capi.dequant_matmul(w, x, t, N)
    ys = [torch.zeros((M, N), dtype=torch.float16, device=DEV) for _ in range(world)]
    flags = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(world)]
    epochs = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(world)]
    slot = 5
    for rep in range(2):
        for y in ys:
            y.zero_()
        for r in range(world):
            capi.matmul_tp(op, w[r * N // world:(r + 1) * N // world].contiguous(), x, [y.data_ptr() for y in ys],
                           [f.data_ptr() for f in flags], epochs[r], slot, t, r)
        for r in range(world):
            capi.tp_wait(flags[r], epochs[r], slot, world)
        torch.cuda.synchronize()
        assert capi.last_status() == 0
        for r in range(world):
            assert int(flags[r][slot]) == world * (rep + 1) and int(epochs[r][slot]) == rep + 1
            # same arithmetic per element; only a different split of K may reorder the fp32 sums
            assert rel_l2(ys[r].float().cpu(), want.float().cpu()) <= 3e-4
        assert torch.equal(ys[0], ys[1])


def test_waits_on_other_gpus_run_out_and_report():
    """A packet that nobody sends and a flag that nobody raises: with a limit of about a millisecond
    the waiting kernels give up by themselves, the status word reads E_TIMEOUT (-8) and the
    context stays usable."""
    capi.set_wait_limit_cycles(2_000_000)
    try:
        arena = torch.zeros(4 * 256 * 4, dtype=torch.uint8, device=DEV)
        epochs = torch.ones(4, dtype=torch.int32, device=DEV)        # expects launch 1 of every slot: never sent
        out = capi.tp_unpack(arena, epochs, 0, 1, 256, 256, torch.float16)
        torch.cuda.synchronize()
        assert capi.last_status() == -8
        assert capi.last_status() == 0                               # reading clears it
        flags = torch.zeros(8, dtype=torch.int32, device=DEV)
        capi.tp_wait(flags, epochs, 0, 2)
        torch.cuda.synchronize()
        assert capi.last_status() == -8
        # the quantizer's packet poll of a chained decode call gives up the same way
        t, N, K = 12, 64, 1024
        _, w = dev_w(t, N, K, seed=1)
        x = dev_x(1, K, seed=1)
        big = torch.zeros(4 * 1024 * 4, dtype=torch.uint8, device=DEV)
        ep = torch.zeros(4, dtype=torch.int32, device=DEV)
        ep[0] = 1
        capi.mul_mat_vec_a8_tp(w, x, [big.data_ptr()], ep, 1, 1024, t, 0, add_slot=0, add_scale=1.0)
        torch.cuda.synchronize()
        assert capi.last_status() == -8
    finally:
        capi.set_wait_limit_cycles(0)
    y = capi.mul_mat_vec_a8(w, x, t, N)                              # the device still works
    torch.cuda.synchronize()
    assert capi.last_status() == 0 and bool(torch.isfinite(y).all())


def test_mmq_split_k_matches_unsplit():
    """Few output tiles and long rows: the GEMM splits K over CTAs (fp32 partial tiles in the
    workspace, added in slice order).  With a workspace that only holds the activations the same
    call runs unsplit; both must agree to fp16 rounding and match the oracle."""
    t = TYPES["Q4_K"]
    N, K, M = 512, 8192, 130
    wn, w = dev_w(t, N, K, seed=11)
    x = dev_x(M, K, seed=11)
    y_split = capi.mul_mat_a8(w, x, t, N)
    L = capi.lib()
    full = L.gguf_b200_workspace_bytes(1, t, M, N, K)
    kpad = (K + 511) // 512 * 512
    small = M * (kpad + (kpad // 32 + 63) // 64 * 64) * 2          # the activation matrix alone
    assert full > small
    ws = torch.empty(small, dtype=torch.uint8, device=DEV)
    y_one = torch.empty_like(y_split)
    rc = L.gguf_b200_mul_mat_a8(w.data_ptr(), x.data_ptr(), y_one.data_ptr(), ws.data_ptr(), small, t, 1, M, N, K,
                                torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and capi.last_status() == 0
    assert rel_l2(y_split.float().cpu(), y_one.float().cpu()) <= 3e-4
    y64, _ = cpu.matmul_a8(wn, t, x.cpu().numpy(), "float16", mmq=True)
    assert rel_l2(y_split.float().cpu().numpy(), y64) <= REL_L2_TOL
    assert rel_l2(y_one.float().cpu().numpy(), y64) <= REL_L2_TOL


# ---------------------------------------------------------------- full benchmark sizes -----------

def test_mmq_full_size_deterministic_linear_and_close_to_reference(ref):
    """Q4_K 14336x4096 at 512 tokens (the prefill benchmark shape): two runs give identical bits;
    doubling every d and dmin (exact in fp16) doubles the output exactly; the reference's own
    tiled kernel, when it was built, agrees within the tolerance."""
    t, N, K, M = 12, 14336, 4096, 512
    wn = synth.make_weight(t, N, K, seed=3)
    w = torch.from_numpy(wn).to(DEV)
    x = dev_x(M, K, seed=3)
    y1 = capi.mul_mat_a8(w, x, t, N)
    y2 = capi.mul_mat_a8(w, x, t, N)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert torch.equal(y1, y2)
    blocks = wn.reshape(-1, 144).copy()
    d = blocks[:, 0:4].copy().view(np.float16) * np.float16(2)
    blocks[:, 0:4] = d.view(np.uint8)
    y3 = capi.mul_mat_a8(torch.from_numpy(blocks.reshape(N, -1)).to(DEV), x, t, N)
    assert torch.equal(y3.float(), 2 * y1.float())
    if ref.available:
        r = ref.ops.ggml_mul_mat_a8(w, x, t, N)
        assert rel_l2(y1.float().cpu(), r.float().cpu()) <= REL_L2_TOL


def test_mmq_split_k_full_size_close_to_reference(ref):
    """Q4_K 4096x14336 at 64 tokens: 32 output tiles, so K is split over four CTAs per tile."""
    if not ref.available:
        pytest.skip("reference kernels not built")
    t, N, K, M = 12, 4096, 14336, 64
    wn, w = dev_w(t, N, K, seed=5)
    x = dev_x(M, K, seed=5)
    y = capi.mul_mat_a8(w, x, t, N)
    r = ref.ops.ggml_mul_mat_a8(w, x, t, N)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL


def test_moe_full_size_close_to_reference(ref):
    """The MoE benchmark configuration (64 experts, top-8, hidden 2048 -> 2 x 1024, Q4_0, 256 tokens):
    both expert GEMMs against the reference's kernels, and the decode form for 4 tokens."""
    if not ref.available:
        pytest.skip("reference kernels not built")
    t, E, top_k, hid, inter, T = 2, 64, 8, 2048, 1024, 256
    w13 = torch.from_numpy(np.stack([synth.make_weight(t, 2 * inter, hid, seed=100 + e) for e in range(E)])).to(DEV)
    x = torch.from_numpy(synth.make_activation(T, hid, seed=1)).to(DEV)
    _, ids = synth.make_routing(T, E, top_k, 0)
    blk = capi.lib().gguf_b200_moe_block_size(t)
    s, e, n = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(ids, blk, E)]
    s4, e4, n4 = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(ids, 4, E)]
    y = capi.moe_a8(x, w13, s, e, n, t, 2 * inter, top_k, T)
    r = ref.ops.ggml_moe_a8(x, w13, s4, e4, n4, t, 2 * inter, top_k, T)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL
    tid = torch.from_numpy(np.ascontiguousarray(ids[:4])).to(DEV).to(torch.int32)
    yv = capi.moe_a8_vec(x[:4].contiguous(), w13, tid, top_k, t, 2 * inter, 4)
    rv = ref.ops.ggml_moe_a8_vec(x[:4].contiguous(), w13, tid, top_k, t, 2 * inter, 4)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert rel_l2(yv.float().cpu(), rv.float().cpu()) <= REL_L2_TOL


FULL_GEMV = [("Q6_K", 37888, 3584), ("Q6_K", 3584, 18944), ("IQ4_XS", 37888, 3584), ("IQ4_XS", 3584, 18944),
             ("IQ2_XXS", 28672, 8192), ("IQ2_XXS", 8192, 28672), ("Q4_K", 4096, 14336), ("Q8_0", 3072, 1024)]


@pytest.mark.parametrize("case", FULL_GEMV)
def test_gemv_full_size_configs_close_to_reference(ref, case):
    """Decode GEMV at the full size of every benchmark configuration, against the reference's kernel."""
    if not ref.available:
        pytest.skip("reference kernels not built")
    name, N, K = case
    t = TYPES[name]
    w = torch.from_numpy(synth.make_weight(t, N, K, seed=11)).to(DEV)
    x = dev_x(1, K, seed=11)
    y = capi.mul_mat_vec_a8(w, x, t, N)
    r = ref.ops.ggml_mul_mat_vec_a8(w, x, t, N)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert rel_l2(y.float().cpu(), r.float().cpu()) <= 1e-4


FULL_GEMM = [("Q6_K", 37888, 3584, 256), ("Q6_K", 3584, 18944, 256), ("IQ4_XS", 37888, 3584, 256), ("IQ4_XS", 3584, 18944, 256),
             ("IQ2_XXS", 28672, 8192, 128), ("IQ2_XXS", 8192, 28672, 128)]


@pytest.mark.parametrize("case", FULL_GEMM)
def test_gemm_full_size_configs_close_to_reference(ref, case):
    """Prefill at the full size of the Qwen2.5-7B and 70B-class configurations: q8_1 tensor-core GEMM
    against the reference's tiled kernel (Q6_K), fused dequantize-GEMM against the reference's
    dequantize followed by a dense product (IQ types)."""
    if not ref.available:
        pytest.skip("reference kernels not built")
    name, N, K, M = case
    t = TYPES[name]
    w = torch.from_numpy(synth.make_weight(t, N, K, seed=13)).to(DEV)
    x = dev_x(M, K, seed=13)
    if name in MMQ_TYPES:
        y = capi.mul_mat_a8(w, x, t, N)
        r = ref.ops.ggml_mul_mat_a8(w, x, t, N)
    else:
        y = capi.dequant_matmul(w, x, t, N)
        r = x @ ref.ops.ggml_dequantize(w, t, N, K, torch.float16).T
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL


def test_moe_down_projection_full_size_close_to_reference(ref):
    """The second expert GEMM of the MoE configuration: 2048 routed rows of 1024 values, top_k = 1, w2 [64, 2048, 576 bytes]."""
    if not ref.available:
        pytest.skip("reference kernels not built")
    t, E, top_k, hid, inter, T = 2, 64, 8, 2048, 1024, 256
    w2 = torch.from_numpy(np.stack([synth.make_weight(t, hid, inter, seed=200 + e) for e in range(E)])).to(DEV)
    x2 = torch.from_numpy(synth.make_activation(T * top_k, inter, seed=2)).to(DEV)
    _, ids = synth.make_routing(T, E, top_k, 0)
    blk = capi.lib().gguf_b200_moe_block_size(t)
    s, e, n = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(ids, blk, E)]
    s4, e4, n4 = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(ids, 4, E)]
    y = capi.moe_a8(x2, w2, s, e, n, t, hid, 1, T * top_k)
    r = ref.ops.ggml_moe_a8(x2, w2, s4, e4, n4, t, hid, 1, T * top_k)
    torch.cuda.synchronize()
    assert capi.last_status() == 0
    assert rel_l2(y.float().cpu(), r.float().cpu()) <= REL_L2_TOL
