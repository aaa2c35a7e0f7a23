"""GPU: the workspace-free GEMV entry point (gguf_b200_mul_mat_vec_a8_noalloc).

It serves hosts that cannot allocate -- an FFI caller inside an engine that has reserved the
whole device -- by keeping the quantized activations in a fixed array inside the library.  The
test calls it through the C-ABI and requires the same bits as the regular entry point (both
run the same kernels, so the comparison is exact), on two calls in a row whose shapes differ,
so that anything left in the shared array by the first call would show up in the second.
Collected last on purpose: a failure here cannot hide other results under `-x`."""
import ctypes

import numpy as np
import pytest
import torch

from gguf_b200 import capi, synth

pytestmark = pytest.mark.gpu
DEV = "cuda"


def case(t, n, k, m, seed, dtype=torch.float16):
    w = torch.from_numpy(synth.make_weight(t, n, k, seed=seed)).to(DEV)
    x = torch.from_numpy(synth.make_activation(m, k, seed=seed, dtype=np.float32)).to(DEV).to(dtype)
    return w, x


def test_noalloc_matches_regular_entry_point_twice_in_a_row(native_libs):
    # first call: large K, several vectors -- fills much of the shared array
    w1, x1 = case(synth.Q4_K, 384, 8192, 4, seed=1)
    y1 = capi.mul_mat_vec_a8_noalloc(w1, x1, synth.Q4_K, 384)
    # second call, immediately after, smaller and of another type: must not see stale scratch
    w2, x2 = case(synth.Q8_0, 520, 1024, 1, seed=2, dtype=torch.float32)
    y2 = capi.mul_mat_vec_a8_noalloc(w2, x2, synth.Q8_0, 520)
    torch.cuda.synchronize()
    assert torch.equal(y1, capi.mul_mat_vec_a8(w1, x1, synth.Q4_K, 384))
    assert torch.equal(y2, capi.mul_mat_vec_a8(w2, x2, synth.Q8_0, 520))
    # and once more with the first shape: same answer as before
    assert torch.equal(capi.mul_mat_vec_a8_noalloc(w1, x1, synth.Q4_K, 384), y1)
    assert capi.last_status() == 0


def test_noalloc_at_its_limits(native_libs):
    """The largest case the fixed array admits (8 vectors of K = 32768 fill it to the last byte)
    and a 5..8-vector case at moderate K, bit for bit against the regular entry point.  A bounded
    wait that expired inside these kernels would show in the same status word as everywhere else."""
    w, x = case(synth.Q8_0, 64, 32768, 8, seed=3)
    assert capi.lib().gguf_b200_workspace_bytes(capi.OP_GEMV, synth.Q8_0, 8, 64, 32768) == capi.lib().gguf_b200_noalloc_scratch_bytes()
    y = capi.mul_mat_vec_a8_noalloc(w, x, synth.Q8_0, 64)
    assert torch.equal(y, capi.mul_mat_vec_a8(w, x, synth.Q8_0, 64))
    for m in (5, 7, 8):
        w2, x2 = case(synth.Q4_K, 200, 4096, m, seed=m)
        assert torch.equal(capi.mul_mat_vec_a8_noalloc(w2, x2, synth.Q4_K, 200), capi.mul_mat_vec_a8(w2, x2, synth.Q4_K, 200))
    torch.cuda.synchronize()
    assert capi.last_status() == 0


def test_noalloc_rejects_sizes_beyond_its_array(native_libs):
    lib = capi.lib()
    assert lib.gguf_b200_noalloc_scratch_bytes() == 8 * (32768 + 8192)
    p = ctypes.c_void_p(4096)
    null = ctypes.c_void_p(0)
    assert lib.gguf_b200_mul_mat_vec_a8_noalloc(p, p, p, 12, 1, 9, 64, 4096, null) == -7      # M > 8
    assert lib.gguf_b200_mul_mat_vec_a8_noalloc(p, p, p, 12, 1, 1, 64, 65536, null) == -7     # K > 32768
    assert lib.gguf_b200_mul_mat_vec_a8_noalloc(p, p, p, 9, 1, 1, 64, 4096, null) == -1       # unsupported type (Q8_1 is not a weight type)
    assert b"limit" in lib.gguf_b200_error_string(-7)
