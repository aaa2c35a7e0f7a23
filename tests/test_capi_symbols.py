"""CPU: the C-ABI library builds, loads, exports every declared symbol and validates arguments
(no kernel is launched here)."""
import ctypes
import re

from helpers import ROOT


def declared_symbols():
    text = (ROOT / "include" / "gguf_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gguf_b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(native_libs):
    lib = ctypes.CDLL(str(native_libs[0]))
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/gguf_b200.h but not exported"


def test_binding_table_covers_the_header(native_libs):
    from gguf_b200 import capi

    assert set(declared_symbols()) == set(capi.SIGNATURES)


def test_geometry_and_error_codes(native_libs):
    from gguf_b200 import capi

    lib = capi.lib()
    sizes = {2: (32, 18), 8: (32, 34), 12: (256, 144), 14: (256, 210), 16: (256, 66), 23: (256, 136)}
    for t, (bs, ts) in sizes.items():
        assert lib.gguf_b200_block_size(t) == bs and lib.gguf_b200_type_size(t) == ts
    assert lib.gguf_b200_type_size(10) == 84 and lib.gguf_b200_block_size(11) == 256
    assert lib.gguf_b200_type_size(9) == 0 and lib.gguf_b200_block_size(9) == 0
    assert lib.gguf_b200_q8_1_row_bytes(1024) == 1024 // 32 * 36
    assert lib.gguf_b200_q8_1_row_bytes(800) == 1024 // 32 * 36
    assert lib.gguf_b200_moe_block_size(2) == 64 and lib.gguf_b200_moe_block_size(11) == 64 and lib.gguf_b200_moe_block_size(16) == 0
    assert lib.gguf_b200_workspace_bytes(capi.OP_GEMV, 12, 2, 0, 4096) == 2 * 4096 + 2 * 128 * 8
    assert lib.gguf_b200_workspace_bytes(capi.OP_MMQ, 8, 4, 0, 1024) == 4 * 1024 * 2
    assert lib.gguf_b200_workspace_bytes(capi.OP_MMQ, 12, 4, 0, 1024) == 4 * (1024 + 64) * 2
    # argument validation happens before any CUDA call
    null = ctypes.c_void_p(0)
    p = ctypes.c_void_p(4096)
    assert lib.gguf_b200_mul_mat_vec_a8(p, p, p, p, 1 << 20, 9, 1, 1, 8, 256, null) == -1   # type (Q8_1 is not a weight type)
    assert lib.gguf_b200_mul_mat_a8(p, p, p, p, 1 << 20, 21, 1, 1, 8, 256, null) == -1       # IQ3_S has no tiled kernel
    assert lib.gguf_b200_mul_mat_vec_a8(p, p, p, p, 1 << 20, 12, 7, 1, 8, 256, null) == -2  # dtype
    assert lib.gguf_b200_mul_mat_vec_a8(p, p, p, p, 1 << 20, 12, 1, 1, 8, 100, null) == -3  # K % 256
    assert lib.gguf_b200_mul_mat_vec_a8(null, p, p, p, 1 << 20, 12, 1, 1, 8, 256, null) == -4
    assert lib.gguf_b200_mul_mat_vec_a8(ctypes.c_void_p(4100), p, p, p, 1 << 20, 12, 1, 1, 8, 256, null) == -4  # alignment
    assert lib.gguf_b200_mul_mat_vec_a8(p, p, p, p, 16, 12, 1, 1, 8, 256, null) == -5       # workspace
    assert lib.gguf_b200_mul_mat_a8(p, p, p, p, 1 << 20, 16, 1, 1, 8, 256, null) == -1      # IQ has no q8_1 GEMM
    assert lib.gguf_b200_dequant_matmul(p, p, p, p, 0, 12, 1, 1, 8, 256, null) == -1
    assert lib.gguf_b200_dequant_matmul(p, p, p, p, 0, 16, 0, 1, 8, 256, null) == -2        # fp32 not fused
    assert lib.gguf_b200_dequantize(p, 12, p, 1, 100, null) == -3
    assert lib.gguf_b200_mul_mat_vec_a8(p, p, p, p, 0, 12, 1, 0, 8, 256, null) == 0          # empty batch
    assert b"workspace" in lib.gguf_b200_error_string(-5)
    # dense GEMM workspace: activations (+ fp32 partial tiles when few tiles and long rows split K)
    act = lambda m, k: (m * (k + (k // 32 + 63) // 64 * 64) * 2 + 255) // 256 * 256
    assert lib.gguf_b200_workspace_bytes(capi.OP_MMQ, 12, 512, 14336, 4096) == act(512, 4096)              # 224 tiles: no split
    assert lib.gguf_b200_workspace_bytes(capi.OP_MMQ, 12, 512, 4096, 14336) == act(512, 14336) + 2 * 512 * 4096 * 4
    assert lib.gguf_b200_workspace_bytes(capi.OP_MMQ, 12, 64, 4096, 14336) == act(64, 14336) + 4 * 64 * 4096 * 4
    assert lib.gguf_b200_workspace_bytes(capi.OP_DEQUANT_MATMUL, 16, 128, 28672, 8192) == 0
    assert lib.gguf_b200_workspace_bytes(capi.OP_DEQUANT_MATMUL, 16, 128, 8192, 28672) == 2 * 128 * 8192 * 4
    assert lib.gguf_b200_workspace_bytes(capi.OP_DEQUANT_MATMUL, 16, 128, 1024, 28672) == 16 * 128 * 1024 * 4   # 8 tiles: 16 K slices


def test_tensor_parallel_entry_points_validate_arguments(native_libs):
    from gguf_b200 import capi

    lib = capi.lib()
    null = ctypes.c_void_p(0)
    p = ctypes.c_void_p(4096)
    two = (ctypes.c_void_p * 2)(4096, 8192)
    ptrs = ctypes.cast(two, ctypes.c_void_p)
    # decode: W, X, packet arenas, epochs, slot, add_slot, add_scale, add_parts, slot_packets, ws, ws_bytes, type, dtype, N_local, K, rank, world, stream
    args = lambda **kw: [kw.get("W", p), kw.get("X", p), kw.get("y", ptrs), kw.get("e", p), kw.get("slot", 0), kw.get("add", -1), 0.0,
                         kw.get("parts", 1), kw.get("sp", 1024), p, 1 << 20, kw.get("type", 12), 1, 64, 256, kw.get("rank", 0),
                         kw.get("world", 2), null]
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(y=null)) == -4
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(e=null)) == -4
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(X=null)) == -4          # no activations at all
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(world=9)) == -3
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(rank=2)) == -3
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(slot=-1)) == -3
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(sp=100)) == -3          # slot too small for world * N_local
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(add=0)) == -3           # a call cannot consume its own slot
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(type=9)) == -1
    assert lib.gguf_b200_mul_mat_vec_a8_tp(*args(add=1, parts=3)) == -3  # partial vectors come one per rank, or not at all
    # row-parallel: same arguments, N and K_local in place of N_local and K; a slot holds world * N fp32 partials
    assert lib.gguf_b200_mul_mat_vec_a8_tp_rowpar(*args(y=null)) == -4
    assert lib.gguf_b200_mul_mat_vec_a8_tp_rowpar(*args(world=9)) == -3
    assert lib.gguf_b200_mul_mat_vec_a8_tp_rowpar(*args(sp=200)) == -3   # 2 ranks x 64 rows x 8 bytes > 200 x 4
    assert lib.gguf_b200_mul_mat_vec_a8_tp_rowpar(*args(type=9)) == -1
    assert lib.gguf_b200_tp_unpack_sum(null, p, 0, 1024, 64, 2, p, 1, null) == -4
    assert lib.gguf_b200_tp_unpack_sum(p, p, 0, 1024, 64, 9, p, 1, null) == -3
    assert lib.gguf_b200_tp_unpack_sum(p, p, 0, 1024, 4096, 2, p, 1, null) == -3   # partials beyond the slot
    assert lib.gguf_b200_tp_unpack(null, p, 0, 1, 1024, 64, p, 64, 1, null) == -4
    assert lib.gguf_b200_tp_unpack(p, p, 0, 1, 1024, 2048, p, 2048, 1, null) == -3   # n beyond the slot
    assert lib.gguf_b200_tp_unpack(p, p, 0, 1, 1024, 64, p, 64, 9, null) == -2
    # prefill: op, W, X, outputs, flags, epochs, slot, ws, ws_bytes, type, dtype, M, N_local, K, rank, world, stream
    margs = lambda **kw: [kw.get("op", capi.OP_MMQ), p, p, kw.get("y", ptrs), ptrs, p, 0, p, 1 << 30, kw.get("type", 12),
                          kw.get("dtype", 1), 32, 64, 256, 0, kw.get("world", 2), null]
    assert lib.gguf_b200_matmul_tp(*margs(y=null)) == -4
    assert lib.gguf_b200_matmul_tp(*margs(op=capi.OP_GEMV)) == -3
    assert lib.gguf_b200_matmul_tp(*margs(world=0)) == -3
    assert lib.gguf_b200_matmul_tp(*margs(type=16)) == -1                # IQ types go through OP_DEQUANT_MATMUL
    assert lib.gguf_b200_matmul_tp(*margs(op=capi.OP_DEQUANT_MATMUL, type=12)) == -1
    assert lib.gguf_b200_matmul_tp(*margs(op=capi.OP_DEQUANT_MATMUL, type=16, dtype=0)) == -2
    assert lib.gguf_b200_tp_wait(null, p, 0, 2, null) == -4
    assert lib.gguf_b200_tp_wait(p, p, 0, 0, null) == -3
    lib.gguf_b200_set_wait_limit_cycles(0)                                # restores the default; no device call


def test_ops_module_fails_loudly_without_extension(tmp_path, monkeypatch):
    """The product path has no fallback: importing ops next to a missing extension raises."""
    import importlib
    import shutil
    import sys

    pkg = tmp_path / "vllm_gguf_plugin"
    pkg.mkdir()
    src = ROOT / "vllm-gguf-plugin-prism_b200" / "vllm_gguf_plugin"
    shutil.copy(src / "ops.py", pkg / "ops.py")
    (pkg / "__init__.py").write_text("")
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k.split(".")[0] == "vllm_gguf_plugin"}
    monkeypatch.syspath_prepend(str(tmp_path))
    try:
        try:
            importlib.import_module("vllm_gguf_plugin.ops")
            raised = False
        except ImportError as e:
            raised = "not built" in str(e)
        assert raised
    finally:
        for k in [k for k in sys.modules if k.split(".")[0] == "vllm_gguf_plugin"]:
            del sys.modules[k]
        sys.modules.update(saved)
