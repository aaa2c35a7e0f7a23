"""Seeded synthetic GGUF blocks and routing tables with the shapes and value distributions of
the benchmark configurations (they stand in for the model-hub fixture files the reference's
kernel tests download, tests/utils.py:22-41, which cannot be fetched offline).

Weights are produced as raw block bytes, viewed ``uint8 [N, K/QK * type_size]`` -- exactly
what the plugin's loader hands to the ops (weight_utils.py:189-191).  Scales ``d`` are drawn
explicitly (|N(0,1)| * scale, rounded to fp16) so that no block carries a NaN/Inf scale;
every other field is uniform random bits.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K, IQ2_XXS, IQ4_XS = 2, 8, 12, 14, 16, 23
Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL = 3, 6, 7, 10, 11, 13, 20
IQ2_XS, IQ3_XXS, IQ1_S, IQ3_S, IQ2_S, IQ1_M = 17, 18, 19, 21, 22, 29
#             type: (values per block, bytes per block)
QUANT_SIZES = {Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210), IQ2_XXS: (256, 66),
               IQ4_XS: (256, 136),
               Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q2_K: (256, 84), Q3_K: (256, 110), Q5_K: (256, 176),
               IQ4_NL: (32, 18),
               IQ2_XS: (256, 74), IQ2_S: (256, 82), IQ3_XXS: (256, 98), IQ3_S: (256, 110), IQ1_S: (256, 50), IQ1_M: (256, 56)}
NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K", IQ2_XXS: "IQ2_XXS", IQ4_XS: "IQ4_XS",
         Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1", Q2_K: "Q2_K", Q3_K: "Q3_K", Q5_K: "Q5_K", IQ4_NL: "IQ4_NL",
         IQ2_XS: "IQ2_XS", IQ2_S: "IQ2_S", IQ3_XXS: "IQ3_XXS", IQ3_S: "IQ3_S", IQ1_S: "IQ1_S", IQ1_M: "IQ1_M"}
# where the fp16 scale(s) sit inside a block, and the |N(0,1)| multiplier the configs name
_D_OFFSETS = {Q4_0: (0,), Q8_0: (0,), Q4_K: (0, 2), Q6_K: (208,), IQ2_XXS: (0,), IQ4_XS: (0,),
              Q4_1: (0, 2), Q5_0: (0,), Q5_1: (0, 2), Q2_K: (80, 82), Q3_K: (108,), Q5_K: (0, 2), IQ4_NL: (0,),
              IQ2_XS: (0,), IQ2_S: (0,), IQ3_XXS: (0,), IQ3_S: (0,), IQ1_S: (0,), IQ1_M: ()}
_D_SCALE = {Q4_0: 0.01, Q8_0: 0.002, Q4_K: 0.01, Q6_K: 0.01, IQ2_XXS: 0.01, IQ4_XS: 0.01}


def weight_bytes(qtype: int, n: int, k: int) -> int:
    bs, ts = QUANT_SIZES[qtype]
    return n * (k // bs) * ts


def make_weight(qtype: int, n: int, k: int, seed: int = 0, d_scale: float | None = None) -> np.ndarray:
    """uint8 [n, k/QK*type_size] of random blocks of `qtype`."""
    bs, ts = QUANT_SIZES[qtype]
    assert k % bs == 0
    rng = np.random.default_rng(seed)
    nb = n * (k // bs)
    blocks = rng.integers(0, 256, size=(nb, ts), dtype=np.uint8)
    scale = _D_SCALE.get(qtype, 0.01) if d_scale is None else d_scale
    for off in _D_OFFSETS[qtype]:
        d = (np.abs(rng.standard_normal(nb)) * scale).astype(np.float16)
        blocks[:, off:off + 2] = d.view(np.uint8).reshape(nb, 2)
    if qtype == IQ1_M:
        # the fp16 scale has no field of its own: its four nibbles are the top nibbles of the four
        # 16-bit scale words at byte 48 (bits 0-3 in word 0, .. bits 12-15 in word 3)
        d = (np.abs(rng.standard_normal(nb)) * scale).astype(np.float16).view(np.uint16)
        sc = blocks[:, 48:56].copy().view(np.uint16)
        for i in range(4):
            sc[:, i] = (sc[:, i] & 0x0FFF) | (((d >> (4 * i)) & 0xF) << 12).astype(np.uint16)
        blocks[:, 48:56] = sc.view(np.uint8)
    if qtype == Q8_0:
        # int8 quants uniform in [-127, 127]
        blocks[:, 2:] = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    if qtype == Q6_K:
        # int8 sub-block scales uniform in [-32, 31]
        blocks[:, 192:208] = rng.integers(-32, 32, size=(nb, 16), dtype=np.int8).view(np.uint8)
    return blocks.reshape(n, (k // bs) * ts)


def make_activation(m: int, k: int, seed: int = 0, dtype=np.float16) -> np.ndarray:
    """[m, k] ~ N(0,1), rounded to `dtype` (float16 or float32)."""
    rng = np.random.default_rng(1_000_003 + seed)
    return rng.standard_normal((m, k)).astype(np.float32).astype(dtype)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def make_routing(tokens: int, experts: int, top_k: int, seed: int = 0):
    """Router logits ~N(0,1) -> softmax -> top-k: (topk_weights fp32 [T,k], topk_ids int32 [T,k])."""
    rng = np.random.default_rng(2_000_003 + seed)
    logits = rng.standard_normal((tokens, experts)).astype(np.float32)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    ids = np.argsort(-p, axis=1, kind="stable")[:, :top_k].astype(np.int32)
    w = np.take_along_axis(p, ids, axis=1).astype(np.float32)
    return w, ids


def moe_align_block_size(topk_ids: np.ndarray, block: int, experts: int):
    """Host restatement of the alignment step the caller runs before ggml_moe_a8
    (vLLM's moe_align_block_size, used at quantization/fused_moe.py:66-68): slots
    (token*top_k + j) grouped by expert, each group padded to a multiple of `block` with the
    sentinel ``topk_ids.size``; expert_ids holds one expert per block.
    Returns (sorted_token_ids int32, expert_ids int32, num_tokens_post_padded int32[1])."""
    flat = np.asarray(topk_ids, dtype=np.int64).reshape(-1)
    numel = flat.size
    max_padded = numel + experts * (block - 1) if numel >= experts else numel * block
    max_padded = max(max_padded, block)
    sorted_ids = np.full(((max_padded + block - 1) // block) * block, numel, dtype=np.int32)
    expert_ids = np.zeros(sorted_ids.size // block, dtype=np.int32)
    pos = 0
    for e in range(experts):
        slots = np.nonzero(flat == e)[0]
        if slots.size == 0:
            continue
        padded = (slots.size + block - 1) // block * block
        sorted_ids[pos:pos + slots.size] = slots
        expert_ids[pos // block:(pos + padded) // block] = e
        pos += padded
    return sorted_ids, expert_ids, np.array([pos], dtype=np.int32)
