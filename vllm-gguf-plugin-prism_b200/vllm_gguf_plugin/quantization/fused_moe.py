# SPDX-License-Identifier: Apache-2.0
"""MoE method of the GGUF matmul path (reference: quantization/fused_moe.py).

``_fused_moe_gguf`` keeps the reference's routing (fused_moe.py:56-133): above 64 tokens and
for standard/K quants, two block-aligned expert GEMMs (``ops.ggml_moe_a8``) around the
activation; otherwise one GEMV per (token, expert) pair (``ops.ggml_moe_a8_vec``).  The
alignment step, the activation and the final top-k reduction are vLLM ops in the reference;
here they use vLLM when it is importable and small torch restatements otherwise, so the
expert GEMMs can be exercised on a box without vLLM.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .. import ops
from .utils import MMQ_QUANT_TYPES, MMVQ_QUANT_TYPES, logger

try:
    from vllm.model_executor.layers.fused_moe.fused_moe_method_base import FusedMoEMethodBase
    from vllm.model_executor.utils import set_weight_attrs
    from vllm.utils.torch_utils import direct_register_custom_op

    _HAVE_VLLM = True
except Exception:  # pragma: no cover
    FusedMoEMethodBase = object
    direct_register_custom_op = None
    _HAVE_VLLM = False

    def set_weight_attrs(weight, attrs):
        for k, v in (attrs or {}).items():
            setattr(weight, k, v)


def moe_align_block_size_torch(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Device-side restatement of vLLM's ``moe_align_block_size`` (the step the reference calls
    at fused_moe.py:66-68): slots (token*top_k + j) grouped by expert, each group padded to a
    multiple of ``block_size`` with the sentinel ``topk_ids.numel()``, one expert id per block.
    Returns (sorted_token_ids int32, expert_ids int32, num_tokens_post_padded int32[1])."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    numel = flat.numel()
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    padded = (counts + block_size - 1) // block_size * block_size
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    max_padded = numel + num_experts * (block_size - 1)
    max_padded = (max_padded + block_size - 1) // block_size * block_size
    sorted_ids = torch.full((max_padded,), numel, dtype=torch.int32, device=flat.device)
    order = torch.argsort(flat, stable=True)
    sorted_experts = flat[order]
    first = torch.cumsum(counts, 0) - counts
    rank = torch.arange(numel, device=flat.device) - first[sorted_experts]
    sorted_ids[starts[sorted_experts] + rank] = order.to(torch.int32)
    blocks = torch.arange(max_padded // block_size, device=flat.device) * block_size
    expert_ids = torch.searchsorted(ends, blocks, right=True).clamp_(max=num_experts - 1).to(torch.int32)
    return sorted_ids, expert_ids, ends[-1:].to(torch.int32)


def _align(topk_ids, block_size, num_experts):
    if _HAVE_VLLM:
        try:
            from vllm.model_executor.layers.fused_moe.fused_moe import moe_align_block_size

            return moe_align_block_size(topk_ids, block_size, num_experts)
        except Exception:
            pass
    return moe_align_block_size_torch(topk_ids, block_size, num_experts)


def _act(activation: str, inp: torch.Tensor) -> torch.Tensor:
    d = inp.shape[-1] // 2
    if _HAVE_VLLM:
        try:
            from vllm.model_executor.layers.fused_moe.activation import MoEActivation, apply_moe_activation

            out = torch.empty(inp.shape[:-1] + (d,), dtype=inp.dtype, device=inp.device)
            apply_moe_activation(MoEActivation.from_str(activation), out, inp)
            return out
        except Exception:
            pass
    gate, up = inp[..., :d], inp[..., d:]
    if activation == "silu":
        return F.silu(gate) * up
    if activation == "gelu":
        return F.gelu(gate) * up
    raise NotImplementedError(f"activation {activation!r}")


def _fused_moe_gguf(
    x: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    weight_type: int,
    weight_type2: int,
    activation: str,
) -> torch.Tensor:
    out_hidden_states = torch.empty_like(x)
    num_tokens, _ = x.shape
    E, N, _ = w1.shape
    top_k = topk_ids.shape[1]
    if weight_type2 in MMQ_QUANT_TYPES and weight_type in MMQ_QUANT_TYPES and x.shape[0] > 64:
        if (activation in ops.MOE_ACTIVATIONS and E <= 256 and w2.shape[0] == E and (N // 2) % 8 == 0
                and os.environ.get("VLLM_GGUF_FUSED_MOE", "1") == "1"):
            # one call: alignment, both expert GEMMs, activation, routing weights and top-k sum
            return ops.ggml_fused_moe(x, w1, w2, topk_weights, topk_ids, weight_type, weight_type2, activation)
        # the reference's sequence of separate ops (fused_moe.py:64-95)
        block_size = ops.ggml_moe_get_block_size(weight_type)
        sorted_token_ids, expert_ids, num_tokens_post_padded = _align(topk_ids, block_size, E)
        out = ops.ggml_moe_a8(x, w1, sorted_token_ids, expert_ids, num_tokens_post_padded, weight_type, N, top_k,
                              num_tokens)
        out = _act(activation, out)
        out = ops.ggml_moe_a8(out, w2, sorted_token_ids, expert_ids, num_tokens_post_padded, weight_type2,
                              w2.shape[1], 1, num_tokens * top_k)
    elif weight_type2 in MMVQ_QUANT_TYPES and weight_type in MMVQ_QUANT_TYPES:
        ids = topk_ids.to(torch.int32).contiguous()
        out = ops.ggml_moe_a8_vec(x, w1, ids, top_k, weight_type, N, num_tokens)
        out = _act(activation, out)
        out = ops.ggml_moe_a8_vec(out, w2, ids, 1, weight_type2, w2.shape[1], num_tokens * top_k)
    else:
        raise NotImplementedError(
            f"no GGUF MoE kernel for quantization types ({int(weight_type)}, {int(weight_type2)})")
    out = out.reshape(num_tokens, top_k, w2.shape[1]).mul_(topk_weights.view(num_tokens, top_k, 1).to(out.dtype))
    ops.moe_sum(out, out_hidden_states)
    return out_hidden_states


def _fused_moe_gguf_fake(x, w1, w2, topk_weights, topk_ids, weight_type, weight_type2, activation):
    return torch.empty_like(x)


fused_moe_gguf = _fused_moe_gguf
if _HAVE_VLLM:
    try:
        direct_register_custom_op(op_name="_fused_moe_gguf", op_func=_fused_moe_gguf, fake_impl=_fused_moe_gguf_fake)
        fused_moe_gguf = torch.ops.vllm._fused_moe_gguf
    except Exception:
        fused_moe_gguf = getattr(getattr(torch.ops, "vllm", None), "_fused_moe_gguf", _fused_moe_gguf)


class _TypeParam(torch.nn.Parameter):
    def __new__(cls):
        obj = super().__new__(cls, torch.empty(1, dtype=torch.uint8), requires_grad=False)
        obj.weight_type = 0
        return obj


class GGUFMoEMethod(FusedMoEMethodBase):
    """MoE method for GGUF (reference: fused_moe.py:161-278)."""

    def __init__(self, quant_config, moe=None):
        if _HAVE_VLLM and moe is not None:
            super().__init__(moe)
        self.quant_config = quant_config

    def create_weights(self, layer: torch.nn.Module, num_experts: int, hidden_size: int,
                       intermediate_size_per_partition: int, params_dtype: torch.dtype, **extra_weight_attrs):
        """Registers w13_weight [E, 2I, bytes] / w2_weight [E, H, bytes] as raw GGUF bytes (sized on
        load: the byte width depends on the quant type) and their type parameters."""
        # vLLM's FusedMoE passes its own loader among the extras; its set_weight_attrs refuses to
        # overwrite an attribute, so it is taken out first (reference: fused_moe.py:182)
        base_loader = extra_weight_attrs.pop("weight_loader", None)
        for name in ("w13_weight", "w2_weight"):
            w = torch.nn.Parameter(torch.empty(0, dtype=torch.uint8), requires_grad=False)
            w.num_experts = num_experts
            set_weight_attrs(w, {"is_gguf_weight": True, "weight_loader": self._load_weight, "base_weight_loader": base_loader})
            set_weight_attrs(w, extra_weight_attrs)
            layer.register_parameter(name, w)
            t = _TypeParam()
            set_weight_attrs(t, {"is_gguf_weight_type": True, "weight_loader": self._load_type})
            set_weight_attrs(t, extra_weight_attrs)
            layer.register_parameter(name + "_type", t)

    @staticmethod
    def _load_weight(param, loaded_weight, weight_name=None, shard_id=None, expert_id=None, return_success=False):
        """vLLM's MoE loader call (param, loaded_weight, weight_name, shard_id, expert_id).  GGUF stores
        the experts of one projection stacked ([E, rows, bytes]) or one expert at a time ([rows,
        bytes] with expert_id).  shard_id "w1" / "w3" are the gate / up halves of w13 (rows [0, I)
        and [I, 2I) of every expert), "w2" the down projection.  Tensor parallelism slices w1/w3 by
        rows and w2 by whole blocks of every row (reference: params.py:158-208)."""
        from .linear import tensor_parallel_rank_and_size

        w = loaded_weight.to(torch.uint8)
        rank, size = tensor_parallel_rank_and_size()
        if size > 1:
            dim = w.dim() - (1 if shard_id == "w2" else 2)      # bytes for w2, rows for w1 / w3
            n = w.shape[dim] // size
            if n > 0:
                w = w.narrow(dim, rank * n, n)
        rows, width = w.shape[-2], w.shape[-1]
        halves = 2 if shard_id in ("w1", "w3") else 1
        if param.data.numel() == 0:
            param.data = torch.zeros((param.num_experts, rows * halves, width), dtype=torch.uint8, device=w.device)
        r0 = rows if shard_id == "w3" else 0
        if w.dim() == 3:
            param.data[:, r0:r0 + rows].copy_(w)
        else:
            param.data[int(expert_id), r0:r0 + rows].copy_(w)
        return True if return_success else None

    @staticmethod
    def _load_type(param, loaded_weight, *args, **kwargs):
        param.weight_type = int(loaded_weight.item()) if isinstance(loaded_weight, torch.Tensor) else int(loaded_weight)
        return True if kwargs.get("return_success") else None

    def get_fused_moe_quant_config(self, layer: torch.nn.Module):
        return None

    def apply(self, layer, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
              shared_experts=None, shared_experts_input: torch.Tensor | None = None) -> torch.Tensor:
        if getattr(layer, "apply_router_weight_on_input", False):
            raise NotImplementedError("Apply router weight on input is not supported for fused GGUF MoE method.")
        activation = getattr(layer, "activation", "silu")
        activation = getattr(activation, "value", activation)
        return fused_moe_gguf(x, layer.w13_weight, layer.w2_weight, topk_weights, topk_ids,
                              layer.w13_weight_type.weight_type, layer.w2_weight_type.weight_type, activation)
