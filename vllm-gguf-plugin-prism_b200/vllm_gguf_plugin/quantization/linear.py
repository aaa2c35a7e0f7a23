# SPDX-License-Identifier: Apache-2.0
"""Linear method of the GGUF matmul path (reference: quantization/linear.py).

``_fused_mul_mat_gguf`` keeps the reference's batch-size routing (linear.py:35-58):
GEMV for small batches, the tensor-core q8_1 GEMM for standard/K quants, and for IQ types
above the GEMV threshold the dequantize-then-matmul route -- fused here into one kernel for
fp16/bf16 activations.  ``GGUFLinearMethod`` keeps the reference's method signatures
(linear.py:80-101, 154, 221-226); weights are raw GGUF bytes ``uint8 [N, K/QK*type_size]``.
vLLM is optional at import time: with it the method registers as a vLLM LinearMethodBase and
the dispatcher as the custom op ``vllm::_fused_mul_mat_gguf``; without it the same Python
objects are plain classes/functions, so the kernels stay testable on a box without vLLM.
"""
from __future__ import annotations

import torch

from .. import ops
from .utils import (
    DEQUANT_TYPES,
    IMATRIX_QUANT_TYPES,
    MMQ_QUANT_TYPES,
    MMVQ_QUANT_TYPES,
    UNQUANTIZED_TYPES,
    quant_sizes,
)

try:  # vLLM glue is optional (see module docstring)
    from vllm.model_executor.layers.linear import LinearMethodBase
    from vllm.model_executor.utils import set_weight_attrs
    from vllm.utils.torch_utils import direct_register_custom_op

    _HAVE_VLLM = True
except Exception:  # pragma: no cover - exercised on boxes without vLLM
    LinearMethodBase = object
    direct_register_custom_op = None
    _HAVE_VLLM = False

    def set_weight_attrs(weight, attrs):
        for k, v in (attrs or {}).items():
            setattr(weight, k, v)


def tensor_parallel_rank_and_size() -> tuple[int, int]:
    """(rank, size) of vLLM's tensor-parallel group, (0, 1) when vLLM or the group is absent.
    The weight loaders slice by it as the reference's parameter classes do
    (quantization/params.py:227-265)."""
    try:
        from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size

        return get_tensor_model_parallel_rank(), get_tensor_model_parallel_world_size()
    except Exception:
        return 0, 1


def _fused_mul_mat_gguf(x: torch.Tensor, weight: torch.Tensor, weight_type: int) -> torch.Tensor:
    # thresholds as in the reference (linear.py:38-41)
    if weight_type in IMATRIX_QUANT_TYPES:
        mmvq_safe = 8 if weight.shape[0] > 5120 else 16
    else:
        mmvq_safe = 2 if weight.shape[0] > 5120 else 6
    if x.shape[0] == 0:
        return torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)
    if weight_type in UNQUANTIZED_TYPES:
        return x @ weight.T
    if x.shape[0] <= mmvq_safe and weight_type in MMVQ_QUANT_TYPES:
        y = ops.ggml_mul_mat_vec_a8(weight, x, weight_type, weight.shape[0])
    elif weight_type in MMQ_QUANT_TYPES and int(weight_type) in ops._CUDA_GEMM_QUANT_TYPES:
        y = ops.ggml_mul_mat_a8(weight, x, weight_type, weight.shape[0])
    elif weight_type in DEQUANT_TYPES:
        # the reference's route for the code-book types: dequantize, then a dense product (fused for three of them)
        if x.dtype in (torch.float16, torch.bfloat16) and int(weight_type) in ops._DEQUANT_MATMUL_TYPES:
            y = ops.ggml_dequant_matmul(weight, x, weight_type, weight.shape[0])
        else:  # fp32 activations: the reference's two steps
            block_size, type_size = quant_sizes(weight_type)
            shape = (weight.shape[0], weight.shape[1] // type_size * block_size)
            y = x @ ops.ggml_dequantize(weight, weight_type, *shape, x.dtype).T
    else:
        raise NotImplementedError(f"Unsupported GGUF quantization type: {int(weight_type)}")
    return y


def _fused_mul_mat_gguf_fake(x: torch.Tensor, weight: torch.Tensor, weight_type: int) -> torch.Tensor:
    return torch.empty(x.shape[0], weight.shape[0], dtype=x.dtype, device=x.device)


fused_mul_mat_gguf = _fused_mul_mat_gguf
if _HAVE_VLLM:
    try:
        direct_register_custom_op(
            op_name="_fused_mul_mat_gguf",
            op_func=_fused_mul_mat_gguf,
            fake_impl=_fused_mul_mat_gguf_fake,
        )
        fused_mul_mat_gguf = torch.ops.vllm._fused_mul_mat_gguf
    except Exception:  # already registered by another copy of the plugin
        fused_mul_mat_gguf = getattr(getattr(torch.ops, "vllm", None), "_fused_mul_mat_gguf", _fused_mul_mat_gguf)


class GGUFWeightType(torch.nn.Parameter):
    """Scalar parameter carrying the GGML type id of a layer (and of each merged shard)."""

    def __new__(cls):
        obj = super().__new__(cls, torch.empty(1, dtype=torch.uint8), requires_grad=False)
        obj.weight_type = 0
        obj.shard_weight_type = {}
        return obj


class GGUFLinearMethod(LinearMethodBase):
    """Linear method for GGUF (reference: linear.py:80-264)."""

    def __init__(self, quant_config, layout=None) -> None:
        self.quant_config = quant_config
        self.layout = layout

    def create_weights(
        self,
        layer: torch.nn.Module,
        input_size_per_partition: int,
        output_partition_sizes: list[int],
        input_size: int,
        output_size: int,
        params_dtype: torch.dtype,
        **extra_weight_attrs,
    ):
        """Registers ``weight`` (raw GGUF bytes, sized when the first shard arrives because
        the byte width depends on the tensor's quant type) and ``weight_type``."""
        self.params_dtype = params_dtype
        # vLLM's layers pass their own `weight_loader` among the extras, and its set_weight_attrs
        # refuses to overwrite an attribute: take it out first, as the reference does
        # (linear.py:104).  It is kept as `fallback_weight_loader`; the loaders below are the ones
        # that understand raw GGUF bytes whose width is only known when the tensor arrives.
        fallback = extra_weight_attrs.pop("weight_loader", None)
        weight = torch.nn.Parameter(torch.empty(0, dtype=torch.uint8), requires_grad=False)
        weight.shard_id = []
        weight.shard_offset_map = {}
        weight.output_partition_sizes = list(output_partition_sizes)
        weight.input_size_per_partition = input_size_per_partition
        # how the layer is sharded over the tensor-parallel group: by output rows (column-parallel:
        # the per-partition output is smaller than the full one) or by input columns (row-parallel)
        weight.tp_shard_rows = sum(output_partition_sizes) < output_size
        weight.tp_shard_cols = input_size_per_partition < input_size
        set_weight_attrs(weight, {"input_dim": 1, "output_dim": 0, "is_gguf_weight": True,
                                  "weight_loader": self._load_weight, "fallback_weight_loader": fallback})
        set_weight_attrs(weight, extra_weight_attrs)
        layer.register_parameter("weight", weight)
        wtype = GGUFWeightType()
        set_weight_attrs(wtype, {"is_gguf_weight_type": True, "ignore_warning": True,
                                 "weight_loader": self._load_weight_type})
        set_weight_attrs(wtype, extra_weight_attrs)
        layer.register_parameter("weight_type", wtype)

    @staticmethod
    def _load_weight_type(param, loaded_weight, loaded_shard_id=None):
        t = int(loaded_weight.item()) if isinstance(loaded_weight, torch.Tensor) else int(loaded_weight)
        ids = loaded_shard_id if isinstance(loaded_shard_id, tuple) else (loaded_shard_id,)
        for sid in ids:
            if sid is None:
                param.weight_type = t
            else:
                param.shard_weight_type[sid] = t
                param.weight_type = param.weight_type or t

    @staticmethod
    def _load_weight(param, loaded_weight, loaded_shard_id=None):
        """Stores one tensor (or one shard of a merged layer) of raw block bytes, narrowed to this
        tensor-parallel rank: rows for a column-parallel layer (params.py:227-236), whole blocks of
        every row for a row-parallel one (params.py:259-264)."""
        if not hasattr(param, "_shards"):
            param._shards = {}
        w = loaded_weight.to(torch.uint8)
        rank, size = tensor_parallel_rank_and_size()
        if size > 1 and w.dim() == 2:
            if getattr(param, "tp_shard_rows", False) and w.shape[0] // size > 0:
                n = w.shape[0] // size
                w = w.narrow(0, rank * n, n)
            if getattr(param, "tp_shard_cols", False) and w.shape[1] // size > 0:
                b = w.shape[1] // size
                w = w.narrow(1, rank * b, b)
        param._shards[loaded_shard_id] = w.contiguous()
        if loaded_shard_id is not None and loaded_shard_id not in param.shard_id:
            param.shard_id.append(loaded_shard_id)

    def process_weights_after_loading(self, layer: torch.nn.Module):
        """Materializes ``layer.weight``: a single tensor, or merged shards stacked along the
        output dim and padded to the widest byte row (reference: linear.py:154-219)."""
        w = layer.weight
        shards = getattr(w, "_shards", None)
        if not shards:
            return
        if None in shards:
            data = shards[None].contiguous()
        else:
            order = [k for k in ("q", "k", "v") if k in shards] or sorted(shards)
            width = max(shards[k].shape[1] for k in order)
            rows = sum(shards[k].shape[0] for k in order)
            data = torch.zeros(rows, width, dtype=torch.uint8, device=shards[order[0]].device)
            start = 0
            for k in order:
                s = shards[k]
                data[start:start + s.shape[0], :s.shape[1]] = s
                w.shard_offset_map[k] = (start, start + s.shape[0], s.shape[1])
                start += s.shape[0]
            w.shard_id[:] = order
        w.data = data
        w._shards = {}

    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if self.layout is not None:
            x = self.layout.input_to_gguf(x)
        shard_id = layer.weight.shard_id
        if shard_id:
            shard_id = ["q", "k", "v"] if "q" in shard_id else shard_id
            weight = layer.weight
            fallback = layer.weight_type.weight_type
            types = [layer.weight_type.shard_weight_type.get(i, fallback) for i in shard_id]
            same_width = len({weight.shard_offset_map[i][2] for i in shard_id}) == 1
            if len(set(types)) == 1 and same_width:
                # same-type shards: one call on the stacked weight (reference: linear.py:241-245)
                out = fused_mul_mat_gguf(x, weight.data, types[0])
            else:
                result = []
                for i, t in zip(shard_id, types):
                    start, end, offset = weight.shard_offset_map[i]
                    result.append(fused_mul_mat_gguf(x, weight.data[start:end, :offset].contiguous(), t))
                out = torch.cat(result, axis=1)
        else:
            out = fused_mul_mat_gguf(x, layer.weight.data, layer.weight_type.weight_type)
        if bias is not None:
            out.add_(bias)
        return out
