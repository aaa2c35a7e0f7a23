"""Column-sharded tensor parallelism for the GGUF matmul path.

The reference only *slices* weights per tensor-parallel rank at load time
(``quantization/params.py:227-236``: ``loaded_weight.narrow(0, tp_rank * shard, shard)`` on the
packed ``[N, bytes]`` tensor) and leaves the collective to vLLM's parallel linear layers.  This
module is that pair in one place: rank r keeps rows ``[r*N/g, (r+1)*N/g)`` of the packed weight,
every rank holds the full activations, computes its ``[M, N/g]`` output slice with the local
kernel and the slices are all-gathered along the output dimension over ``torch.distributed``
(NCCL over NVLink on GPUs; the same code runs on the gloo backend for host-only tests).

Rows are independent, so the sharded result equals the single-GPU result bit for bit.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_rows(weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank ``rank``'s contiguous row slice of a packed ``[N, bytes]`` (or ``[E, N, bytes]``) weight."""
    dim = weight.dim() - 2
    n = weight.shape[dim]
    if n % world != 0:
        raise ValueError(f"output dimension {n} is not divisible by the tensor-parallel size {world}")
    shard = n // world
    return weight.narrow(dim, rank * shard, shard).contiguous()


def gather_columns(y_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather ``[M, N/g]`` slices into ``[M, N]`` (rank order = column order)."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    m, n_local = y_local.shape
    buf = torch.empty((world, m, n_local), dtype=y_local.dtype, device=y_local.device)
    if y_local.is_cuda:
        dist.all_gather_into_tensor(buf, y_local.contiguous(), group=group)
    else:  # gloo (host tensors) has no flat all-gather: gather into views of the same buffer
        dist.all_gather([buf[r] for r in range(world)], y_local.contiguous(), group=group)
    if m == 1:
        return buf.view(1, world * n_local)  # decode: the gathered buffer already is the row
    return buf.permute(1, 0, 2).reshape(m, world * n_local)


class ColumnParallelGGUFLinear:
    """A packed GGUF weight split by rows over the ranks of ``group``; ``__call__`` returns the full
    ``[M, N]`` product on every rank.  ``matmul(x, w_local, qtype)`` defaults to the plugin's
    dispatcher (GEMV / tensor-core GEMM by batch size)."""

    def __init__(self, weight: torch.Tensor, qtype: int, group=None,
                 matmul: Callable[[torch.Tensor, torch.Tensor, int], torch.Tensor] | None = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.qtype = int(qtype)
        self.weight = shard_rows(weight, self.rank, self.world)
        if matmul is None:
            from vllm_gguf_plugin.quantization.linear import _fused_mul_mat_gguf as matmul
        self.matmul = matmul

    def local(self, x: torch.Tensor) -> torch.Tensor:
        return self.matmul(x, self.weight, self.qtype)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        return gather_columns(y, self.group) if self.world > 1 else y
