"""Column-sharded tensor parallelism for the GGUF matmul path.

The reference only *slices* weights per tensor-parallel rank at load time
(``quantization/params.py:227-236``: ``loaded_weight.narrow(0, tp_rank * shard, shard)`` on the
packed ``[N, bytes]`` tensor) and leaves the collective to vLLM's parallel linear layers.  This
module is that pair in one place: rank r keeps rows ``[r*N/g, (r+1)*N/g)`` of the packed weight,
every rank holds the full activations, computes its ``[M, N/g]`` output slice with the local
kernel and the slices are all-gathered along the output dimension over ``torch.distributed``
(NCCL over NVLink on GPUs; the same code runs on the gloo backend for host-only tests).

Rows are independent, so the sharded result equals the single-GPU result bit for bit.

For decode (one activation vector) :class:`FusedGatherGemv` removes the separate collective: the
GEMV kernel stores its slice straight into every rank's output vector over NVLink (peer-mapped
symmetric memory) and raises a per-call flag; a one-thread kernel on each rank waits for the
flags of all ranks.  No NCCL call sits on that path.
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


class FusedGatherGemv:
    """Decode GEMVs of one tensor-parallel group whose outputs land in every rank's memory.

    ``slots`` output vectors of ``n_total`` elements live in one symmetric-memory arena that all
    ranks map; ``__call__(slot, w_local, x, qtype)`` runs this rank's rows of the product and
    returns the full ``[1, n_total]`` vector of that slot once all ranks' slices have arrived
    (stream-ordered: the wait is a kernel on the current stream, or rides in the next call's quantizer).  All ranks must make the same
    sequence of calls.  Needs CUDA peer access between the ranks' GPUs.
    """

    FLAG_BYTES = 4096  # 1024 uint32 flags at the head of the arena

    def __init__(self, n_total: int, slots: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        from . import capi

        self.capi = capi
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if slots > 1024:
            raise ValueError("at most 1024 call slots")
        self.n_total, self.slots, self.dtype = int(n_total), int(slots), dtype
        esz = torch.empty((), dtype=dtype).element_size()
        self.row_bytes = (self.n_total * esz + 255) // 256 * 256
        nbytes = self.FLAG_BYTES + self.slots * self.row_bytes
        self.arena = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.arena.zero_()
        self.handle = symm_mem.rendezvous(self.arena, self.group)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.flags = self.arena[: self.FLAG_BYTES].view(torch.int32)
        self.epochs = torch.zeros(1024, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # every rank's flags are zero before anyone raises one

    def out(self, slot: int) -> torch.Tensor:
        o = self.FLAG_BYTES + slot * self.row_bytes
        return self.arena[o: o + self.row_bytes].view(self.dtype)[: self.n_total].view(1, self.n_total)

    def __call__(self, slot: int, w_local: torch.Tensor, x: torch.Tensor, qtype: int, wait_slot: int = -1,
                 wait: bool = True) -> torch.Tensor:
        """``wait_slot``: slot whose gathered vector ``x`` was computed from (the quantizer waits for
        it, no separate kernel).  ``wait=False`` leaves the gather of ``slot`` to a later call's
        ``wait_slot`` or to :meth:`wait`."""
        off = self.FLAG_BYTES + slot * self.row_bytes
        self.capi.mul_mat_vec_a8_tp(w_local, x, [b + off for b in self.base_ptrs], self.base_ptrs, self.epochs, slot, qtype,
                                    self.rank, wait_slot)
        if wait:
            self.wait(slot)
        return self.out(slot)

    def wait(self, slot: int) -> None:
        self.capi.tp_wait(self.flags, self.epochs, slot, self.world)
