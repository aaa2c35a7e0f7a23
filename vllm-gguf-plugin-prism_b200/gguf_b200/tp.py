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
GEMV kernel sends every output element, as one tagged packet, straight into every rank's memory
over NVLink (peer-mapped symmetric memory); the next GEMV's quantizer reads the packets.  For
prefill :class:`FusedGatherMatmul` does the same with the tensor-core kernel's output tiles and a
per-call flag.  No NCCL call sits on either path.
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


def shard_cols(weight: torch.Tensor, qtype: int, rank: int, world: int) -> torch.Tensor:
    """Rank ``rank``'s K-shard of a packed ``[N, bytes]`` weight: whole blocks of every row, the way
    the reference narrows dim 1 of a row-parallel layer (quantization/params.py:259-264)."""
    from . import synth

    block, size = synth.QUANT_SIZES[int(qtype)]
    blocks = weight.shape[-1] // size
    if blocks % world != 0:
        raise ValueError(f"{blocks} blocks per row are not divisible by the tensor-parallel size {world}")
    b = blocks // world * size
    return weight.narrow(weight.dim() - 1, rank * b, b).contiguous()


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


class RowParallelGGUFLinear:
    """A packed GGUF weight split by K (whole blocks of every row) over the ranks of ``group``;
    ``__call__(x_local)`` takes this rank's K/g activations and returns the all-reduced ``[M, N]``
    product on every rank (plain collective: the baseline of the fused ``FusedGatherGemv.rowpar``)."""

    def __init__(self, weight: torch.Tensor, qtype: int, group=None,
                 matmul: Callable[[torch.Tensor, torch.Tensor, int], torch.Tensor] | None = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.qtype = int(qtype)
        self.weight = shard_cols(weight, qtype, self.rank, self.world)
        if matmul is None:
            from vllm_gguf_plugin.quantization.linear import _fused_mul_mat_gguf as matmul
        self.matmul = matmul

    def local(self, x_local: torch.Tensor) -> torch.Tensor:
        return self.matmul(x_local, self.weight, self.qtype)

    def __call__(self, x_local: torch.Tensor) -> torch.Tensor:
        y = self.local(x_local)
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        return y


def _group_info(group):
    """(group, rank, world); without an initialised process group: a group of one."""
    if not dist.is_initialized():
        return None, 0, 1
    group = group if group is not None else dist.group.WORLD
    return group, dist.get_rank(group), dist.get_world_size(group)


def _symmetric_arena(nbytes: int, device, group):
    """A zeroed uint8 buffer of `nbytes` that every rank of `group` maps; returns (tensor, handle,
    [base pointers]).  A group of one gets ordinary device memory."""
    if group is None or dist.get_world_size(group) == 1:
        arena = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        return arena, None, [arena.data_ptr()]
    import torch.distributed._symmetric_memory as symm_mem

    arena = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    arena.zero_()
    handle = symm_mem.rendezvous(arena, group)
    ptrs = [int(p) for p in handle.buffer_ptrs]
    torch.cuda.synchronize(device)
    dist.barrier(group)  # every rank's buffer is zero before anyone writes into it
    return arena, handle, ptrs


class FusedGatherGemv:
    """Decode GEMVs of one tensor-parallel group whose outputs land in every rank's memory.

    Each of ``slots`` call slots holds one gathered vector of up to ``n_total`` elements as tagged
    packets (see ``gguf_b200_mul_mat_vec_a8_tp``) in a symmetric-memory arena that all ranks map.
    ``__call__(slot, w_local, x, qtype, add_slot, add_scale)`` runs this rank's rows of the product
    and sends them to all ranks; the activations may include the vector gathered in another slot
    (``x + add_scale * gathered[add_slot]``), which the call's own quantizer waits for -- a chain of
    dependent GEMVs then contains no collective and no wait kernel.  ``gathered(slot)`` returns plain
    vectors for any other consumer.  All ranks must make the same sequence of calls; needs CUDA
    peer access between the ranks' GPUs.

    ``rowpar(slot, w_kshard, x_local, qtype, ...)`` is the row-parallel (K-sharded) form with the
    all-reduce fused in: this rank's partial sums over its K columns go to every rank as fp32
    packets, and ``reduced(slot, n)`` -- or a later call with ``add_slot=slot, add_parts=world`` --
    adds the ``world`` partial vectors in rank order.  ``reduce_n`` (constructor) is the longest
    vector reduced that way; a slot then has room for ``world`` fp32 partial vectors of that length.
    """

    def __init__(self, n_total: int, slots: int, dtype: torch.dtype, device: torch.device, group=None, reduce_n: int = 0):
        from . import capi

        self.capi = capi
        self.group, self.rank, self.world = _group_info(group)
        self.n_total, self.slots, self.dtype = int(n_total), int(slots), dtype
        self.packet_bytes = 8 if dtype == torch.float32 else 4
        units = max(self.n_total, (self.world * int(reduce_n) * 8 + self.packet_bytes - 1) // self.packet_bytes)
        self.slot_packets = (units + 63) // 64 * 64
        self.arena, self.handle, self.base_ptrs = _symmetric_arena(self.slots * self.slot_packets * self.packet_bytes,
                                                                   device, self.group)
        self.epochs = torch.zeros(self.slots, dtype=torch.int32, device=device)

    def __call__(self, slot: int, w_local: torch.Tensor, x: torch.Tensor | None, qtype: int, add_slot: int = -1,
                 add_scale: float = 0.0, add_parts: int = 1) -> None:
        self.capi.mul_mat_vec_a8_tp(w_local, x, self.base_ptrs, self.epochs, slot, self.slot_packets, qtype, self.rank,
                                    add_slot, add_scale, dtype=self.dtype, add_parts=add_parts)

    def rowpar(self, slot: int, w_kshard: torch.Tensor, x_local: torch.Tensor | None, qtype: int, add_slot: int = -1,
               add_scale: float = 0.0, add_parts: int = 1) -> None:
        self.capi.mul_mat_vec_a8_tp_rowpar(w_kshard, x_local, self.base_ptrs, self.epochs, slot, self.slot_packets, qtype,
                                           self.rank, add_slot, add_scale, dtype=self.dtype, add_parts=add_parts)

    def reduced(self, slot: int, n: int, out: torch.Tensor | None = None) -> torch.Tensor:
        """The all-reduced ``[n]`` vector of a row-parallel call (waits for all ranks' partial sums)."""
        return self.capi.tp_unpack_sum(self.arena, self.epochs, slot, self.slot_packets, n, self.world, self.dtype, out=out)

    def gathered(self, slot0: int, nslots: int = 1, n: int | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """Plain ``[nslots, n]`` tensor of the vectors gathered in slots slot0.. (waits for all ranks' packets)."""
        return self.capi.tp_unpack(self.arena, self.epochs, slot0, nslots, self.slot_packets,
                                   self.n_total if n is None else n, self.dtype, out=out)


class FusedGatherMatmul:
    """Prefill GEMMs of one tensor-parallel group: every rank's tensor-core kernel stores its
    column block of the ``[m, n_total]`` result into all ranks' output matrices (symmetric memory)
    and raises a per-call flag; ``wait`` queues the one-thread kernel that waits for all ranks."""

    FLAG_BYTES = 4096

    def __init__(self, m: int, n_total: int, slots: int, dtype: torch.dtype, device: torch.device, group=None):
        from . import capi

        self.capi = capi
        self.group, self.rank, self.world = _group_info(group)
        if slots > 1024:
            raise ValueError("at most 1024 call slots")
        self.m, self.n_total, self.slots, self.dtype = int(m), int(n_total), int(slots), dtype
        esz = torch.empty((), dtype=dtype).element_size()
        self.slot_bytes = (self.m * self.n_total * esz + 255) // 256 * 256
        self.arena, self.handle, self.base_ptrs = _symmetric_arena(self.FLAG_BYTES + self.slots * self.slot_bytes, device,
                                                                   self.group)
        self.flags = self.arena[: self.FLAG_BYTES].view(torch.int32)
        self.epochs = torch.zeros(1024, dtype=torch.int32, device=device)

    def out(self, slot: int, m: int | None = None, n_total: int | None = None) -> torch.Tensor:
        m = self.m if m is None else m
        n_total = self.n_total if n_total is None else n_total
        o = self.FLAG_BYTES + slot * self.slot_bytes
        esz = torch.empty((), dtype=self.dtype).element_size()
        return self.arena[o: o + m * n_total * esz].view(self.dtype).view(m, n_total)

    def __call__(self, slot: int, op: int, w_local: torch.Tensor, x: torch.Tensor, qtype: int, wait: bool = True) -> torch.Tensor:
        n_total = w_local.shape[0] * self.world
        off = self.FLAG_BYTES + slot * self.slot_bytes
        self.capi.matmul_tp(op, w_local, x, [b + off for b in self.base_ptrs], self.base_ptrs, self.epochs, slot, qtype,
                            self.rank)
        if wait:
            self.wait(slot)
        return self.out(slot, x.shape[0], n_total)

    def wait(self, slot: int) -> None:
        self.capi.tp_wait(self.flags, self.epochs, slot, self.world)
