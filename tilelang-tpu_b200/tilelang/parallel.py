"""Single-node multi-GPU sharding of the operator path.

The reference has no distributed code at all (one TPU core, `core_num = 1` in
src/tl_templates/tpu/kernel_template.cpp:33-43).  Every operator of the path is made of
independent units, so the work is split without any collective on the data path and the outputs
are assembled with ONE all-gather at the end (NCCL over NVLink on GPUs, gloo in the CPU tests):

    rows     RMSNorm / RoPE / SwiGLU / row reductions / top-k : contiguous row blocks
    heads    FlashAttention                                   : head blocks of bshd tensors
    columns  GEMM                                             : N-column blocks of B and C
    batch    MLA decode                                       : sequences, balanced by length

Partitions are static: every rank computes every rank's share from (n, world, rank), so nothing
about sizes is ever exchanged and the host never waits for the device.  A `ShardedOutput` is built
once per output tensor: it owns a rank-major receive buffer [world, slot], hands the kernel this
rank's slot to write into (so the all-gather runs in place, no staging copy), and gives the
gathered result back as a zero-copy view (rows) or assembles the final layout with one strided
copy launch per rank (heads, columns) or one gather launch (index lists).

One process per GPU; kernels only ever read the local GPU's memory.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def partition(n: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """[start, stop) of rank's share of n units, in multiples of `multiple` (the last rank takes
    the remainder); shares differ by at most one multiple."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    blocks = -(-n // multiple)
    base, extra = divmod(blocks, world)
    start_b = rank * base + min(rank, extra)
    stop_b = start_b + base + (1 if rank < extra else 0)
    return min(start_b * multiple, n), min(stop_b * multiple, n)


def shard(t: torch.Tensor, dim: int, world: int, rank: int, multiple: int = 1) -> torch.Tensor:
    """Rank's contiguous copy of its block of `t` along `dim`."""
    lo, hi = partition(t.shape[dim], world, rank, multiple)
    return t.narrow(dim, lo, hi - lo).contiguous()


def balance_by_length(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Longest-first greedy assignment of sequences to ranks, so every rank decodes about the
    same number of cached tokens.  Returns the sequence indices of each rank (each list sorted)."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(x) for x in out]


def _world(group=None) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def _bits(t: torch.Tensor) -> torch.Tensor:
    """Collectives move bytes; 8-bit float and bf16 tensors are sent as integer views so every
    backend (gloo included) accepts them."""
    if t.dtype in (torch.float32, torch.int32, torch.int64, torch.uint8):
        return t
    return t.view(torch.uint8)


class ShardedOutput:
    """One output tensor of logical shape `full_shape`, split along `dim` over the ranks of `group`.

    blocks along `dim` come from `partition(full_shape[dim], world, r, multiple)`, or - with
    `index_lists` (dim 0 only) - rank r owns the rows `index_lists[r]`, as `balance_by_length` gives.
    """

    def __init__(self, full_shape: Sequence[int], dim: int, dtype: torch.dtype, device, multiple: int = 1,
                 index_lists: Optional[List[List[int]]] = None, group=None):
        self.group = group
        self.world, self.rank = _world(group)
        self.full_shape = tuple(int(s) for s in full_shape)
        self.dim = dim % len(self.full_shape)
        self.dtype, self.device = dtype, torch.device(device)
        self.index_lists = index_lists
        if index_lists is not None:
            if self.dim != 0 or len(index_lists) != self.world:
                raise ValueError("index lists split dim 0 and need one list per rank")
            self.sizes = [len(lst) for lst in index_lists]
            self.spans = None
        else:
            self.spans = [partition(self.full_shape[self.dim], self.world, r, multiple) for r in range(self.world)]
            self.sizes = [hi - lo for lo, hi in self.spans]
        self.slot_units = max(self.sizes) if self.sizes else 0
        self._slot_shape = self._shape_with(self.slot_units)
        # rank-major receive buffer: slot r holds rank r's block, padded to the largest block
        self.recv = torch.empty((self.world,) + self._slot_shape, dtype=dtype, device=self.device)
        self._gloo_send = None
        self._inverse = None

    def _shape_with(self, units: int) -> Tuple[int, ...]:
        s = list(self.full_shape)
        s[self.dim] = units
        return tuple(s)

    @property
    def local(self) -> torch.Tensor:
        """This rank's block, contiguous, inside the receive buffer: the kernel writes its output here."""
        n = self.sizes[self.rank]
        slot = self.recv[self.rank]
        if n == self.slot_units:
            return slot
        if self.dim == 0:
            return slot[:n]
        # a smaller block of an inner dimension is not contiguous inside its padded slot: give a
        # contiguous prefix of the slot's memory with the block's own shape
        return slot.reshape(-1)[: n * (slot.numel() // max(self.slot_units, 1))].view(self._shape_with(n))

    def gather(self) -> torch.Tensor:
        """ONE all-gather of every rank's slot; returns the rank-major buffer [world, *slot]."""
        if self.world == 1:
            return self.recv
        backend = dist.get_backend(self.group)
        flat = _bits(self.recv).view(self.world, -1)
        if backend == "nccl":
            # in place: the send buffer is this rank's slot of the receive buffer
            dist.all_gather_into_tensor(flat, flat[self.rank], group=self.group)
        else:
            parts = list(flat.unbind(0))
            dist.all_gather(parts, flat[self.rank].clone(), group=self.group)
        return self.recv

    def block(self, r: int) -> torch.Tensor:
        """Rank r's gathered block with its true shape (zero-copy view)."""
        n = self.sizes[r]
        slot = self.recv[r]
        if n == self.slot_units:
            return slot
        if self.dim == 0:
            return slot[:n]
        return slot.reshape(-1)[: n * (slot.numel() // max(self.slot_units, 1))].view(self._shape_with(n))

    def full_view(self) -> Optional[torch.Tensor]:
        """The gathered tensor in its final layout WITHOUT a copy, when the rank-major buffer already is that
        layout (contiguous blocks of dim 0, equal sizes); None otherwise (use `split_view` or `assemble`)."""
        if self.index_lists is None and self.dim == 0 and len(set(self.sizes)) == 1:
            return self.recv.view(self.full_shape)
        return None

    def split_view(self) -> torch.Tensor:
        """Zero-copy strided view with the split dimension opened as (world, block): shape
        full_shape[:dim] + (world, block) + full_shape[dim+1:].  Equal blocks only."""
        if self.index_lists is not None or len(set(self.sizes)) != 1:
            raise ValueError("split_view needs equal contiguous blocks")
        return self.recv.movedim(0, self.dim)

    def assemble(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The gathered tensor in its final layout: a view when possible, else one strided copy per rank
        (heads / columns) or one row gather (index lists) into `out`."""
        v = self.full_view()
        if v is not None and out is None:
            return v
        if out is None:
            out = torch.empty(self.full_shape, dtype=self.dtype, device=self.device)
        on_gpu = out.is_cuda
        if self.index_lists is not None:
            if self._inverse is None:
                inv = torch.empty(self.full_shape[0], dtype=torch.int32)
                for r, lst in enumerate(self.index_lists):
                    for pos, i in enumerate(lst):
                        inv[i] = r * self.slot_units + pos
                self._inverse = inv.to(self.device)
            rows = self.recv.view(self.world * self.slot_units, -1)
            if on_gpu:
                from . import ops
                ops.gather_rows(rows, self._inverse, out.view(self.full_shape[0], -1))
            else:
                out.view(self.full_shape[0], -1).copy_(rows[self._inverse.long()])
            return out
        outer = 1
        for s in self.full_shape[:self.dim]:
            outer *= s
        inner = 1
        for s in self.full_shape[self.dim + 1:]:
            inner *= s
        dst2 = out.view(outer, self.full_shape[self.dim] * inner)
        for r, (lo, hi) in enumerate(self.spans):
            if hi == lo:
                continue
            src = self.block(r).reshape(outer, (hi - lo) * inner)
            dst = dst2[:, lo * inner:hi * inner]
            if on_gpu and src.dtype in (torch.float32, torch.float16, torch.bfloat16, torch.int32):
                from . import ops
                ops.copy2d(src, dst)
            else:
                dst.copy_(src)
        return out


# ------------------------------------------------------------------------------- conveniences
def all_gather_cat(local: torch.Tensor, dim: int = 0, group=None, multiple: int = 1, total: Optional[int] = None) -> torch.Tensor:
    """Concatenate every rank's block along `dim`, for blocks cut by `partition(total, world, r, multiple)`
    (`total` defaults to world x this block for equal blocks).  One-shot form of `ShardedOutput`; code on
    a hot path builds the `ShardedOutput` once and lets its kernel write into `.local`."""
    world, rank = _world(group)
    if world == 1:
        return local
    if total is None:
        t = torch.tensor([local.shape[dim]], dtype=torch.int64, device=local.device)
        dist.all_reduce(t, group=group)                   # the only size exchange, and only in this convenience form
        total = int(t.item())
    full = list(local.shape)
    full[dim] = total
    so = ShardedOutput(full, dim, local.dtype, local.device, multiple=multiple, group=group)
    if tuple(so.local.shape) != tuple(local.shape):
        raise ValueError(f"rank {rank}: block {tuple(local.shape)} is not partition({total}, {world}, {rank}, {multiple}) along dim {dim}")
    so.local.copy_(local)
    so.gather()
    return so.assemble()


def all_gather_rows_by_index(local: torch.Tensor, index_lists: List[List[int]], group=None) -> torch.Tensor:
    """Inverse of an index-list split along dim 0 (e.g. `balance_by_length`): every rank ends with
    all rows in their original order."""
    world, rank = _world(group)
    n = sum(len(x) for x in index_lists)
    so = ShardedOutput((n,) + tuple(local.shape[1:]), 0, local.dtype, local.device, index_lists=index_lists, group=group)
    so.local.copy_(local)
    so.gather()
    return so.assemble()
