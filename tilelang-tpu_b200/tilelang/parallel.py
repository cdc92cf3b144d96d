"""Single-node multi-GPU sharding of the operator path.

The reference has no distributed code at all (one TPU core, `core_num = 1` in
src/tl_templates/tpu/kernel_template.cpp:33-43).  Every operator of the path is made of
independent units, so the work is split without any collective on the data path and the outputs
are assembled with ONE all-gather at the end (NCCL over NVLink on GPUs, gloo in the CPU tests):

    rows     RMSNorm / RoPE / SwiGLU / row reductions / top-k : contiguous row blocks
    heads    FlashAttention                                   : head blocks of bshd tensors
    columns  GEMM                                             : N-column blocks of B and C
    batch    MLA decode                                       : sequences, balanced by length

One process per GPU; kernels only ever read the local GPU's memory.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

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


def all_gather_cat(local: torch.Tensor, dim: int = 0, group=None) -> torch.Tensor:
    """Concatenate every rank's block along `dim` (blocks may differ in size along `dim`)."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    sizes = [torch.zeros(1, dtype=torch.int64, device=local.device) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([local.shape[dim]], dtype=torch.int64, device=local.device), group=group)
    sizes = [int(s.item()) for s in sizes]
    moved = local.movedim(dim, 0).contiguous()
    biggest = max(sizes)
    if moved.shape[0] < biggest:                 # uneven blocks travel padded to the largest one
        pad = torch.zeros((biggest - moved.shape[0],) + tuple(moved.shape[1:]), dtype=local.dtype, device=local.device)
        moved = torch.cat([moved, pad], dim=0)
    parts = [torch.empty_like(moved) for _ in range(world)]
    dist.all_gather([_bits(p) for p in parts], _bits(moved), group=group)
    out = torch.cat([p[:s] for p, s in zip(parts, sizes)], dim=0)
    return out.movedim(0, dim)


def all_gather_rows_by_index(local: torch.Tensor, index_lists: List[List[int]], group=None) -> torch.Tensor:
    """Inverse of an index-list split along dim 0 (e.g. `balance_by_length`): every rank ends with
    all rows in their original order."""
    cat = all_gather_cat(local, 0, group)
    flat = [i for lst in index_lists for i in lst]
    out = torch.empty_like(cat)
    out[torch.tensor(flat, dtype=torch.long, device=cat.device)] = cat
    return out


def _bits(t: torch.Tensor) -> torch.Tensor:
    """Collectives move bytes; 8-bit float and bf16 tensors are sent as integer views so every
    backend (gloo included) accepts them."""
    if t.dtype in (torch.float32, torch.int32, torch.int64, torch.uint8):
        return t
    return t.view(torch.uint8)
