"""Sharding helpers for running the operators on several GPUs of one node (one process per GPU).

Every operator is independent per sequence and per KV-head group, so the data path needs no collective:
a varlen batch is split by sequence (balanced by a cost proxy), a single long sequence by KV head.  The only
exchange is at the caller's level -- gathering outputs (or gradients of shared parameters) -- for which thin
wrappers over torch.distributed are provided.  Backend "nccl" on GPUs, "gloo" in the CPU tests.
"""
from typing import List, Sequence, Tuple

import torch


def sequence_cost(length: int, kernel_stride: int = 16, block_size: int = 64, topk: int = 16) -> float:
    """Relative cost of one sequence: compressed attention is quadratic, sparse attention linear in length."""
    return length * (length / (2.0 * kernel_stride)) + length * float(topk * block_size)


def partition_sequences(seqlens: Sequence[int], world_size: int, **cost_kw) -> List[List[int]]:
    """Longest-processing-time assignment of sequence indices to ranks; every rank's list is sorted."""
    order = sorted(range(len(seqlens)), key=lambda i: -sequence_cost(int(seqlens[i]), **cost_kw))
    load = [0.0] * world_size
    parts: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (load[j], j))
        parts[r].append(i)
        load[r] += sequence_cost(int(seqlens[i]), **cost_kw)
    return [sorted(p) for p in parts]


def shard_varlen(x: torch.Tensor, cu_seqlens: torch.Tensor, seq_ids: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows of the sequences `seq_ids` (in that order) and their re-based cu_seqlens (int32, on x's device)."""
    cu = cu_seqlens.tolist()
    pieces = [x[cu[i]:cu[i + 1]] for i in seq_ids]
    lens = [cu[i + 1] - cu[i] for i in seq_ids]
    out = torch.cat(pieces, 0) if pieces else x[:0]
    new_cu = torch.zeros(len(lens) + 1, dtype=torch.int32, device=cu_seqlens.device)
    if lens:
        new_cu[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int32, device=cu_seqlens.device), 0)
    return out, new_cu


def unshard_varlen(pieces: List[torch.Tensor], parts: List[List[int]], cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Inverse of shard_varlen over all ranks: pieces[r] holds rank r's sequences in parts[r] order."""
    cu = cu_seqlens.tolist()
    total = cu[-1]
    ref = next(p for p in pieces if p is not None)
    out = ref.new_empty((total,) + tuple(ref.shape[1:]))
    for r, ids in enumerate(parts):
        off = 0
        for i in ids:
            L = cu[i + 1] - cu[i]
            out[cu[i]:cu[i + 1]] = pieces[r][off:off + L]
            off += L
    return out


def kv_head_range(rank: int, world_size: int, num_kv_heads: int) -> Tuple[int, int]:
    """[begin, end) KV heads of a rank when one sequence is split by KV-head group (world_size <= num_kv_heads)."""
    if num_kv_heads % world_size:
        raise ValueError("num_kv_heads must be a multiple of the world size for head sharding")
    per = num_kv_heads // world_size
    return rank * per, (rank + 1) * per


def _all_gather_rows(gathered: torch.Tensor, local: torch.Tensor, group) -> None:
    """gathered[r] = rank r's `local`, in one collective where the backend has one (NCCL); the gloo backend of the CPU tests
    takes the list form over views of the same buffer."""
    import torch.distributed as dist

    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(gathered, local, group=group)
    else:
        dist.all_gather(list(gathered.unbind(0)), local, group=group)


def gather_varlen(local: torch.Tensor, parts: List[List[int]], cu_seqlens: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather the per-rank outputs of a sequence-sharded operator back into the original token order."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    cu = cu_seqlens.tolist()
    sizes = [sum(cu[i + 1] - cu[i] for i in ids) for ids in parts]
    mx = max(sizes) if sizes else 0
    if local.shape[0] == mx:
        pad = local.contiguous()
    else:
        pad = local.new_zeros((mx,) + tuple(local.shape[1:]))
        pad[: local.shape[0]] = local
    # one collective into one buffer [world, mx, ...]: NCCL lands every rank's rows in local memory, then they are put in
    # token order (a rank's sequences are not contiguous in the original batch)
    gathered = local.new_empty((world, mx) + tuple(local.shape[1:]))
    _all_gather_rows(gathered, pad, group)
    return unshard_varlen([gathered[r, :s] for r, s in enumerate(sizes)], parts, cu_seqlens)


def gather_heads(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather head-sharded outputs [tokens, heads_local, d] along the head dimension."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    local = local.contiguous()
    gathered = local.new_empty((world,) + tuple(local.shape))
    _all_gather_rows(gathered, local, group)
    # [world, tokens, heads_local, d] -> [tokens, world * heads_local, d]
    return gathered.permute(1, 0, 2, 3).reshape(local.shape[0], world * local.shape[1], local.shape[2])
