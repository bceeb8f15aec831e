"""Sharding of a decode batch over the GPUs of one box. Requests are independent (a request's pages, block-table row
and output rows live on one GPU), so the batch is partitioned by request with no collective on the hot path; the only
communication is an optional gather of the outputs for validation.

`partition_requests` balances the FP4 cache bytes each rank must stream (L_b * KVH * D * 1.125): longest-processing-time
greedy, deterministic for equal inputs on every rank."""
from typing import List, Sequence


def kv_bytes(seq_len: int, KVH: int, D: int) -> int:
    """FP4 cache bytes one decode step reads for a request: K and V codes plus block scales"""
    return seq_len * KVH * (D + D // 8)


def partition_requests(seq_lens: Sequence[int], n_ranks: int) -> List[List[int]]:
    """request indices per rank, balanced by cached tokens; ties broken by request index"""
    if n_ranks < 1:
        raise ValueError("n_ranks must be >= 1")
    order = sorted(range(len(seq_lens)), key=lambda i: (-int(seq_lens[i]), i))
    load = [0] * n_ranks
    shards: List[List[int]] = [[] for _ in range(n_ranks)]
    for i in order:
        r = min(range(n_ranks), key=lambda k: (load[k], k))
        shards[r].append(i)
        load[r] += int(seq_lens[i])
    for s in shards:
        s.sort()
    return shards


def gather_outputs(local_out, local_rows, n_total, group=None):
    """validation only: all-gather the per-rank output rows (padded to the largest shard) and scatter them back into
    request order. local_out (n_local, ...) tensor, local_rows the request index of each local row."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    n_local = torch.tensor([local_out.shape[0]], device=local_out.device)
    sizes = [torch.zeros_like(n_local) for _ in range(world)]
    dist.all_gather(sizes, n_local, group=group)
    mx = int(max(int(s) for s in sizes))
    pad = torch.zeros((mx, *local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    pad[:local_out.shape[0]] = local_out
    idx = torch.full((mx,), -1, dtype=torch.int64, device=local_out.device)
    idx[:len(local_rows)] = torch.as_tensor(local_rows, dtype=torch.int64, device=local_out.device)
    outs = [torch.empty_like(pad) for _ in range(world)]
    idxs = [torch.empty_like(idx) for _ in range(world)]
    dist.all_gather(outs, pad, group=group)
    dist.all_gather(idxs, idx, group=group)
    full = torch.zeros((n_total, *local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    for o, ix in zip(outs, idxs):
        m = ix >= 0
        full[ix[m]] = o[m]
    return full
