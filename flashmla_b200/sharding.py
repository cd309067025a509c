"""Host-side sharding of the sparse MLA path over the GPUs of one node.

Decode is partitioned by batch: a rank owns a contiguous slice of the requests together with the KV
pages those requests reference, renumbered into a rank-local pool (sparse decode: through the index lists; dense
decode: through the block table).  Prefill is partitioned by query token; the bf16 KV is replicated.  There is no collective inside the kernels; results are simply
concatenated in rank order.
"""
from __future__ import annotations

from typing import Tuple

import torch


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [lo, hi) slice of n units for `rank` of `world` (first n % world ranks get one more)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_decode_inputs(q: torch.Tensor, kv_rows: torch.Tensor, indices: torch.Tensor, world: int, rank: int):
    """Slice of a decode problem owned by `rank`.

    q (b, s_q, h_q, 576), kv_rows (num_blocks, page, 1, 656) bytes, indices (b, s_q, topk) in-cache rows
    (-1 invalid).  Returns (q_local, kv_local, indices_local, (lo, hi)) where kv_local holds only the
    pages the slice references and indices_local addresses that local pool.
    """
    lo, hi = shard_bounds(q.shape[0], world, rank)
    page = kv_rows.shape[1]
    idx = indices[lo:hi]
    valid = idx >= 0
    pages = torch.unique(torch.div(idx[valid], page, rounding_mode="floor"))
    if pages.numel() == 0:
        pages = torch.zeros(1, dtype=idx.dtype, device=idx.device)
    remap = torch.full((kv_rows.shape[0],), -1, dtype=torch.int64, device=idx.device)
    remap[pages.long()] = torch.arange(pages.numel(), device=idx.device)
    safe = idx.clamp_min(0).long()
    local = remap[safe // page] * page + safe % page
    local = torch.where(valid, local, torch.full_like(local, -1)).to(torch.int32)
    return q[lo:hi], kv_rows[pages.long()].contiguous(), local, (lo, hi)


def shard_dense_decode_inputs(q: torch.Tensor, k_cache: torch.Tensor, block_table: torch.Tensor, cache_seqlens: torch.Tensor,
                              world: int, rank: int):
    """Slice of a dense decode problem owned by `rank`.

    q (b, s_q, h_q, 576), k_cache (num_blocks, page, h_kv, 576) bf16, block_table (b, max_blocks) int32,
    cache_seqlens (b,) int32.  Returns (q_local, cache_local, block_table_local, cache_seqlens_local, (lo, hi)):
    cache_local holds only the blocks that the slice's requests reach within their lengths, and the local block
    table addresses it; entries beyond a request's length (never read) become 0.
    """
    lo, hi = shard_bounds(q.shape[0], world, rank)
    page = k_cache.shape[1]
    bt, lens = block_table[lo:hi], cache_seqlens[lo:hi]
    used = torch.arange(bt.shape[1], device=bt.device).view(1, -1) * page < lens.view(-1, 1)      # pages a request reaches
    blocks = torch.unique(bt[used])
    if blocks.numel() == 0:
        blocks = torch.zeros(1, dtype=bt.dtype, device=bt.device)
    remap = torch.zeros((k_cache.shape[0],), dtype=torch.int64, device=bt.device)
    remap[blocks.long()] = torch.arange(blocks.numel(), device=bt.device)
    local = torch.where(used, remap[bt.clamp(0, k_cache.shape[0] - 1).long()], torch.zeros_like(bt, dtype=torch.int64)).to(torch.int32)
    return q[lo:hi], k_cache[blocks.long()].contiguous(), local, lens, (lo, hi)


def shard_prefill_inputs(q: torch.Tensor, indices: torch.Tensor, world: int, rank: int):
    """Query-token slice [lo, hi) of a prefill problem; kv stays whole on every rank."""
    lo, hi = shard_bounds(q.shape[0], world, rank)
    return q[lo:hi], indices[lo:hi], (lo, hi)
