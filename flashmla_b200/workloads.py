"""Seeded synthetic workloads for the sparse MLA path: paged KV pools, index lists, queries.

Plain torch, device-agnostic (runs on the CPU for tests and on the GPU for the
benchmark).  The shapes and value distributions follow the five benchmark
configurations: bf16 N(0,1) queries and latent KV, KV quantised to 656-byte rows,
a randomly permuted page table, distinct uniform-random token positions per
query with a fraction replaced by -1.

Row formats (d_qk = 576 = 512 NoPE + 64 RoPE):
  "v32"            512 e4m3 | 4 fp32 scales (one per 128 elements) | 64 bf16
                   (flash_mla/flash_mla_interface.py:94-98 of the reference)
  "mxfp8_e8m0_32"  512 e4m3 | 16 e8m0 scale bytes (one per 32 elements) | 64 bf16
Scales are the smallest power of two >= max(amax/448, 1e-4).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

D_QK, D_NOPE, D_V, ROW_BYTES = 576, 512, 512, 656
LAYOUT_V32 = "v32"
LAYOUT_MXFP8 = "mxfp8_e8m0_32"
LAYOUT_MODEL1 = "model1"      # d_qk = 512: 448 e4m3 + 64 bf16 per token, 7 e8m0 scales per 64, stored block-wise (584 bytes per token)


def quantize_kv_rows(kv: torch.Tensor, layout: str = LAYOUT_V32, row_pad: int = 0) -> torch.Tensor:
    """bf16 [num_blocks, page, 1, 576] -> uint8 [num_blocks, page, 1, 656] (block stride (page+row_pad)*656)."""
    nb, page, hk, d = kv.shape
    if layout == LAYOUT_MODEL1:
        # [nb, page, 1, 512] -> [nb, page, 1, 584] viewing blocks [page x (448 e4m3 | 64 bf16)] [page x (7 e8m0 | pad)],
        # padded to a multiple of 576 bytes like the reference's fixture (tests/quant.py:55-75)
        assert hk == 1 and d == 512 and kv.dtype == torch.bfloat16 and row_pad == 0
        x = kv.view(nb, page, d)
        tiles = x[..., :448].float().view(nb, page, 7, 64)
        scale = torch.exp2(torch.ceil(torch.log2((tiles.abs().amax(-1) / 448.0).clamp_min(1e-4))))
        fp8 = (tiles / scale.unsqueeze(-1)).to(torch.float8_e4m3fn).view(nb, page, 448)
        pool = torch.zeros((nb, (page * 584 + 575) // 576 * 576), dtype=torch.uint8, device=kv.device)
        data = pool[:, :page * 576].view(nb, page, 576)
        data[..., :448] = fp8.view(torch.uint8)
        data[..., 448:] = x[..., 448:].contiguous().view(torch.uint8).view(nb, page, 128)
        pool[:, page * 576:page * 584].view(nb, page, 8)[..., :7] = (torch.log2(scale).round().to(torch.int32) + 127).to(torch.uint8)
        return pool[:, :page * 584].view(nb, page, 1, 584)
    assert hk == 1 and d == D_QK and kv.dtype == torch.bfloat16
    tile = 128 if layout == LAYOUT_V32 else 32
    x = kv.view(nb, page, d)
    nope = x[..., :D_NOPE].float().view(nb, page, D_NOPE // tile, tile)
    inv = nope.abs().amax(-1) / 448.0
    scale = torch.exp2(torch.ceil(torch.log2(inv.clamp_min(1e-4))))
    fp8 = (nope / scale.unsqueeze(-1)).to(torch.float8_e4m3fn).view(nb, page, D_NOPE)
    pool = torch.zeros((nb, page + row_pad, ROW_BYTES), dtype=torch.uint8, device=kv.device)
    rows = pool[:, :page]
    rows[..., :512] = fp8.view(torch.uint8)
    if layout == LAYOUT_V32:
        rows[..., 512:528] = scale.contiguous().view(torch.uint8).view(nb, page, 16)
    elif layout == LAYOUT_MXFP8:
        rows[..., 512:528] = (torch.log2(scale).round().to(torch.int32) + 127).to(torch.uint8)
    else:
        raise ValueError(f"unknown KV row layout {layout!r}")
    rows[..., 528:] = x[..., D_NOPE:].contiguous().view(torch.uint8).view(nb, page, 128)
    return rows.view(nb, page, 1, ROW_BYTES)


def distinct_positions(limits: torch.Tensor, count: int, gen: torch.Generator, pad: int = -1) -> torch.Tensor:
    """[rows] limits -> [rows, count] int32: distinct uniform positions in [0, limit), padded with ``pad``."""
    rows = limits.numel()
    width = max(int(limits.max().item()) if rows else 0, count)
    out = torch.empty((rows, count), dtype=torch.int32, device=limits.device)
    step = max(1, (1 << 24) // max(width, 1))
    col = torch.arange(width, device=limits.device).unsqueeze(0)
    for lo in range(0, rows, step):
        hi = min(rows, lo + step)
        r = torch.rand((hi - lo, width), generator=gen, device=limits.device)
        lim = limits[lo:hi].to(torch.int64).unsqueeze(1)
        r.masked_fill_(col >= lim, -1.0)
        pick = r.topk(count, dim=-1, sorted=True).indices
        pick = pick.masked_fill(pick >= lim, pad)
        out[lo:hi] = pick.to(torch.int32)
    return out


def positions_to_cache_rows(positions: torch.Tensor, block_table: torch.Tensor, page: int) -> torch.Tensor:
    """Logical positions [b, s_q, topk] -> in-cache row indices; -1 stays -1."""
    b = positions.shape[0]
    pos = positions.to(torch.int64)
    bad = pos < 0
    pos = pos.clamp_min(0)
    pages = torch.gather(block_table.to(torch.int64), 1, (pos // page).view(b, -1)).view_as(pos)
    return (pages * page + pos % page).masked_fill(bad, -1).to(torch.int32)


@dataclasses.dataclass
class DecodeWorkload:
    q: torch.Tensor                 # [b, s_q, h_q, 576] bf16
    kv_rows: torch.Tensor           # [num_blocks, page, 1, 656] uint8
    kv_bf16: Optional[torch.Tensor]  # [num_blocks, page, 1, 576] bf16 source (None when dropped to save memory)
    block_table: torch.Tensor       # [b, max_pages] int32
    cache_seqlens: torch.Tensor     # [b] int32
    positions: torch.Tensor         # [b, s_q, topk] int32 logical positions (-1 invalid)
    indices: torch.Tensor           # [b, s_q, topk] int32 in-cache rows (-1 invalid)
    sm_scale: float
    layout: str
    attn_sink: Optional[torch.Tensor] = None
    topk_length: Optional[torch.Tensor] = None

    @property
    def flops(self) -> float:
        b, s_q, h_q, d = self.q.shape
        return 2.0 * h_q * b * s_q * self.indices.shape[-1] * (d + D_V)

    @property
    def algorithmic_bytes(self) -> float:
        b, s_q, h_q, d = self.q.shape
        uniq = int(torch.unique(self.indices).numel()) - int(bool((self.indices < 0).any()))
        return 2.0 * b * s_q * h_q * d + self.kv_rows.shape[-1] * uniq + 2.0 * b * s_q * h_q * D_V


def make_decode_workload(
    b: int, s_q: int, h_q: int, topk: int, seqlen_lo: int, seqlen_hi: int, *,
    page: int = 64, layout: str = LAYOUT_V32, seed: int = 0, device: str = "cpu",
    invalid_frac: float = 0.0, invalid_tail: int = 0, row_pad: int = 0,
    q_std: float = 1.0, kv_std: float = 1.0, clamp: Optional[float] = None,
    with_sink: bool = False, with_topk_length: bool = False, poison_unused: bool = False,
    keep_bf16: bool = True, sm_scale: Optional[float] = None,
) -> DecodeWorkload:
    """Builds one decode problem.  seqlens uniform in [seqlen_lo, seqlen_hi]; pages randomly permuted."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    seqlens = torch.randint(seqlen_lo, seqlen_hi + 1, (b,), generator=gen, device=device, dtype=torch.int32)
    pages_per_seq = max((int(seqlens.max().item()) + page - 1) // page, 1)
    n_pages = b * pages_per_seq
    block_table = torch.randperm(n_pages, generator=gen, device=device).to(torch.int32).view(b, pages_per_seq)

    d_qk = 512 if layout == LAYOUT_MODEL1 else D_QK
    q = (torch.randn((b, s_q, h_q, d_qk), generator=gen, device=device) * q_std)
    if clamp is not None:
        q.clamp_(-clamp, clamp)
    q = q.to(torch.bfloat16)
    # A large pool whose bf16 source nobody needs is generated and quantised page chunk by page chunk, so that the
    # fp32 temporaries stay small (the 11 GB pool of the MXFP8 configuration would otherwise need ~100 GB of them).
    chunked = not keep_bf16 and not poison_unused and n_pages * page * D_QK > (1 << 28) and layout != LAYOUT_MODEL1
    kv = None
    if chunked:
        kv_rows = torch.empty((n_pages, page + row_pad, 1, ROW_BYTES), dtype=torch.uint8, device=device)[:, :page]
        step = max(1, (1 << 26) // (page * D_QK))
        for lo in range(0, n_pages, step):
            part = torch.randn((min(step, n_pages - lo), page, 1, D_QK), generator=gen, device=device) * kv_std
            if clamp is not None:
                part.clamp_(-clamp, clamp)
            kv_rows[lo:lo + part.shape[0]] = quantize_kv_rows(part.to(torch.bfloat16), layout)
    else:
        kv = (torch.randn((n_pages, page, 1, d_qk), generator=gen, device=device) * kv_std)
        if clamp is not None:
            kv.clamp_(-clamp, clamp)
        kv = kv.to(torch.bfloat16)

    positions = distinct_positions(seqlens.repeat_interleave(s_q), topk, gen).view(b, s_q, topk)
    if invalid_tail:
        positions[..., topk - invalid_tail:] = -1
    if invalid_frac > 0:
        positions.masked_fill_(torch.rand(positions.shape, generator=gen, device=device) < invalid_frac, -1)
    indices = positions_to_cache_rows(positions, block_table, page)

    topk_length = None
    if with_topk_length:
        topk_length = torch.randint(0, topk + 1, (b,), generator=gen, device=device, dtype=torch.int32)
    attn_sink = None
    if with_sink:
        attn_sink = torch.randn((h_q,), generator=gen, device=device)
        sel = torch.randn((h_q,), generator=gen, device=device)
        attn_sink[sel > 0.5] = float("inf")
        attn_sink[sel < -0.5] = float("-inf")

    if poison_unused:
        used = indices
        if topk_length is not None:
            beyond = torch.arange(topk, device=device).view(1, 1, topk) >= topk_length.view(b, 1, 1)
            used = indices.masked_fill(beyond, -1)
        keep = torch.zeros(n_pages * page, dtype=torch.bool, device=device)
        keep[used[used >= 0].to(torch.int64)] = True
        kv.view(-1, d_qk)[~keep] = float("nan")

    if not chunked:
        kv_rows = quantize_kv_rows(kv, layout, row_pad=row_pad)
    return DecodeWorkload(
        q=q, kv_rows=kv_rows, kv_bf16=kv if keep_bf16 else None, block_table=block_table,
        cache_seqlens=seqlens, positions=positions, indices=indices,
        sm_scale=float(d_qk ** -0.5) if sm_scale is None else sm_scale, layout=layout,
        attn_sink=attn_sink, topk_length=topk_length)


@dataclasses.dataclass
class PrefillWorkload:
    q: torch.Tensor          # [s_q, h_q, 576] bf16
    kv: torch.Tensor         # [s_kv, 1, 576] bf16
    indices: torch.Tensor    # [s_q, 1, topk] int32
    dout: torch.Tensor       # [s_q, h_q, 512] bf16
    sm_scale: float
    attn_sink: Optional[torch.Tensor] = None
    topk_length: Optional[torch.Tensor] = None

    @property
    def fwd_flops(self) -> float:
        s_q, h_q, d = self.q.shape
        return 2.0 * s_q * self.indices.shape[-1] * h_q * (d + D_V)

    @property
    def bwd_flops(self) -> float:
        s_q, h_q, d = self.q.shape
        return 2.0 * s_q * self.indices.shape[-1] * h_q * (3 * d + 2 * D_V)


def make_prefill_workload(
    s_q: int, s_kv: int, h_q: int, topk: int, *, seed: int = 0, device: str = "cpu",
    causal_offset: Optional[int] = None, std: float = 1.0, sm_scale: Optional[float] = None,
    invalid_pads=(-1,), with_sink: bool = False, with_topk_length: bool = False, d_qk: int = D_QK,
) -> PrefillWorkload:
    """Query i draws ``topk`` distinct positions from [0, causal_offset+i] (or [0, s_kv) when no offset), padded with invalid values."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    q = (torch.randn((s_q, h_q, d_qk), generator=gen, device=device) * std).to(torch.bfloat16)
    kv = (torch.randn((s_kv, 1, d_qk), generator=gen, device=device) * std).to(torch.bfloat16)
    dout = (torch.randn((s_q, h_q, D_V), generator=gen, device=device) * std).to(torch.bfloat16)
    if causal_offset is None:
        limits = torch.full((s_q,), s_kv, dtype=torch.int32, device=device)
    else:
        limits = (torch.arange(s_q, device=device, dtype=torch.int32) + causal_offset + 1).clamp_max(s_kv)
    idx = distinct_positions(limits, topk, gen, pad=-1)
    if len(invalid_pads) > 1 or invalid_pads[0] != -1:
        pads = torch.tensor(list(invalid_pads), dtype=torch.int32, device=device)
        fill = pads[torch.randint(0, len(invalid_pads), idx.shape, generator=gen, device=device)]
        idx = torch.where(idx < 0, fill, idx)
    attn_sink = None
    if with_sink:
        attn_sink = torch.randn((h_q,), generator=gen, device=device)
        sel = torch.randn((h_q,), generator=gen, device=device)
        attn_sink[sel > 0.5] = float("inf")
        attn_sink[sel < -0.5] = float("-inf")
    topk_length = None
    if with_topk_length:
        topk_length = torch.randint(0, topk + 1, (s_q,), generator=gen, device=device, dtype=torch.int32)
    return PrefillWorkload(q=q, kv=kv, indices=idx.view(s_q, 1, topk), dout=dout,
                           sm_scale=float(d_qk ** -0.5) if sm_scale is None else sm_scale,
                           attn_sink=attn_sink, topk_length=topk_length)
