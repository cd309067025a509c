"""KV-cache row formats of the sparse decode path, restated on the CPU (test infrastructure).

Two 656-byte-per-token formats, both for d_qk = 576 (512 "NoPE" + 64 "RoPE" dims):

``V32``  (reference: tests/quant.py:35-53 quantise, :93-104 dequantise;
          flash_mla/flash_mla_interface.py:94-98 layout)
    bytes [0,512)    512 x float8_e4m3fn, the quantised NoPE part
    bytes [512,528)  4 x float32 scales, scale k covers elements [128k, 128k+128)
    bytes [528,656)  64 x bfloat16, the RoPE part, unquantised

``MXFP8``  (not in the reference; layout defined here)
    bytes [0,512)    512 x float8_e4m3fn
    bytes [512,528)  16 x e8m0 scale bytes (value 2**(byte-127)), byte k covers
                     elements [32k, 32k+32)
    bytes [528,656)  64 x bfloat16 RoPE

``MODEL1``  (reference: tests/quant.py:55-75 quantise, :106-118 dequantise) for d_qk = 512 (448 NoPE + 64 RoPE),
          584 bytes per token, stored per cache block of `page` tokens as
    page x [448 x float8_e4m3fn | 64 x bfloat16]      576 bytes per token
    page x [7 x e8m0 scale bytes (one per 64 NoPE values) | 1 pad byte]
    and padded to a multiple of 576 bytes.  Dequantisation multiplies in bfloat16 (exact: e4m3 times a power of two).

The scale of a tile is the smallest power of two >= max(amax/448, 1e-4)
(reference: tests/quant.py:17-18).  Dequantisation is fp8 -> fp32, times the
scale, rounded to bfloat16.
"""
from __future__ import annotations

import torch

D_QK = 576
D_NOPE = 512
D_ROPE = 64
ROW_BYTES = 656
SCALE_OFF = 512
ROPE_OFF = 528

V32_TILE = 128
MX_TILE = 32

LAYOUT_V32 = "v32"
LAYOUT_MXFP8 = "mxfp8_e8m0_32"
LAYOUT_MODEL1 = "model1"

M1_D_QK, M1_D_NOPE, M1_TILE, M1_DATA_BYTES, M1_ROW_BYTES = 512, 448, 64, 576, 584


def pow2_scale(amax: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= max(amax/448, 1e-4), fp32 (tests/quant.py:17-18)."""
    inv = amax.float() / 448.0
    return torch.pow(2, torch.clamp_min(inv, 1e-4).log2().ceil()).float()


def _tile_scales(nope: torch.Tensor, tile: int) -> torch.Tensor:
    # nope [..., 512] -> scales [..., 512/tile]
    t = nope.reshape(*nope.shape[:-1], D_NOPE // tile, tile)
    return pow2_scale(t.abs().amax(dim=-1))


def _quantise(kv: torch.Tensor, tile: int):
    assert kv.shape[-1] == D_QK and kv.dtype == torch.bfloat16
    nope = kv[..., :D_NOPE]
    scales = _tile_scales(nope, tile)                              # [..., ntiles]
    q = (nope.float().reshape(*nope.shape[:-1], -1, tile) / scales.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q.reshape(*nope.shape), scales


def quantize_rows_model1(kv: torch.Tensor) -> torch.Tensor:
    """bf16 [num_blocks, page, 1, 512] -> uint8 [num_blocks, page, 1, 584], a view of blocks padded to a multiple of 576
    bytes and laid out as the module docstring says (tests/quant.py:55-75)."""
    nb, page, hk, d = kv.shape
    assert hk == 1 and d == M1_D_QK and kv.dtype == torch.bfloat16
    x = kv.reshape(nb, page, d)
    tiles = x[..., :M1_D_NOPE].float().reshape(nb, page, 7, M1_TILE)
    scales = pow2_scale(tiles.abs().amax(-1))                                     # [nb, page, 7]
    fp8 = (tiles / scales.unsqueeze(-1)).to(torch.float8_e4m3fn).reshape(nb, page, M1_D_NOPE)
    padded = (page * M1_ROW_BYTES + 575) // 576 * 576
    pool = torch.zeros((nb, padded), dtype=torch.uint8)
    data = pool[:, :page * M1_DATA_BYTES].view(nb, page, M1_DATA_BYTES)
    data[..., :M1_D_NOPE] = fp8.view(torch.uint8)
    data[..., M1_D_NOPE:] = x[..., M1_D_NOPE:].contiguous().view(torch.uint8).reshape(nb, page, 128)
    sc = pool[:, page * M1_DATA_BYTES:page * M1_ROW_BYTES].view(nb, page, 8)
    sc[..., :7] = (torch.log2(scales).round().to(torch.int32) + 127).to(torch.uint8)
    return pool[:, :page * M1_ROW_BYTES].view(nb, page, 1, M1_ROW_BYTES)


def dequantize_rows_model1(rows: torch.Tensor) -> torch.Tensor:
    """uint8 [num_blocks, page, 1, 584] (block-wise layout) -> bf16 [num_blocks, page, 1, 512] (tests/quant.py:106-118)."""
    nb, page, hk, nbytes = rows.shape
    assert hk == 1 and nbytes == M1_ROW_BYTES
    flat = rows.reshape(nb, page * M1_ROW_BYTES)
    data = flat[:, :page * M1_DATA_BYTES].reshape(nb, page, M1_DATA_BYTES)
    sc = flat[:, page * M1_DATA_BYTES:].reshape(nb, page, 8)[..., :7]
    scales = torch.pow(2.0, sc.float() - 127.0).to(torch.bfloat16)                 # [nb, page, 7]
    nope = data[..., :M1_D_NOPE].contiguous().view(torch.float8_e4m3fn).to(torch.bfloat16).reshape(nb, page, 7, M1_TILE)
    out = torch.empty((nb, page, M1_D_QK), dtype=torch.bfloat16)
    out[..., :M1_D_NOPE] = (nope * scales.unsqueeze(-1)).reshape(nb, page, M1_D_NOPE)
    out[..., M1_D_NOPE:] = data[..., M1_D_NOPE:].contiguous().view(torch.bfloat16)
    return out.view(nb, page, 1, M1_D_QK)


def quantize_rows(kv: torch.Tensor, layout: str = LAYOUT_V32, row_pad: int = 0) -> torch.Tensor:
    """bf16 [num_blocks, page, 1, 576] -> uint8 [num_blocks, page, 1, 656] (MODEL1: see quantize_rows_model1).

    ``row_pad`` extra rows are allocated per page (and sliced off) so that the
    block stride exceeds page*656, as the reference's fixture does with one
    spare row (tests/quant.py:37).
    """
    if layout == LAYOUT_MODEL1:
        return quantize_rows_model1(kv)
    nb, page, hk, d = kv.shape
    assert hk == 1 and d == D_QK
    kv = kv.reshape(nb, page, d)
    tile = V32_TILE if layout == LAYOUT_V32 else MX_TILE
    q, scales = _quantise(kv, tile)
    pool = torch.zeros((nb, page + row_pad, ROW_BYTES), dtype=torch.uint8)
    out = pool[:, :page]
    out[..., :D_NOPE] = q.view(torch.uint8)
    if layout == LAYOUT_V32:
        out[..., SCALE_OFF:ROPE_OFF] = scales.contiguous().view(torch.uint8).reshape(nb, page, 16)
    elif layout == LAYOUT_MXFP8:
        exp = torch.log2(scales).round().to(torch.int32) + 127
        assert int(exp.min()) >= 0 and int(exp.max()) <= 254
        out[..., SCALE_OFF:ROPE_OFF] = exp.to(torch.uint8)
    else:
        raise ValueError(layout)
    out[..., ROPE_OFF:] = kv[..., D_NOPE:].contiguous().view(torch.uint8).reshape(nb, page, 128)
    return out.view(nb, page, 1, ROW_BYTES)


def dequantize_rows(rows: torch.Tensor, layout: str = LAYOUT_V32) -> torch.Tensor:
    """uint8 [num_blocks, page, 1, 656] -> bf16 [num_blocks, page, 1, 576] (MODEL1: see dequantize_rows_model1)."""
    if layout == LAYOUT_MODEL1:
        return dequantize_rows_model1(rows)
    nb, page, hk, nbytes = rows.shape
    assert hk == 1 and nbytes == ROW_BYTES
    rows = rows.reshape(nb, page, ROW_BYTES).contiguous()
    nope = rows[..., :D_NOPE].contiguous().view(torch.float8_e4m3fn).float()
    if layout == LAYOUT_V32:
        scales = rows[..., SCALE_OFF:ROPE_OFF].contiguous().view(torch.float32)     # [nb,page,4]
        tile = V32_TILE
    elif layout == LAYOUT_MXFP8:
        scales = torch.pow(2.0, rows[..., SCALE_OFF:ROPE_OFF].float() - 127.0)       # [nb,page,16]
        tile = MX_TILE
    else:
        raise ValueError(layout)
    out = torch.empty((nb, page, D_QK), dtype=torch.bfloat16)
    out[..., :D_NOPE] = (nope.reshape(nb, page, -1, tile) * scales.unsqueeze(-1)).reshape(nb, page, D_NOPE)
    out[..., D_NOPE:] = rows[..., ROPE_OFF:].contiguous().view(torch.bfloat16)
    return out.view(nb, page, 1, D_QK)


def abs_to_cache_indices(abs_indices: torch.Tensor, block_table: torch.Tensor, page: int) -> torch.Tensor:
    """Logical token position -> in-cache row index, -1 preserved (tests/quant.py:126-158).

    abs_indices [b, s_q, topk] int32, block_table [b, max_pages] int32.
    result[i,j,k] = block_table[i, pos // page] * page + pos % page.
    """
    b = abs_indices.shape[0]
    out = torch.empty_like(abs_indices)
    for i in range(b):
        pos = abs_indices[i].to(torch.int64)
        bad = pos == -1
        pos = pos.masked_fill(bad, 0)
        pages = block_table[i].to(torch.int64)[pos // page]
        row = pages * page + pos % page
        out[i] = row.masked_fill(bad, -1).to(abs_indices.dtype)
    return out
