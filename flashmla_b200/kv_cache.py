"""Writing the paged KV cache on the GPU: the two helpers that sit in front of the sparse decode path.

``quantize_k_cache`` and ``abs_indices2indices_in_kvcache`` carry the names and argument meaning of the
reference's torch fixtures (tests/quant.py:20-78 and :126-158), which is all the reference offers for these
steps; here they are CUDA kernels behind the C ABI (``fmla_kv_quantize``, ``fmla_cache_indices``).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .interface import D_QK, ROW_BYTES, M1_D_QK, M1_ROW_BYTES, _LAYOUTS, _require_cuda, _stream


def quantize_k_cache(kv: torch.Tensor, kvcache_layout: Optional[str] = None, *, out: Optional[torch.Tensor] = None,
                     row_pad: int = 0) -> torch.Tensor:
    """bf16 (num_blocks, page_block_size, 1, 576) -> bytes (num_blocks, page_block_size, 1, 656), or with the
    "model1" layout bf16 (.., 512) -> bytes (num_blocks, page_block_size, 1, 584) laid out block-wise.

    ``kvcache_layout``: "v32" (default for 576 values per row; 4 fp32 scales per row), "mxfp8_e8m0_32" (16 e8m0 scale
    bytes per row) or "model1" (default for 512 values per row; tests/quant.py:55-75 of the reference: a block is
    [page x (448 e4m3 | 64 bf16)] followed by [page x (7 e8m0 | pad)], padded to a multiple of 576 bytes).
    ``row_pad`` spare rows per block make the block stride exceed page_block_size*656, as the reference's fixture
    does; ``out`` reuses an existing pool of the right shape.
    """
    _require_cuda(kv, "kv")
    if kvcache_layout is None and kv.dim() == 4 and kv.shape[3] == M1_D_QK:
        kvcache_layout = "model1"
    if kvcache_layout not in _LAYOUTS:
        raise ValueError(f"kvcache_layout must be one of {[k for k in _LAYOUTS if k]}, got {kvcache_layout!r}")
    m1 = _LAYOUTS[kvcache_layout] == _lib.LAYOUT_MODEL1
    d, row = (M1_D_QK, M1_ROW_BYTES) if m1 else (D_QK, ROW_BYTES)
    if kv.dim() != 4 or kv.shape[2] != 1 or kv.shape[3] != d or kv.dtype != torch.bfloat16:
        raise RuntimeError(f"kv must be bfloat16 of shape (num_blocks, page_block_size, 1, {d})")
    nb, page = kv.shape[0], kv.shape[1]
    kv = kv.contiguous()
    if out is None:
        if m1:
            padded = (page * row + 575) // 576 * 576
            pool = torch.zeros((nb, padded), dtype=torch.uint8, device=kv.device)
            out = pool[:, :page * row].view(nb, page, 1, row)
        else:
            pool = torch.zeros((nb, page + row_pad, 1, row), dtype=torch.uint8, device=kv.device)
            out = pool[:, :page]
    elif (out.dtype != torch.uint8 or tuple(out.shape) != (nb, page, 1, row) or out.device != kv.device
          or out.stride(1) != row or out.stride(3) != 1):
        raise RuntimeError(f"out must be a uint8 CUDA tensor of shape (num_blocks, page_block_size, 1, {row}) with packed rows")
    a = _lib.KvQuantArgs(kv.device.index, _LAYOUTS[kvcache_layout], nb * page, page, kv.data_ptr(), d,
                         out.data_ptr(), out.stride(0))
    _lib.check(_lib.load().fmla_kv_quantize(C.byref(a), _stream(kv.device)))
    return out


def abs_indices2indices_in_kvcache(abs_indices: torch.Tensor, block_table: torch.Tensor, block_size: int) -> torch.Tensor:
    """Logical positions (b, s_q, topk) int32 -> in-cache row indices; -1 stays -1.  block_table: (b, max_pages) int32."""
    _require_cuda(abs_indices, "abs_indices")
    if abs_indices.dtype != torch.int32 or block_table.dtype != torch.int32 or block_table.dim() != 2:
        raise RuntimeError("abs_indices and block_table must be int32, block_table of shape (b, max_pages)")
    if block_table.device != abs_indices.device or block_table.shape[0] != abs_indices.shape[0]:
        raise RuntimeError("block_table must be on the same device as abs_indices and have one row per request")
    pos, table = abs_indices.contiguous(), block_table.contiguous()
    out = torch.empty_like(pos)
    b = pos.shape[0]
    a = _lib.CacheIndexArgs(pos.device.index, b, int(block_size), table.shape[1], pos.numel() // b, pos.data_ptr(),
                            table.data_ptr(), out.data_ptr())
    _lib.check(_lib.load().fmla_cache_indices(C.byref(a), _stream(pos.device)))
    return out
