"""Python operator interface of the sparse MLA path, mirroring the reference's
flash_mla/flash_mla_interface.py:8-211 (same names, argument order, defaults, return values and
assertion behaviour) on top of the C ABI in include/flashmla_b200.h.

Differences from the reference, all additive:
  * ``flash_mla_with_kvcache`` takes a keyword-only ``kvcache_layout``.  Left out, the format follows the query
    width like the reference's dispatch (csrc/api/sparse_decode.h:318-325): d_qk = 576 means "v32" (656 bytes per
    token), d_qk = 512 means "model1" (584 bytes per token, stored block-wise).  "mxfp8_e8m0_32" selects rows with
    one e8m0 scale per 32 elements (656 bytes per token, d_qk = 576), a format the reference does not have.
  * ``flash_mla_with_kvcache`` takes a keyword-only ``attn_done_event`` (a timing event recorded
    between its two kernels).
  * ``flash_mla_sparse_bwd`` and ``SparseMLAFunction`` provide the backward of the sparse prefill.
  * the dense decode branch (``indices is None``, bf16 cache with block_table / cache_seqlens / causal), for which
    the reference has no sm_100 kernel, runs split-KV on the decode kernel (fmla_dense_decode) for one KV head and
    h_q % 64 == 0, else on the sparse prefill kernels over index lists that enumerate each request's cache rows (see
    _dense_decode); an FP8 cache without indices raises NotImplementedError.
torch is used for device memory, streams and, in that second dense route, for building the index lists (integer
indexing on the device); every attention computation runs in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import os
from typing import Optional, Tuple

import torch

from . import _lib

D_QK, D_V, ROW_BYTES = 576, 512, 656
M1_D_QK, M1_ROW_BYTES = 512, 584        # the MODEL1 cache format (d_qk = 512; tests/quant.py:55-75 of the reference)
_LAYOUTS = {None: _lib.LAYOUT_V32, "v32": _lib.LAYOUT_V32, "mxfp8_e8m0_32": _lib.LAYOUT_MXFP8, "model1": _lib.LAYOUT_MODEL1}
_KERNELS = {"auto": _lib.KERNEL_AUTO, "simt": _lib.KERNEL_SIMT, "tc": _lib.KERNEL_TC}


def _kernel_choice() -> int:
    """FMLA_KERNEL=auto|simt|tc forces a kernel family (debugging aid; default auto)."""
    name = os.environ.get("FMLA_KERNEL", "auto").lower()
    if name not in _KERNELS:
        raise ValueError(f"FMLA_KERNEL must be one of {sorted(_KERNELS)}, got {name!r}")
    return _KERNELS[name]


@dataclasses.dataclass
class FlashMLASchedMeta:
    """Tile-scheduler metadata of one decode shape (flash_mla_interface.py:8-34 of the reference).

    Filled in by the first ``flash_mla_with_kvcache`` call it is passed to and reused afterwards;
    reuse is only valid while shapes and ``topk_length`` values stay the same.  It also keeps the
    split-KV accumulators so that later calls allocate nothing.
    """

    @dataclasses.dataclass
    class Config:
        b: int
        s_q: int
        h_q: int
        page_block_size: int
        h_k: int
        causal: bool
        is_fp8_kvcache: bool
        topk: Optional[int]
        extra_page_block_size: Optional[int]
        extra_topk: Optional[int]

    have_initialized: bool = False
    config: Optional[Config] = None
    tile_scheduler_metadata: Optional[torch.Tensor] = None   # (num_sm_parts, 8) int32
    num_splits: Optional[torch.Tensor] = None                # (b+1,) int32
    o_accum: Optional[torch.Tensor] = None                   # (b+num_sm_parts, s_q, h_q, 512) fp32
    lse_accum: Optional[torch.Tensor] = None                 # (b+num_sm_parts, s_q, h_q) fp32
    kernel: Optional[int] = None


def get_mla_metadata(*args, **kwargs) -> Tuple[FlashMLASchedMeta, None]:
    """Returns an empty FlashMLASchedMeta; arguments are accepted and ignored for compatibility with
    the older interface (flash_mla_interface.py:37-50).  The schedule is computed by the first
    ``flash_mla_with_kvcache`` call."""
    return FlashMLASchedMeta(), None


_status_words = {}


def _status(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that a kernel sets non-zero when one of its bounded waits gives up."""
    t = _status_words.get(device)
    if t is None:
        t = torch.zeros((1,), dtype=torch.int32, device=device)
        _status_words[device] = t
    return t


def kernel_status(device=None) -> int:
    """Synchronises `device` and returns its kernel status word (0 = no kernel reported a time-out),
    clearing it.  Intended for tests and debugging; normal calls never synchronise."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _status(device)
    torch.cuda.synchronize(device)
    code = int(t.item())
    t.zero_()
    return code


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor; flashmla_b200 has no CPU path")


def _dense_decode(q, k_cache, block_table, cache_seqlens, head_dim_v, softmax_scale, causal, is_fp8_kvcache, sched_meta):
    """Dense MLA decode over a paged bf16 cache (the reference has no sm_100 kernel for it: csrc/api/dense_decode.h:27-29;
    semantics as its torch reference, tests/test_flash_mla_dense_decoding.py:73-141).

    One KV head and a head count that is a multiple of 64 (the MLA decode shapes): split-KV decode through
    fmla_dense_decode, whose kernel walks each request's block table itself; ``sched_meta`` keeps the schedule and the
    accumulators, as in the sparse branch.

    Otherwise it runs as a sparse prefill whose index lists enumerate the cache rows of each request: query row j of
    request i becomes one "query token" per kv head with the list block_table[i][t // page] * page + t % page for the
    tokens t it may see (all cache_seqlens[i] of them, or cache_seqlens[i] - (s_q - 1 - j) with ``causal``), and the
    attention kernel's own per-query length does the masking.  No host synchronisation either way: the lists are as long
    as the block table allows and the lengths stay on the device.
    """
    _require_cuda(q, "q")
    if is_fp8_kvcache:
        raise NotImplementedError("dense MLA decode takes a bf16 cache; FP8 caches are read through top-k indices")
    if q.dim() != 4 or k_cache.dim() != 4 or block_table.dim() != 2 or cache_seqlens.dim() != 1:
        raise RuntimeError("q must be (b, s_q, h_q, d), k_cache (num_blocks, page_block_size, h_kv, d), block_table (b, max_blocks), cache_seqlens (b,)")
    b, s_q, h_q, d_qk = q.shape
    num_blocks, page, h_kv, d_k = k_cache.shape
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise RuntimeError("dense MLA decode: q and k_cache must be bfloat16")
    if d_qk != D_QK or d_k != D_QK or head_dim_v != D_V:
        raise RuntimeError(f"dense MLA decode: only head_dim 576 with head_dim_v 512 is supported (got {d_qk}, {d_k}, {head_dim_v})")
    if h_q % h_kv != 0:
        raise RuntimeError("dense MLA decode: num_heads_q must be a multiple of num_heads_k")
    if block_table.shape[0] != b or cache_seqlens.shape[0] != b or block_table.dtype != torch.int32 or cache_seqlens.dtype != torch.int32:
        raise RuntimeError("dense MLA decode: block_table must be int32 (b, max_blocks) and cache_seqlens int32 (b,)")
    for name, t in (("k_cache", k_cache), ("block_table", block_table), ("cache_seqlens", cache_seqlens)):
        if t.device != q.device:
            raise RuntimeError(f"{name} must be on the same device as q")
    dev = q.device
    if block_table.stride(-1) != 1 or not cache_seqlens.is_contiguous() or q.stride(-1) != 1:
        raise RuntimeError("dense MLA decode: the last dimension of q and block_table must be contiguous, and cache_seqlens contiguous")
    one_pitch = k_cache.stride(-1) == 1 and k_cache.stride(0) == page * k_cache.stride(1) and k_cache.stride(1) % 8 == 0
    if h_kv == 1 and h_q % 64 == 0 and one_pitch and softmax_scale > 0 and _kernel_choice() != _lib.KERNEL_SIMT:
        return _dense_decode_split_kv(q, k_cache, block_table, cache_seqlens, softmax_scale, causal, sched_meta)
    if not k_cache.is_contiguous():
        raise RuntimeError("dense MLA decode: k_cache must be contiguous (one KV head and h_q a multiple of 64: rows at one pitch)")
    hg = h_q // h_kv
    max_len = block_table.shape[1] * page
    pos = torch.arange(max_len, device=dev, dtype=torch.int32)
    rows = block_table[:, (pos // page).long()] * page + (pos % page)                 # [b, max_len] cache token of position t
    seen = cache_seqlens.view(b, 1).expand(b, s_q)
    if causal:
        seen = seen - (s_q - 1 - torch.arange(s_q, device=dev, dtype=torch.int32)).view(1, s_q)
    seen = seen.clamp(min=0)                                                           # [b, s_q] tokens visible to each row
    heads = torch.arange(h_kv, device=dev, dtype=torch.int32)
    idx = rows.view(b, 1, 1, max_len) * h_kv + heads.view(1, 1, h_kv, 1)               # row of (token, kv head) in the flat cache
    idx = torch.where(pos.view(1, 1, 1, max_len) < seen.view(b, s_q, 1, 1), idx.expand(b, s_q, h_kv, max_len),
                      torch.full((), -1, device=dev, dtype=torch.int32))
    n = b * s_q * h_kv
    out, _, lse = flash_mla_sparse_fwd(q.reshape(n, hg, d_qk), k_cache.view(num_blocks * page * h_kv, 1, d_k),
                                       idx.reshape(n, 1, max_len).contiguous(), softmax_scale, head_dim_v, None,
                                       seen.view(b, s_q, 1).expand(b, s_q, h_kv).reshape(n).contiguous())
    return out.view(b, s_q, h_q, head_dim_v), lse.view(b, s_q, h_q).transpose(1, 2)


def _dense_decode_split_kv(q, k_cache, block_table, cache_seqlens, softmax_scale, causal, sched_meta):
    lib = _lib.load()
    dev = q.device
    stream = _stream(dev)
    b, s_q, h_q, _ = q.shape
    num_blocks, page = k_cache.shape[:2]
    max_blocks = block_table.shape[1]
    if sched_meta.tile_scheduler_metadata is None:
        parts, overhead, block = C.c_int32(), C.c_int32(), C.c_int32()
        _lib.check(lib.fmla_decode_plan(dev.index, h_q, s_q, _lib.KERNEL_TC, C.byref(parts), C.byref(overhead), C.byref(block)))
        meta = torch.empty((parts.value, _lib.SCHED_META_INTS), dtype=torch.int32, device=dev)
        splits = torch.empty((b + 1,), dtype=torch.int32, device=dev)
        sa = _lib.SchedArgs(dev.index, b, max_blocks * page, block.value, overhead.value, parts.value,
                            cache_seqlens.data_ptr(), meta.data_ptr(), splits.data_ptr(), 0, None)
        _lib.check(lib.fmla_sched_meta(C.byref(sa), stream))
        sched_meta.tile_scheduler_metadata = meta
        sched_meta.num_splits = splits
        sched_meta.kernel = _lib.KERNEL_TC
    meta, splits = sched_meta.tile_scheduler_metadata, sched_meta.num_splits
    parts = meta.shape[0]
    if sched_meta.o_accum is None or sched_meta.o_accum.device != dev:
        sched_meta.o_accum = torch.empty((b + parts, s_q, h_q, D_V), dtype=torch.float32, device=dev)
        sched_meta.lse_accum = torch.empty((b + parts, s_q, h_q), dtype=torch.float32, device=dev)
    out = torch.empty((b, s_q, h_q, D_V), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((b, s_q, h_q), dtype=torch.float32, device=dev)
    a = _lib.DenseDecodeArgs()
    a.device, a.b, a.s_q, a.h_q, a.causal, a.sm_scale = dev.index, b, s_q, h_q, int(bool(causal)), float(softmax_scale)
    a.q, a.q_stride_b, a.q_stride_s, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    a.kv, a.num_blocks, a.page_block_size, a.kv_stride_row = k_cache.data_ptr(), num_blocks, page, k_cache.stride(1)
    a.block_table, a.block_table_stride, a.max_blocks_per_seq = block_table.data_ptr(), block_table.stride(0), max_blocks
    a.cache_seqlens = cache_seqlens.data_ptr()
    a.out, a.o_stride_b, a.o_stride_s, a.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    a.lse, a.lse_stride_b, a.lse_stride_s = lse.data_ptr(), lse.stride(0), lse.stride(1)
    a.sched_meta, a.num_splits, a.num_sm_parts = meta.data_ptr(), splits.data_ptr(), parts
    a.o_accum, a.lse_accum, a.status = sched_meta.o_accum.data_ptr(), sched_meta.lse_accum.data_ptr(), _status(dev).data_ptr()
    _lib.check(lib.fmla_dense_decode(C.byref(a), stream))
    return out, lse.transpose(1, 2)


def flash_mla_with_kvcache(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    block_table: Optional[torch.Tensor],
    cache_seqlens: Optional[torch.Tensor],
    head_dim_v: int,
    tile_scheduler_metadata: FlashMLASchedMeta,
    num_splits: None = None,
    softmax_scale: Optional[float] = None,
    causal: bool = False,
    is_fp8_kvcache: bool = False,
    indices: Optional[torch.Tensor] = None,
    attn_sink: Optional[torch.Tensor] = None,
    extra_k_cache: Optional[torch.Tensor] = None,
    extra_indices_in_kvcache: Optional[torch.Tensor] = None,
    topk_length: Optional[torch.Tensor] = None,
    extra_topk_length: Optional[torch.Tensor] = None,
    *,
    kvcache_layout: Optional[str] = None,
    attn_done_event: Optional["torch.cuda.Event"] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse MLA decode over a paged FP8 KV cache, or, with indices=None, dense MLA decode over a paged bf16 cache with
    block_table / cache_seqlens / causal (see _dense_decode) (flash_mla_interface.py:53-173 of the reference).

    q: (b, s_q, h_q, 576) bf16.  k_cache: (num_blocks, page_block_size, 1, 656) bytes (fp8/uint8/int8);
    the block stride may exceed page_block_size*656.  With q (b, s_q, h_q, 512) the cache is the reference's MODEL1
    format, (num_blocks, page_block_size, 1, 584) as tests/quant.py:55-75 lays it out.  indices: (b, s_q, topk) int32 with
    indices[i,j,k] = page_index*page_block_size + offset_in_page, or -1.  attn_sink: (h_q,) fp32.
    topk_length: (b,) int32, only the leftmost topk_length[i] slots are attended.
    attn_done_event: an optional timing event, recorded between the attention and the combine kernel.
    Returns (out (b, s_q, h_q, 512) bf16, lse (b, h_q, s_q) fp32, natural log).
    """
    sched_meta = tile_scheduler_metadata
    assert isinstance(sched_meta, FlashMLASchedMeta), "tile_scheduler_metadata must be of type FlashMLASchedMeta"
    assert num_splits is None, "num_splits must be None"

    topk = indices.shape[-1] if indices is not None else None
    extra_page = extra_k_cache.shape[1] if extra_k_cache is not None else None
    extra_topk = extra_indices_in_kvcache.shape[-1] if extra_indices_in_kvcache is not None else None
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)

    if not sched_meta.have_initialized:
        if indices is not None:
            assert not causal, "causal must be False when indices_in_kvcache is not None (i.e. sparse attention is enabled)"
        sched_meta.have_initialized = True
        sched_meta.config = FlashMLASchedMeta.Config(
            q.shape[0], q.shape[1], q.shape[2], k_cache.shape[1], k_cache.shape[2],
            causal, is_fp8_kvcache, topk, extra_page, extra_topk)
    else:
        msg = (" Your input arguments are inconsistent with sched_meta. Please make sure the input arguments are "
               "consistent across different invocations of flash_mla_with_kvcache on the same sched_meta.")
        cfg = sched_meta.config
        assert cfg is not None
        assert cfg.b == q.shape[0], "sched_meta.config.b must be equal to batch_size." + msg
        assert cfg.s_q == q.shape[1], "sched_meta.config.s_q must be equal to seq_len_q." + msg
        assert cfg.h_q == q.shape[2], "sched_meta.config.h_q must be equal to num_heads_q." + msg
        assert cfg.page_block_size == k_cache.shape[1], "sched_meta.config.page_block_size must be equal to page_block_size." + msg
        assert cfg.h_k == k_cache.shape[2], "sched_meta.config.h_k must be equal to num_heads_k." + msg
        assert cfg.causal == causal, "sched_meta.config.causal must be equal to causal." + msg
        assert cfg.is_fp8_kvcache == is_fp8_kvcache, "sched_meta.config.is_fp8_kvcache must be equal to is_fp8_kvcache." + msg
        assert cfg.topk == topk, "sched_meta.config.topk must be equal to the last dim of indices_in_kvcache." + msg
        assert cfg.extra_page_block_size == extra_page, "sched_meta.config.extra_page_block_size must be equal to the page_block_size of extra_k_cache." + msg
        assert cfg.extra_topk == extra_topk, "sched_meta.config.extra_topk must be equal to the last dim of extra_indices_in_kvcache." + msg

    if topk is None:
        # Dense attention (flash_mla_interface.py:161-170 of the reference)
        assert attn_sink is None and extra_k_cache is None and extra_indices_in_kvcache is None and topk_length is None and extra_topk_length is None, \
            "indices_in_kvcache, attn_sink, extra_k_cache, extra_indices_in_kvcache, topk_length and extra_topk_length must be None when dense attention is used."
        assert block_table is not None and cache_seqlens is not None, "block_table and cache_seqlens must be provided when dense attention is used."
        return _dense_decode(q, k_cache, block_table, cache_seqlens, head_dim_v, softmax_scale, causal, is_fp8_kvcache, sched_meta)
    assert not causal, "causal must be False when sparse attention is enabled"
    assert is_fp8_kvcache, "is_fp8_kvcache must be True when sparse attention is enabled"
    if extra_k_cache is not None:
        if extra_indices_in_kvcache is None:
            raise RuntimeError("extra_indices_in_kvcache must be provided when extra_kcache is provided for sparse attention")
    else:
        if extra_indices_in_kvcache is not None:
            raise RuntimeError("extra_indices_in_kvcache must not be provided when extra_k_cache is not provided")
        if extra_topk_length is not None:
            raise RuntimeError("extra_topk_length must not be provided when extra_k_cache is not provided")
    if kvcache_layout not in _LAYOUTS:
        raise ValueError(f"kvcache_layout must be one of {[k for k in _LAYOUTS if k]}, got {kvcache_layout!r}")

    # ---- argument checks (csrc/api/sparse_decode.h:203-310 of the reference) ----
    _require_cuda(q, "q")
    if q.dim() != 4 or k_cache.dim() != 4 or indices.dim() != 3:
        raise RuntimeError("q must be 4-D (b, s_q, h_q, d), k_cache 4-D (blocks, page, 1, bytes), indices 3-D (b, s_q, topk)")
    b, s_q, h_q, d_qk = q.shape
    if q.dtype != torch.bfloat16:
        raise RuntimeError("q must be bfloat16")
    if d_qk not in (D_QK, M1_D_QK) or head_dim_v != D_V:
        raise RuntimeError(f"only head_dim 576 or 512 with head_dim_v 512 is supported (got {d_qk}, {head_dim_v})")
    if kvcache_layout is None and d_qk == M1_D_QK:
        kvcache_layout = "model1"
    if (_LAYOUTS[kvcache_layout] == _lib.LAYOUT_MODEL1) != (d_qk == M1_D_QK):
        raise RuntimeError(f"kvcache_layout {kvcache_layout!r} does not go with head_dim {d_qk}")
    ROW = M1_ROW_BYTES if d_qk == M1_D_QK else ROW_BYTES
    if k_cache.element_size() != 1:
        raise RuntimeError("k_cache must have a 1-byte dtype (float8_e4m3fn, uint8 or int8)")
    num_blocks, page, h_k, row_bytes = k_cache.shape
    if h_k != 1 or row_bytes != ROW:
        raise RuntimeError(f"k_cache must be (num_blocks, page_block_size, 1, {ROW}); got {tuple(k_cache.shape)}")
    if k_cache.stride(-1) != 1 or k_cache.stride(1) != ROW:
        raise RuntimeError(f"k_cache rows must be contiguous {ROW}-byte records (stride(1) == {ROW})")
    if indices.dtype != torch.int32 or tuple(indices.shape[:2]) != (b, s_q):
        raise RuntimeError("indices must be int32 of shape (b, s_q, topk)")
    if q.stride(-1) != 1 or indices.stride(-1) != 1:
        raise RuntimeError("the last dimension of q and indices must be contiguous")
    for name, t in (("k_cache", k_cache), ("indices", indices), ("attn_sink", attn_sink), ("topk_length", topk_length)):
        if t is not None and t.device != q.device:
            raise RuntimeError(f"{name} must be on the same device as q")
    if attn_sink is not None and (attn_sink.dtype != torch.float32 or tuple(attn_sink.shape) != (h_q,) or not attn_sink.is_contiguous()):
        raise RuntimeError("attn_sink must be a contiguous float32 tensor of shape (h_q,)")
    if topk_length is not None and (topk_length.dtype != torch.int32 or tuple(topk_length.shape) != (b,) or not topk_length.is_contiguous()):
        raise RuntimeError("topk_length must be a contiguous int32 tensor of shape (b,)")
    if extra_k_cache is not None:
        if (extra_k_cache.dim() != 4 or extra_k_cache.element_size() != 1 or extra_k_cache.shape[2] != 1
                or extra_k_cache.shape[3] != ROW or extra_k_cache.stride(-1) != 1 or extra_k_cache.stride(1) != ROW):
            raise RuntimeError(f"extra_k_cache must be (num_blocks, page_block_size, 1, {ROW}) bytes with contiguous {ROW}-byte rows")
        if (extra_indices_in_kvcache.dtype != torch.int32 or extra_indices_in_kvcache.dim() != 3
                or tuple(extra_indices_in_kvcache.shape[:2]) != (b, s_q) or extra_indices_in_kvcache.stride(-1) != 1):
            raise RuntimeError("extra_indices_in_kvcache must be int32 of shape (b, s_q, extra_topk) with a contiguous last dimension")
        if extra_topk_length is not None and (extra_topk_length.dtype != torch.int32 or tuple(extra_topk_length.shape) != (b,)
                                              or not extra_topk_length.is_contiguous()):
            raise RuntimeError("extra_topk_length must be a contiguous int32 tensor of shape (b,)")
        for name, t in (("extra_k_cache", extra_k_cache), ("extra_indices_in_kvcache", extra_indices_in_kvcache),
                        ("extra_topk_length", extra_topk_length)):
            if t is not None and t.device != q.device:
                raise RuntimeError(f"{name} must be on the same device as q")

    lib = _lib.load()
    dev = q.device
    stream = _stream(dev)
    kernel = sched_meta.kernel if sched_meta.kernel is not None else _kernel_choice()

    if sched_meta.tile_scheduler_metadata is None:
        parts, overhead, block = C.c_int32(), C.c_int32(), C.c_int32()
        _lib.check(lib.fmla_decode_plan(dev.index, h_q, s_q, kernel, C.byref(parts), C.byref(overhead), C.byref(block)))
        meta = torch.empty((parts.value, _lib.SCHED_META_INTS), dtype=torch.int32, device=dev)
        splits = torch.empty((b + 1,), dtype=torch.int32, device=dev)
        sa = _lib.SchedArgs(dev.index, b, topk, block.value, overhead.value, parts.value,
                            _ptr(topk_length), meta.data_ptr(), splits.data_ptr(),
                            extra_topk or 0, _ptr(extra_topk_length))
        _lib.check(lib.fmla_sched_meta(C.byref(sa), stream))
        sched_meta.tile_scheduler_metadata = meta
        sched_meta.num_splits = splits
        sched_meta.kernel = kernel
    meta, splits = sched_meta.tile_scheduler_metadata, sched_meta.num_splits
    parts = meta.shape[0]
    if sched_meta.o_accum is None or sched_meta.o_accum.device != dev:
        sched_meta.o_accum = torch.empty((b + parts, s_q, h_q, D_V), dtype=torch.float32, device=dev)
        sched_meta.lse_accum = torch.empty((b + parts, s_q, h_q), dtype=torch.float32, device=dev)

    out = torch.empty((b, s_q, h_q, D_V), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((b, s_q, h_q), dtype=torch.float32, device=dev)
    a = _lib.DecodeArgs()
    a.device, a.b, a.s_q, a.h_q, a.topk = dev.index, b, s_q, h_q, topk
    a.layout, a.kernel, a.sm_scale = _LAYOUTS[kvcache_layout], kernel, float(softmax_scale)
    a.q, a.q_stride_b, a.q_stride_s, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    a.kv, a.num_blocks, a.page_block_size, a.kv_stride_block = k_cache.data_ptr(), num_blocks, page, k_cache.stride(0)
    a.indices, a.idx_stride_b, a.idx_stride_s = indices.data_ptr(), indices.stride(0), indices.stride(1)
    a.topk_length, a.attn_sink = _ptr(topk_length), _ptr(attn_sink)
    a.out, a.o_stride_b, a.o_stride_s, a.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    a.lse, a.lse_stride_b, a.lse_stride_s = lse.data_ptr(), lse.stride(0), lse.stride(1)
    a.sched_meta, a.num_splits, a.num_sm_parts = meta.data_ptr(), splits.data_ptr(), parts
    a.o_accum, a.lse_accum, a.status = sched_meta.o_accum.data_ptr(), sched_meta.lse_accum.data_ptr(), _status(dev).data_ptr()
    if extra_k_cache is not None:
        a.extra_kv, a.extra_num_blocks, a.extra_page_block_size = extra_k_cache.data_ptr(), extra_k_cache.shape[0], extra_k_cache.shape[1]
        a.extra_kv_stride_block = extra_k_cache.stride(0)
        a.extra_indices = extra_indices_in_kvcache.data_ptr()
        a.extra_idx_stride_b, a.extra_idx_stride_s = extra_indices_in_kvcache.stride(0), extra_indices_in_kvcache.stride(1)
        a.extra_topk, a.extra_topk_length = extra_topk, _ptr(extra_topk_length)
    if attn_done_event is not None:
        if not attn_done_event.cuda_event:     # torch creates the CUDA event lazily, on the first record()
            attn_done_event.record(torch.cuda.current_stream(dev))
        a.attn_done_event = attn_done_event.cuda_event
    _lib.check(lib.fmla_sparse_decode(C.byref(a), stream))
    return out, lse.transpose(1, 2)


def _check_prefill(q, kv, indices, d_v, attn_sink, topk_length):
    _require_cuda(q, "q")
    if q.dim() != 3 or kv.dim() != 3 or indices.dim() != 3:
        raise RuntimeError("q must be (s_q, h_q, d_qk), kv (s_kv, h_kv, d_qk), indices (s_q, h_kv, topk)")
    s_q, h_q, d_qk = q.shape
    s_kv, h_kv, _ = kv.shape
    if q.dtype != torch.bfloat16 or kv.dtype != torch.bfloat16 or indices.dtype != torch.int32:
        raise RuntimeError("q and kv must be bfloat16 and indices int32")
    if d_qk not in (D_QK, M1_D_QK) or kv.shape[2] != d_qk or d_v != D_V:
        raise RuntimeError(f"only d_qk=576 or 512 (q and kv alike) with d_v=512 is supported (got {d_qk}, {kv.shape[2]}, {d_v})")
    if h_kv != 1 or tuple(indices.shape[:2]) != (s_q, 1):
        raise RuntimeError("h_kv must be 1 and indices must be (s_q, 1, topk)")
    if q.stride(-1) != 1 or kv.stride(-1) != 1 or indices.stride(-1) != 1:
        raise RuntimeError("the last dimension of q, kv and indices must be contiguous")
    for name, t in (("kv", kv), ("indices", indices), ("attn_sink", attn_sink), ("topk_length", topk_length)):
        if t is not None and t.device != q.device:
            raise RuntimeError(f"{name} must be on the same device as q")
    if attn_sink is not None and (attn_sink.dtype != torch.float32 or tuple(attn_sink.shape) != (h_q,) or not attn_sink.is_contiguous()):
        raise RuntimeError("attn_sink must be a contiguous float32 tensor of shape (h_q,)")
    if topk_length is not None and (topk_length.dtype != torch.int32 or tuple(topk_length.shape) != (s_q,) or not topk_length.is_contiguous()):
        raise RuntimeError("topk_length must be a contiguous int32 tensor of shape (s_q,)")
    return s_q, s_kv, h_q, indices.shape[-1]


def flash_mla_sparse_fwd(
    q: torch.Tensor,
    kv: torch.Tensor,
    indices: torch.Tensor,
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,
    topk_length: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sparse attention prefill forward (flash_mla_interface.py:176-211 of the reference).

    q (s_q, h_q, d_qk) bf16, kv (s_kv, 1, d_qk) bf16 with d_qk = 576 or 512, indices (s_q, 1, topk) int32 where an index
    outside [0, s_kv) is invalid; topk_length (s_q,) keeps only the leftmost slots of each query.
    Returns (out (s_q, h_q, 512) bf16, max_logits (s_q, h_q) fp32, lse (s_q, h_q) fp32).
    """
    s_q, s_kv, h_q, topk = _check_prefill(q, kv, indices, d_v, attn_sink, topk_length)
    dev = q.device
    out = torch.empty((s_q, h_q, D_V), dtype=torch.bfloat16, device=dev)
    max_logits = torch.empty((s_q, h_q), dtype=torch.float32, device=dev)
    lse = torch.empty((s_q, h_q), dtype=torch.float32, device=dev)
    a = _lib.PrefillArgs()
    a.device, a.s_q, a.s_kv, a.h_q, a.topk = dev.index, s_q, s_kv, h_q, topk
    a.kernel, a.sm_scale = _kernel_choice(), float(sm_scale)
    a.q, a.q_stride_s, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    a.kv, a.kv_stride_s = kv.data_ptr(), kv.stride(0)
    a.indices, a.idx_stride_s = indices.data_ptr(), indices.stride(0)
    a.attn_sink, a.topk_length = _ptr(attn_sink), _ptr(topk_length)
    a.out, a.max_logits, a.lse, a.status = out.data_ptr(), max_logits.data_ptr(), lse.data_ptr(), _status(dev).data_ptr()
    a.d_qk = q.shape[-1]
    _lib.check(_lib.load().fmla_sparse_prefill_fwd(C.byref(a), _stream(dev)))
    return out, max_logits, lse


BWD_CHUNK_TOKENS = 592   # query tokens per pass of the tensor-core backward (1 MiB of workspace per token and 128 heads at topk 2048)


def flash_mla_sparse_bwd(
    q: torch.Tensor,
    kv: torch.Tensor,
    out: torch.Tensor,
    dout: torch.Tensor,
    indices: torch.Tensor,
    lse: torch.Tensor,
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,
    topk_length: Optional[torch.Tensor] = None,
    return_fp32_dkv: bool = False,
    *,
    grad_events: Optional[Tuple["torch.cuda.Event", "torch.cuda.Event"]] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Backward of ``flash_mla_sparse_fwd`` (no counterpart in the reference).

    grad_events: an optional pair of timing events recorded around the first pass's dQ / dKV launch.

    out and lse are the forward's results, dout (s_q, h_q, 512) bf16.  Returns dq (s_q, h_q, 576)
    bf16 and dkv (s_kv, 1, 576): gradients of all queries that index a token are added in fp32 and
    then rounded to bf16 (or returned in fp32 when return_fp32_dkv is set).  attn_sink is treated as
    a constant.
    """
    s_q, s_kv, h_q, topk = _check_prefill(q, kv, indices, d_v, attn_sink, topk_length)
    if q.shape[-1] != D_QK:
        raise RuntimeError("the backward covers d_qk = 576 only")
    dev = q.device
    if out.dtype != torch.bfloat16 or dout.dtype != torch.bfloat16 or tuple(out.shape) != (s_q, h_q, D_V) or tuple(dout.shape) != (s_q, h_q, D_V):
        raise RuntimeError("out and dout must be bfloat16 of shape (s_q, h_q, 512)")
    if lse.dtype != torch.float32 or tuple(lse.shape) != (s_q, h_q):
        raise RuntimeError("lse must be float32 of shape (s_q, h_q)")
    out = out.contiguous()
    lse = lse.contiguous()
    if dout.stride(-1) != 1:
        dout = dout.contiguous()
    dq = torch.empty((s_q, h_q, D_QK), dtype=torch.bfloat16, device=dev)
    dkv_acc = torch.empty((s_kv, D_QK), dtype=torch.float32, device=dev)
    dkv = None if return_fp32_dkv else torch.empty((s_kv, D_QK), dtype=torch.bfloat16, device=dev)
    a = _lib.PrefillBwdArgs()
    a.device, a.s_q, a.s_kv, a.h_q, a.topk = dev.index, s_q, s_kv, h_q, topk
    a.kernel, a.sm_scale = _kernel_choice(), float(sm_scale)
    a.q, a.q_stride_s, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    a.kv, a.kv_stride_s = kv.data_ptr(), kv.stride(0)
    a.out, a.dout, a.do_stride_s, a.do_stride_h = out.data_ptr(), dout.data_ptr(), dout.stride(0), dout.stride(1)
    a.lse, a.indices, a.idx_stride_s = lse.data_ptr(), indices.data_ptr(), indices.stride(0)
    a.attn_sink, a.topk_length = _ptr(attn_sink), _ptr(topk_length)
    a.dq, a.dkv_accum, a.dkv = dq.data_ptr(), dkv_acc.data_ptr(), _ptr(dkv)
    # the tensor-core kernels pass P and dS through a bf16 workspace; BWD_CHUNK_TOKENS query tokens per pass
    lib = _lib.load()
    ws_bytes = lib.fmla_sparse_prefill_bwd_workspace(min(s_q, BWD_CHUNK_TOKENS), h_q, topk, a.kernel)
    workspace = torch.empty((ws_bytes,), dtype=torch.uint8, device=dev) if ws_bytes > 0 else None
    a.workspace, a.workspace_bytes, a.status = _ptr(workspace), ws_bytes, _status(dev).data_ptr()
    if grad_events is not None:
        for ev in grad_events:
            if not ev.cuda_event:          # torch creates the CUDA event lazily, on the first record()
                ev.record(torch.cuda.current_stream(dev))
        a.grad_begin_event, a.grad_end_event = grad_events[0].cuda_event, grad_events[1].cuda_event
    _lib.check(lib.fmla_sparse_prefill_bwd(C.byref(a), _stream(dev)))
    return dq, (dkv_acc if return_fp32_dkv else dkv).view(s_kv, 1, D_QK)


class SparseMLAFunction(torch.autograd.Function):
    """autograd wrapper: out = sparse_attention(q, kv; indices).  max_logits and lse are returned
    as non-differentiable extras."""

    @staticmethod
    def forward(ctx, q, kv, indices, sm_scale, attn_sink=None, topk_length=None):
        out, max_logits, lse = flash_mla_sparse_fwd(q, kv, indices, sm_scale, D_V, attn_sink, topk_length)
        ctx.save_for_backward(q, kv, out, lse, indices, attn_sink, topk_length)
        ctx.sm_scale = sm_scale
        ctx.mark_non_differentiable(max_logits, lse)
        return out, max_logits, lse

    @staticmethod
    def backward(ctx, dout, _dmax, _dlse):
        q, kv, out, lse, indices, attn_sink, topk_length = ctx.saved_tensors
        dq, dkv = flash_mla_sparse_bwd(q, kv, out, dout.contiguous(), indices, lse, ctx.sm_scale, D_V, attn_sink, topk_length)
        return dq, dkv, None, None, None, None


def flash_mla_sparse_attn(q, kv, indices, sm_scale, attn_sink=None, topk_length=None):
    """Differentiable sparse attention: returns (out, max_logits, lse)."""
    return SparseMLAFunction.apply(q, kv, indices, sm_scale, attn_sink, topk_length)
