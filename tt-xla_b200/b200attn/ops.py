"""CUDA ops of the attention / KV-cache path, one per `torch.ops.tt.*` op the reference plugin
calls (python_package/tt_torch/custom_ops.py).  Each takes torch CUDA tensors, validates the
layout the reference documents, and calls the C ABI on torch's current stream.

The reference ops are functional (they return a new cache, which the caller copies back,
attention.py:513-515); these update the caches in place, which is what that copy-back amounts
to.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _lib

_workspaces: dict[tuple[int, int], torch.Tensor] = {}
# Scratch that was outgrown stays allocated: a CUDA graph captured earlier still launches into
# it, and its arrival counters must stay zero (memory handed back to the allocator could be
# given to another tensor).
_retired_workspaces: list[torch.Tensor] = []


CACHE_BF16, CACHE_FP8_E4M3 = 0, 1     # enum b200attn_cache_dtype
TICKET_BYTES = 65536                  # B200ATTN_DECODE_TICKET_BYTES


def _cache_dtype(cache: torch.Tensor) -> int:
    return CACHE_FP8_E4M3 if cache.dtype == torch.float8_e4m3fn else CACHE_BF16


def _env_num_splits() -> int:
    """`B200ATTN_NUM_SPLITS=n` pins the split count of every decode call that leaves it to the
    library (for sweeps and for ruling the cost model out while debugging); unset or 0 = the
    model's choice.  Read on every call: changing it between steps is allowed outside graphs."""
    raw = os.environ.get("B200ATTN_NUM_SPLITS", "")
    if not raw:
        return 0
    n = int(raw)
    if not 0 <= n <= 256:
        raise ValueError(f"B200ATTN_NUM_SPLITS must be 0..256, got {raw!r}")
    return n


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "b200attn ops run on CUDA tensors only (there is no CPU path); got a "
                f"{t.device.type} tensor"
            )


def _check_cache(k_cache: torch.Tensor, v_cache: torch.Tensor) -> tuple[int, int, int, int]:
    if k_cache.dim() != 4 or k_cache.shape != v_cache.shape:
        raise ValueError(
            "k_cache and v_cache must both be [num_blocks, num_kv_heads, block_size, head_size]; "
            f"got {tuple(k_cache.shape)} and {tuple(v_cache.shape)}"
        )
    if k_cache.dtype != v_cache.dtype or k_cache.dtype not in (torch.bfloat16, torch.float8_e4m3fn):
        raise ValueError("caches must both be bfloat16 or both be float8_e4m3fn")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("caches must be contiguous")
    nb, nkv, bs, hd = k_cache.shape
    return nb, nkv, bs, hd


def _token_major(x: torch.Tensor, nheads: int, hd: int, name: str) -> tuple[torch.Tensor, int]:
    """Returns a [tokens, nheads, hd] view whose last two dims are dense, and its row stride."""
    x = x.reshape(-1, nheads, hd) if x.dim() != 3 else x
    if x.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16")
    if x.stride(2) != 1 or x.stride(1) != hd:
        x = x.contiguous()
    return x, x.stride(0) if x.shape[0] > 1 else max(x.stride(0), nheads * hd)


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32:
        raise ValueError(f"{name} must be int32, got {t.dtype}")
    return t


def paged_update_cache(
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    update_indices: torch.Tensor,
    page_table: torch.Tensor,
) -> None:
    """Decode-step KV write: `tt.paged_update_cache` for K and V in one launch
    (custom_ops.py:962-1013).  `key`/`value`: [users, nkv, hd] (the reference's
    [1, users, nkv, hd] is accepted too)."""
    _need_cuda(k_cache, v_cache, key, value, update_indices, page_table)
    nb, nkv, bs, hd = _check_cache(k_cache, v_cache)
    key, kstride = _token_major(key, nkv, hd, "key")
    value, vstride = _token_major(value, nkv, hd, "value")
    if key.shape != value.shape:
        raise ValueError("key and value must have the same shape")
    if kstride != vstride:
        value = value.contiguous()
        key = key.contiguous()
        kstride = nkv * hd
    users = update_indices.shape[0]
    if key.shape[0] != users or page_table.shape[0] < users:
        raise ValueError("key/value rows, update_indices and page_table rows must agree")
    _i32(update_indices, "update_indices")
    _i32(page_table, "page_table")
    if page_table.stride(1) != 1 or not update_indices.is_contiguous():
        raise ValueError("page_table rows and update_indices must be dense")
    L = _lib.lib()
    _lib.check(
        "b200attn_paged_update_cache_ex",
        L.b200attn_paged_update_cache_ex(
            k_cache.data_ptr(), v_cache.data_ptr(), key.data_ptr(), value.data_ptr(), kstride,
            update_indices.data_ptr(), page_table.data_ptr(), page_table.stride(0),
            page_table.shape[1], users, nkv, hd, bs, nb, _cache_dtype(k_cache), _stream(k_cache),
        ),
    )


def paged_fill_cache(
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    fill_page_table: torch.Tensor,
    batch_idx: Optional[torch.Tensor] = None,
) -> None:
    """Prefill / chunk KV write: `tt.paged_fill_cache` for K and V, all users in one launch
    (custom_ops.py:1016-1104).  `key`/`value`: [users, tokens, nkv, hd] token-major (the layout
    the plugin holds before it transposes for the reference op, attention.py:487-488)."""
    _need_cuda(k_cache, v_cache, key, value, fill_page_table, batch_idx)
    nb, nkv, bs, hd = _check_cache(k_cache, v_cache)
    if key.dim() != 4 or key.shape != value.shape or key.shape[2] != nkv or key.shape[3] != hd:
        raise ValueError(
            f"key/value must be [users, tokens, {nkv}, {hd}], got {tuple(key.shape)}"
        )
    users, tokens = key.shape[0], key.shape[1]
    if not key.is_contiguous():
        key = key.contiguous()
    if not value.is_contiguous():
        value = value.contiguous()
    _i32(fill_page_table, "fill_page_table")
    if fill_page_table.stride(1) != 1:
        raise ValueError("fill_page_table rows must be dense")
    if batch_idx is not None:
        _i32(batch_idx, "batch_idx")
        if batch_idx.numel() != users or not batch_idx.is_contiguous():
            raise ValueError("batch_idx must hold one dense entry per user")
    L = _lib.lib()
    _lib.check(
        "b200attn_paged_fill_cache_ex",
        L.b200attn_paged_fill_cache_ex(
            k_cache.data_ptr(), v_cache.data_ptr(), key.data_ptr(), value.data_ptr(), nkv * hd,
            fill_page_table.data_ptr(), fill_page_table.stride(0), fill_page_table.shape[1],
            batch_idx.data_ptr() if batch_idx is not None else None,
            users, tokens, nkv, hd, bs, nb, _cache_dtype(k_cache), _stream(k_cache),
        ),
    )


def kv_scatter_slots(
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> None:
    """KV write addressed by vLLM's `slot_mapping` (int64, negative = skip); the live-layout
    counterpart of `write_to_kv_cache` (attention.py:671-716)."""
    _need_cuda(k_cache, v_cache, key, value, slot_mapping)
    nb, nkv, bs, hd = _check_cache(k_cache, v_cache)
    key, kstride = _token_major(key, nkv, hd, "key")
    value, vstride = _token_major(value, nkv, hd, "value")
    if kstride != vstride:
        key, value = key.contiguous(), value.contiguous()
        kstride = nkv * hd
    if slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a dense int64 tensor")
    n = slot_mapping.numel()
    if key.shape[0] < n or value.shape[0] < n:
        raise ValueError("fewer key/value rows than slots")
    L = _lib.lib()
    _lib.check(
        "b200attn_kv_scatter_slots_ex",
        L.b200attn_kv_scatter_slots_ex(
            k_cache.data_ptr(), v_cache.data_ptr(), key.data_ptr(), value.data_ptr(), kstride,
            slot_mapping.data_ptr(), n, nkv, hd, bs, nb, _cache_dtype(k_cache), _stream(k_cache),
        ),
    )


def rope_kv_scatter_slots(
    query: torch.Tensor,
    key: torch.Tensor,
    value: Optional[torch.Tensor],
    positions: torch.Tensor,
    inv_freq: torch.Tensor,
    rotary_dim: int,
    head_size: int,
    k_cache: Optional[torch.Tensor] = None,
    v_cache: Optional[torch.Tensor] = None,
    slot_mapping: Optional[torch.Tensor] = None,
    is_neox_style: bool = True,
) -> None:
    """Rotary embedding of `query` / `key` IN PLACE, computed like the plugin's rotary layer
    (layers/rotary_embedding.py:51-66), fused with the slot-mapping cache write of the rotated
    key and of `value`.  `query` [tokens, nq*hd], `key` / `value` [tokens, nkv*hd] (dense rows,
    any row stride); `positions` int64 [tokens]; `inv_freq` fp32 [rotary_dim/2].  Without
    `slot_mapping` only the rotation is done."""
    _need_cuda(query, key, value, positions, inv_freq, k_cache, v_cache, slot_mapping)
    tokens = positions.numel()
    if query.dim() != 2 or key.dim() != 2 or query.shape[0] != tokens or key.shape[0] != tokens:
        raise ValueError("query / key must be [tokens, heads*head_size] with one row per position")
    if query.dtype != torch.bfloat16 or key.dtype != torch.bfloat16:
        raise ValueError("query / key must be bfloat16")
    if query.stride(1) != 1 or key.stride(1) != 1:
        raise ValueError("query / key rows must be dense")
    nq, nkv = query.shape[1] // head_size, key.shape[1] // head_size
    if positions.dtype != torch.int64 or not positions.is_contiguous():
        raise ValueError("positions must be a dense int64 tensor")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2 \
            or not inv_freq.is_contiguous():
        raise ValueError("inv_freq must be dense float32 [rotary_dim / 2]")
    nb = bs = 0
    if slot_mapping is not None:
        nb, nkv_c, bs, hd_c = _check_cache(k_cache, v_cache)
        if nkv_c != nkv or hd_c != head_size:
            raise ValueError("cache geometry differs from key geometry")
        if value is None or value.shape != key.shape or value.stride(1) != 1:
            raise ValueError("value must match key")
        if slot_mapping.dtype != torch.int64 or slot_mapping.numel() < tokens:
            raise ValueError("slot_mapping must be int64 with one entry per token")
    L = _lib.lib()
    _lib.check(
        "b200attn_rope_kv_scatter_slots",
        L.b200attn_rope_kv_scatter_slots(
            query.data_ptr(), query.stride(0), key.data_ptr(), key.stride(0),
            value.data_ptr() if value is not None else None,
            value.stride(0) if value is not None else 0,
            positions.data_ptr(), inv_freq.data_ptr(), rotary_dim, 1 if is_neox_style else 0,
            k_cache.data_ptr() if slot_mapping is not None else None,
            v_cache.data_ptr() if slot_mapping is not None else None,
            slot_mapping.data_ptr() if slot_mapping is not None else None,
            tokens, nq, nkv, head_size, bs, nb, _stream(query),
        ),
    )


def decode_auto_splits(users: int, nkv: int, hd: int, max_context_len: int) -> int:
    return _lib.lib().b200attn_decode_auto_splits(users, nkv, hd, max_context_len)


def decode_workspace_bytes(users: int, nq: int, hd: int, splits: int) -> int:
    return _lib.lib().b200attn_decode_workspace_bytes(users, nq, hd, splits)


def _workspace(device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
    """Split-KV scratch, cached per (device, stream) and grown on demand.  torch owns the
    memory; the C library never allocates.  Allocated zeroed: the arrival counters at its start
    have to be zero on first use (every call leaves them zero)."""
    if nbytes == 0:
        return None
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def paged_decode(
    query: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    page_table: torch.Tensor,
    cur_pos: torch.Tensor,
    scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    num_splits: int = 0,
    max_context_len: int = 0,
    workspace: Optional[torch.Tensor] = None,
    sliding_window: int = 0,
    sinks: Optional[torch.Tensor] = None,
    new_key: Optional[torch.Tensor] = None,
    new_value: Optional[torch.Tensor] = None,
    wrap_negative_positions: bool = True,
) -> torch.Tensor:
    """Paged GQA decode attention: `tt.paged_scaled_dot_product_attention_decode` with
    is_causal=True and cur_pos_tensor (custom_ops.py:1198-1331).  `query`: [users, nq, hd]
    (or the reference's [1, users, nq, hd]); returns / fills `out` of the same shape.
    `sliding_window` > 0 limits each user to its last `sliding_window` keys; `sinks` (fp32
    [nq]) adds one denominator-only softmax column per head (the op's `sliding_window_size` /
    `attention_sink` arguments, which the reference CPU branch ignores).
    With `new_key` / `new_value` ([users, nkv, hd] bf16) the same launch first writes those rows
    into the caches at `cur_pos`, i.e. it is `paged_update_cache` + decode in one kernel;
    `wrap_negative_positions=False` skips rows with a negative position instead of wrapping them
    the way the reference's CPU indexing does."""
    _need_cuda(query, k_cache, v_cache, page_table, cur_pos, out, new_key, new_value)
    nb, nkv, bs, hd = _check_cache(k_cache, v_cache)
    orig_shape = query.shape
    if query.dim() == 4:
        if query.shape[0] != 1:
            raise ValueError("4-D query must be [1, users, nq, hd]")
        query = query[0]
    if query.dim() != 3 or query.shape[2] != hd:
        raise ValueError(f"query must be [users, nq, {hd}], got {tuple(orig_shape)}")
    users, nq = query.shape[0], query.shape[1]
    if nq % nkv != 0:
        raise ValueError(f"num_q_heads {nq} is not a multiple of num_kv_heads {nkv}")
    q, qstride = _token_major(query, nq, hd, "query")
    if out is None:
        out_t = torch.empty((users, nq, hd), dtype=torch.bfloat16, device=query.device)
    else:
        out_t = out.reshape(users, nq, hd) if out.dim() != 3 else out
        if out_t.dtype != torch.bfloat16 or out_t.stride(2) != 1 or out_t.stride(1) != hd:
            raise ValueError("out must be a dense-row bfloat16 tensor")
        if out_t.data_ptr() != out.data_ptr():
            raise ValueError("out must be viewable as [users, nq, hd] without a copy")
    ostride = out_t.stride(0) if users > 1 else max(out_t.stride(0), nq * hd)
    _i32(page_table, "page_table")
    _i32(cur_pos, "cur_pos")
    if page_table.stride(1) != 1 or not cur_pos.is_contiguous() or cur_pos.numel() != users:
        raise ValueError("page_table rows must be dense and cur_pos must hold one entry per user")
    if scale is None:
        scale = hd ** -0.5
    L = _lib.lib()
    if sinks is not None:
        _need_cuda(sinks)
        if sinks.dtype != torch.float32 or sinks.numel() != nq or not sinks.is_contiguous():
            raise ValueError("sinks must be a dense float32 tensor with one entry per q head")
    if num_splits == 0:
        num_splits = _env_num_splits()
    if num_splits == 0:
        ctx = max_context_len if max_context_len > 0 else page_table.shape[1] * bs
        if sliding_window > 0:
            ctx = min(ctx, sliding_window + 64)
        num_splits = L.b200attn_decode_auto_splits(users, nkv, hd, ctx)
    need = L.b200attn_decode_workspace_bytes(users, nq, hd, num_splits)
    ws = workspace if workspace is not None else _workspace(query.device, need)
    kn = vn = None
    nstride = 0
    if (new_key is None) != (new_value is None):
        raise ValueError("new_key and new_value go together")
    if new_key is not None:
        kn, nstride = _token_major(new_key, nkv, hd, "new_key")
        vn, vstride = _token_major(new_value, nkv, hd, "new_value")
        if kn.shape[0] != users or vn.shape[0] != users:
            raise ValueError("new_key / new_value must hold one row per user")
        if vstride != nstride:
            kn, vn, nstride = kn.contiguous(), vn.contiguous(), nkv * hd
    _lib.check(
        "b200attn_paged_decode_step",
        L.b200attn_paged_decode_step(
            out_t.data_ptr(), ostride, q.data_ptr(), qstride, k_cache.data_ptr(),
            v_cache.data_ptr(), kn.data_ptr() if kn is not None else None,
            vn.data_ptr() if vn is not None else None, nstride,
            1 if wrap_negative_positions else 0,
            page_table.data_ptr(), page_table.stride(0), page_table.shape[1],
            cur_pos.data_ptr(), users, nq, nkv, hd, bs, nb, float(scale), int(sliding_window),
            sinks.data_ptr() if sinks is not None else None, _cache_dtype(k_cache), max_context_len,
            num_splits, ws.data_ptr() if ws is not None else None,
            ws.numel() * ws.element_size() if ws is not None else 0, _stream(query),
        ),
    )
    if out is not None:
        return out
    return out_t.reshape(orig_shape)


def prefill(
    query: torch.Tensor,
    k_src: torch.Tensor,
    v_src: torch.Tensor,
    cu_q_host: torch.Tensor,
    scale: Optional[float] = None,
    page_table: Optional[torch.Tensor] = None,
    q_start: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    cu_q: Optional[torch.Tensor] = None,
    sliding_window: int = 0,
) -> torch.Tensor:
    """Causal varlen prefill (`tt.scaled_dot_product_attention`, custom_ops.py:635-742) when
    `page_table` is None and `k_src`/`v_src` are the fresh [tokens, nkv, hd] K/V of the same
    tokens; chunked prefill over the paged cache
    (`tt.chunked_scaled_dot_product_attention`, custom_ops.py:1334-1443) when `page_table` is
    given and `k_src`/`v_src` are the caches.  `query`: [tokens, nq, hd] with sequence s owning
    rows cu_q[s]:cu_q[s+1]; `q_start[s]` is the absolute position of its first row."""
    _need_cuda(query, k_src, v_src, page_table, q_start, out, cu_q)
    if cu_q_host.is_cuda or cu_q_host.dtype != torch.int32 or not cu_q_host.is_contiguous():
        raise ValueError("cu_q_host must be a dense int32 CPU tensor")
    num_seqs = cu_q_host.numel() - 1
    if query.dim() != 3:
        raise ValueError(f"query must be [tokens, nq, hd], got {tuple(query.shape)}")
    total_q, nq, hd = query.shape
    q, qstride = _token_major(query, nq, hd, "query")
    paged = page_table is not None
    if paged:
        nb, nkv, bs, _hd = _check_cache(k_src, v_src)
        if _hd != hd:
            raise ValueError("cache head_size differs from query head_size")
        _i32(page_table, "page_table")
        if page_table.stride(1) != 1 or page_table.shape[0] < num_seqs:
            raise ValueError("page_table must have one dense row per sequence")
        kstride = 0
        k, v = k_src, v_src
    else:
        if q_start is not None:
            raise ValueError("q_start needs the paged form (the prefix lives in the cache)")
        if k_src.dim() != 3 or k_src.shape != v_src.shape or k_src.shape[2] != hd:
            raise ValueError("fresh k_src/v_src must be [tokens, nkv, hd]")
        if k_src.shape[0] != total_q:
            raise ValueError("fresh K/V must cover the same tokens as the query")
        nkv = k_src.shape[1]
        k, kstride = _token_major(k_src, nkv, hd, "k_src")
        v, vstride = _token_major(v_src, nkv, hd, "v_src")
        if kstride != vstride:
            k, v = k.contiguous(), v.contiguous()
            kstride = nkv * hd
        nb, bs = 0, 64
    if nq % nkv != 0:
        raise ValueError(f"num_q_heads {nq} is not a multiple of num_kv_heads {nkv}")
    if q_start is not None:
        _i32(q_start, "q_start")
        if q_start.numel() != num_seqs or not q_start.is_contiguous():
            raise ValueError("q_start must hold one dense entry per sequence")
    if cu_q is None:
        cu_q = cu_q_host.to(query.device, non_blocking=True)
    _i32(cu_q, "cu_q")
    if paged and k_src.dtype == torch.float8_e4m3fn:
        # The tcgen05 kernel takes 16-bit tiles: widen the pages this batch reads into a bf16
        # scratch pool laid out [sequence][page slot] and attend over that through the identity
        # page table.  e4m3 -> bf16 is exact, so the kernel sees the cache's own values.
        k, v, page_table, nb = _widen_fp8_pages(k_src, v_src, page_table, cu_q, q_start, num_seqs)
    if out is None:
        out_t = torch.empty((total_q, nq, hd), dtype=torch.bfloat16, device=query.device)
    else:
        out_t = out.reshape(total_q, nq, hd) if out.dim() != 3 else out
        if out_t.dtype != torch.bfloat16 or out_t.stride(2) != 1 or out_t.stride(1) != hd:
            raise ValueError("out must be a dense-row bfloat16 tensor")
        if out_t.data_ptr() != out.data_ptr():
            raise ValueError("out must be viewable as [tokens, nq, hd] without a copy")
    ostride = out_t.stride(0) if total_q > 1 else max(out_t.stride(0), nq * hd)
    if scale is None:
        scale = hd ** -0.5
    L = _lib.lib()
    _lib.check(
        "b200attn_prefill_ex",
        L.b200attn_prefill_ex(
            out_t.data_ptr(), ostride, q.data_ptr(), qstride, k.data_ptr(), v.data_ptr(),
            1 if paged else 0, kstride,
            page_table.data_ptr() if paged else None,
            page_table.stride(0) if paged else 0, page_table.shape[1] if paged else 0,
            cu_q.data_ptr(), cu_q_host.data_ptr(),
            q_start.data_ptr() if q_start is not None else None,
            num_seqs, total_q, nq, nkv, hd, bs, nb, float(scale), int(sliding_window),
            _stream(query),
        ),
    )
    return out if out is not None else out_t


_fp8_scratch: dict[tuple, tuple] = {}


def _widen_fp8_pages(k_cache, v_cache, page_table, cu_q, q_start, num_seqs):
    """bf16 copies of the pages `page_table[:num_seqs]` lists for an e4m3 cache pair; returns
    (k_pool, v_pool, identity page table, pool size in pages).  The scratch is cached per
    (device, stream) and grown on demand; torch owns it."""
    nb, nkv, bs, hd = k_cache.shape
    width = page_table.shape[1]
    pages = num_seqs * width
    dev = k_cache.device
    key = (dev.index or 0, torch.cuda.current_stream(dev).cuda_stream, nkv, bs, hd)
    have = _fp8_scratch.get(key)
    if have is None or have[0].shape[0] < pages:
        if have is not None:
            _retired_workspaces.extend(have[:2])
        grow = max(pages, 2 * have[0].shape[0] if have is not None else 0)
        have = (torch.empty((grow, nkv, bs, hd), dtype=torch.bfloat16, device=dev),
                torch.empty((grow, nkv, bs, hd), dtype=torch.bfloat16, device=dev), {})
        _fp8_scratch[key] = have
    k_pool, v_pool, tables = have
    ident = tables.get((num_seqs, width))
    if ident is None:
        ident = torch.arange(pages, dtype=torch.int32, device=dev).reshape(num_seqs, width)
        tables[(num_seqs, width)] = ident
    _lib.check(
        "b200attn_dequant_pages_fp8",
        _lib.lib().b200attn_dequant_pages_fp8(
            k_pool.data_ptr(), v_pool.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
            page_table.data_ptr(), page_table.stride(0), width, cu_q.data_ptr(),
            q_start.data_ptr() if q_start is not None else None, num_seqs, nkv, hd, bs, nb,
            torch.cuda.current_stream(dev).cuda_stream,
        ),
    )
    return k_pool, v_pool, ident, k_pool.shape[0]


def read_error_word(device: Optional[torch.device] = None) -> int:
    """Returns and clears the device diagnostics word (0 = clean, 1 = a bounded wait ran out,
    2 = a page id or slot pointed outside the cache)."""
    word = ctypes.c_int32(0)
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        _lib.check(
            "b200attn_read_error_word",
            _lib.lib().b200attn_read_error_word(
                ctypes.byref(word), torch.cuda.current_stream(dev).cuda_stream
            ),
        )
    if word.value:
        # an aborted launch may have left arrival counters behind: start the scratch afresh
        for ws in list(_workspaces.values()) + _retired_workspaces:
            if ws.device == dev:
                ws[:TICKET_BYTES].zero_()
    return int(word.value)


class ErrorWordWatch:
    """Once-per-step watch on the device diagnostics word for a serving loop.  `poll()` raises if
    an EARLIER poll's asynchronous copy found the word set, then queues the next copy on the
    current stream; it never synchronises.  A kernel that gave up on a bounded wait (word 1) or
    met a page id outside the cache (word 2) is therefore reported a step or two later instead
    of passing silently."""

    MESSAGES = {
        1: "a bounded wait inside a b200attn kernel ran out (diagnostics word 1): outputs of the "
           "launches around it are invalid; a row-parallel communicator involved must be rebuilt",
        2: "a page id or slot outside the KV cache reached a b200attn kernel (diagnostics word 2): "
           "the access was skipped; the step's metadata is inconsistent with the cache",
    }

    # called with the word's value before poll() raises (e.g. to switch a fused path off)
    on_error: list = []

    def __init__(self, device: Optional[torch.device] = None):
        self.device = device if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self._host = torch.zeros(1, dtype=torch.int32)
        if torch.cuda.is_available():
            self._host = self._host.pin_memory()

    def value(self) -> int:
        return int(self._host[0])

    def poll(self) -> None:
        word = self.value()
        if word:
            self._host.zero_()
            for react in list(self.on_error):
                react(word)
            if self.device.type == "cuda" and torch.cuda.is_available():
                read_error_word(self.device)      # clear on the device too
            raise RuntimeError(self.MESSAGES.get(word, f"device diagnostics word {word}"))
        _lib.check(
            "b200attn_peek_error_word_async",
            _lib.lib().b200attn_peek_error_word_async(
                self._host.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream),
        )
