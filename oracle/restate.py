"""CPU restatement (plain torch tensor ops) of the reference's CPU branches for the attention
and KV-cache ops.  TEST INFRASTRUCTURE ONLY — see the package docstring.

Each function follows one `device.type == "cpu"` branch of
python_package/tt_torch/custom_ops.py, generalised only where the reference's CPU branch is
narrower than its device op (GQA decode, multi-user fill); those generalisations equal looping
the reference op per KV-head group / per user, which the golden generator does literally.

Arithmetic dtype: the functions compute in the dtype they are given (as the reference does).
Tests pass fp32 copies of the bf16 tensors for the primary comparison and native bf16 for the
"what the reference itself would produce" comparison.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def quantize_kv_fp8(x: torch.Tensor) -> torch.Tensor:
    """What the plugin's cache write does to K / V rows for an fp8 cache (attention.py:692-700):
    clamp to the finite range of the cache dtype, then cast (round to nearest even).  No scale."""
    info = torch.finfo(torch.float8_e4m3fn)
    return x.float().clamp(info.min, info.max).to(torch.float8_e4m3fn)


def paged_update_cache(
    cache: torch.Tensor,
    fill_value: torch.Tensor,
    update_indices: torch.Tensor,
    page_table: torch.Tensor,
) -> torch.Tensor:
    """custom_ops.py:962-1000.  cache [nb,nkv,bs,hd]; fill_value [1,users,nkv_in,hd];
    update_indices [users]; page_table [users,nblk].  Returns a new cache."""
    cache = cache.clone()
    num_users = update_indices.shape[0]
    block_size = cache.shape[-2]
    num_heads = cache.shape[-3]
    idx = update_indices.to(torch.int64)
    # torch `//` and `%` on integer tensors floor, like Python (custom_ops.py:985-988)
    block_indices = torch.div(idx, block_size, rounding_mode="floor")
    block_offsets = torch.remainder(idx, block_size)
    user_range = torch.arange(num_users)
    blocks = page_table.to(torch.int64)[user_range, block_indices]  # negative columns wrap
    rows = fill_value[0, :, :num_heads, :]
    cache[blocks, :, block_offsets, :] = (
        quantize_kv_fp8(rows) if cache.dtype == torch.float8_e4m3fn else rows)
    return cache


def paged_fill_cache(
    cache: torch.Tensor,
    fill_value: torch.Tensor,
    page_table: torch.Tensor,
    batch_idx: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """custom_ops.py:1016-1092, for every user of the batch: user u's fill_value[u] ([nkv,T,hd])
    goes to blocks page_table[batch_idx[u]], whole blocks first, then the tail of the last
    block.  (The reference CPU branch does this for one user per call, custom_ops.py:1044.)"""
    cache = cache.clone()
    users, num_heads, fill_seq_len, hd = fill_value.shape
    block_size = cache.shape[-2]
    if batch_idx is None:
        batch_idx = torch.arange(users, dtype=torch.int32)
    full = fill_seq_len // block_size
    tail = fill_seq_len % block_size
    if cache.dtype == torch.float8_e4m3fn:
        fill_value = quantize_kv_fp8(fill_value)
    for u in range(users):
        blocks = page_table[int(batch_idx[u])].to(torch.int64)
        fv = fill_value[u]
        if full > 0:
            # [nkv, full*bs, hd] -> [full, nkv, bs, hd]
            body = fv[:, : full * block_size, :].reshape(num_heads, full, block_size, hd)
            cache[blocks[:full]] = body.transpose(0, 1)
        if tail > 0:
            cache[blocks[full], :, :tail, :] = fv[:, full * block_size:, :]
    return cache


def _gather_user_kv(cache: torch.Tensor, block_ids: torch.Tensor) -> torch.Tensor:
    """[nblk] block ids -> [nkv, nblk*bs, hd] (custom_ops.py:1274-1292, 1381-1398)."""
    blocks = cache[block_ids.to(torch.int64)]            # [nblk, nkv, bs, hd]
    nblk, nkv, bs, hd = blocks.shape
    return blocks.transpose(0, 1).reshape(nkv, nblk * bs, hd)


def paged_sdpa_decode(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    page_table: torch.Tensor,
    cur_pos: torch.Tensor,
    scale: Optional[float] = None,
    sliding_window: Optional[int] = None,
    sinks: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """custom_ops.py:1256-1312 with is_causal=True, for nq >= nkv (GQA: query head h reads KV
    head h // (nq/nkv), the `repeat_interleave` the reference intends at :1305-1306).
    query [1,users,nq,hd]; key/value caches [nb,nkv,bs,hd]; returns [1,users,nq,hd].
    Rows with cur_pos < 0 yield NaN here exactly as in the reference (softmax of all -inf).

    `sliding_window` and `sinks` are the op's `sliding_window_size` / `attention_sink`
    arguments (custom_ops.py:1206-1207), which the reference's CPU branch accepts and ignores.
    PARITY UNPINNED for these two: they follow the published definitions (a user at position p
    attends keys p-W < j <= p; a sink is one extra softmax column per head whose weight is
    dropped), not reference output."""
    _, users, nq, hd = query.shape
    nkv, bs = key.shape[1], key.shape[2]
    rep = nq // nkv
    nblk = page_table.shape[1]
    max_seq = nblk * bs
    dt = query.dtype
    scale = 1 / hd**0.5 if scale is None else scale
    out = torch.empty(users, nq, hd, dtype=dt)
    for u in range(users):
        k = _gather_user_kv(key, page_table[u]).to(dt).repeat_interleave(rep, 0)   # [nq,S,hd]
        v = _gather_user_kv(value, page_table[u]).to(dt).repeat_interleave(rep, 0)
        mask = torch.zeros(max_seq, dtype=dt)
        mask[int(cur_pos[u]) + 1:] = float("-inf")
        if sliding_window:
            mask[: max(0, int(cur_pos[u]) + 1 - int(sliding_window))] = float("-inf")
        w = query[0, u].unsqueeze(1) @ k.transpose(-2, -1) * scale               # [nq,1,S]
        w = w + mask
        if sinks is not None:
            w = torch.cat([w, sinks.to(dt).view(nq, 1, 1)], dim=-1)
            w = torch.softmax(w, dim=-1)[..., :-1]
        else:
            w = torch.softmax(w, dim=-1)
        out[u] = (w @ v).squeeze(1)
    return out.reshape(1, users, nq, hd)


def sdpa(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    is_causal: bool = True,
    scale: Optional[float] = None,
    sliding_window: Optional[int] = None,
) -> torch.Tensor:
    """custom_ops.py:717-727: torch's scaled_dot_product_attention with enable_gqa, written out
    as softmax(Q K^T * scale + causal mask) V.  query [B,nq,T,hd]; key/value [B,nkv,S,hd].
    `sliding_window` (the op's `sliding_window_size`, ignored by the reference's CPU branch;
    PARITY UNPINNED) keeps keys i-W < j <= i for query row i."""
    B, nq, T, hd = query.shape
    nkv, S = key.shape[1], key.shape[2]
    rep = nq // nkv
    scale = 1 / math.sqrt(hd) if scale is None else scale
    k = key.repeat_interleave(rep, 1)
    v = value.repeat_interleave(rep, 1)
    w = query @ k.transpose(-2, -1) * scale
    if is_causal:
        keep = torch.ones(T, S, dtype=torch.bool).tril()
        if sliding_window:
            keep &= torch.ones(T, S, dtype=torch.bool).triu(1 - int(sliding_window))
        w = w.masked_fill(~keep, float("-inf"))
    w = torch.softmax(w, dim=-1)
    return w @ v


def chunked_sdpa(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    page_table: torch.Tensor,
    chunk_start: int,
    scale: Optional[float] = None,
    sliding_window: Optional[int] = None,
) -> torch.Tensor:
    """custom_ops.py:1376-1433.  query [users,nq,T,hd] at absolute positions chunk_start+i;
    key/value caches; page_table [users,nblk] (prefix + chunk).  Returns [users,nq,T,hd].
    `sliding_window`: as in `sdpa` (PARITY UNPINNED; the reference op has no such argument on
    its CPU branch)."""
    users, nq, T, hd = query.shape
    nkv, bs = key.shape[1], key.shape[2]
    s_len = page_table.shape[1] * bs
    rep = nq // nkv
    dt = query.dtype
    scale = 1.0 / hd**0.5 if scale is None else scale
    gk = torch.stack([_gather_user_kv(key, page_table[u]) for u in range(users)]).to(dt)
    gv = torch.stack([_gather_user_kv(value, page_table[u]) for u in range(users)]).to(dt)
    if rep != 1:
        gk = gk.repeat_interleave(rep, dim=1)
        gv = gv.repeat_interleave(rep, dim=1)
    attn = torch.matmul(query, gk.transpose(-2, -1)) * scale
    q_pos = chunk_start + torch.arange(T).view(T, 1)
    k_pos = torch.arange(s_len).view(1, s_len)
    keep = k_pos <= q_pos
    if sliding_window:
        keep = keep & (k_pos > q_pos - int(sliding_window))
    attn = attn.masked_fill(~keep.view(1, 1, T, s_len), float("-inf"))
    attn = torch.softmax(attn, dim=-1)
    return torch.matmul(attn, gv)


def rotary_embedding(
    positions: torch.Tensor,
    query: torch.Tensor,
    key: torch.Tensor,
    inv_freq: torch.Tensor,
    head_size: int,
    rotary_dim: int,
):
    """integrations/vllm_plugin/vllm_tt/layers/rotary_embedding.py:51-66 with the NeoX-style
    rotation of vLLM's ApplyRotaryEmb.forward_static: cos / sin from fp32 `positions x inv_freq`,
    cast to the query dtype, then `o1 = x1*cos - x2*sin`, `o2 = x2*cos + x1*sin` in that dtype.
    query [tokens, nq*hd], key [tokens, nkv*hd]; returns the rotated pair."""
    pos = positions.flatten().to(torch.float32)
    n = pos.shape[0]
    freqs = torch.outer(pos, inv_freq)
    cos = freqs.cos().to(query.dtype).unsqueeze(-2)
    sin = freqs.sin().to(query.dtype).unsqueeze(-2)

    def rot(x):
        shape = x.shape
        x = x.view(n, -1, head_size)
        xr = x[..., :rotary_dim]
        x1, x2 = torch.chunk(xr, 2, dim=-1)
        o = torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)
        if rotary_dim != head_size:
            o = torch.cat((o, x[..., rotary_dim:]), dim=-1)
        return o.reshape(shape)

    return rot(query), rot(key)


# ------------------------------------------------------------------------------------------
# The plugin's forward (attention.py:273-336) restated on top of the ops above, for batches in
# the plugin's [users x tokens] form.  Returns (output, new_k_cache, new_v_cache).
# ------------------------------------------------------------------------------------------
def impl_forward(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    num_heads: int,
    num_kv_heads: int,
    head_size: int,
    scale: float,
    num_users: int,
    cache_position: torch.Tensor,
    page_table: torch.Tensor,
    fill_page_table: Optional[torch.Tensor] = None,
    batch_idx: Optional[torch.Tensor] = None,
    chunk_start_idx: Optional[torch.Tensor] = None,
    compute_dtype: Optional[torch.dtype] = None,
    sliding_window: Optional[int] = None,
    sinks: Optional[torch.Tensor] = None,
):
    q = query.reshape(num_users, -1, num_heads, head_size)
    k = key.reshape(num_users, -1, num_kv_heads, head_size)
    v = value.reshape(num_users, -1, num_kv_heads, head_size)
    T = q.shape[1]
    dt = compute_dtype or query.dtype
    if T == 1:  # decode (attention.py:468-484, 634-668)
        k_cache = paged_update_cache(k_cache, k.transpose(0, 1), cache_position, page_table)
        v_cache = paged_update_cache(v_cache, v.transpose(0, 1), cache_position, page_table)
        out = paged_sdpa_decode(
            q.transpose(0, 1).to(dt), k_cache.to(dt), v_cache.to(dt), page_table,
            cache_position, scale, sliding_window, sinks,
        ).transpose(0, 1)
    else:       # prefill (attention.py:485-511, 545-598)
        assert sinks is None, "Attention sink is unsupported in SDPA prefill"  # attention.py:321
        fpt = fill_page_table if fill_page_table is not None else page_table
        k_cache = paged_fill_cache(k_cache, k.transpose(1, 2), fpt, batch_idx)
        v_cache = paged_fill_cache(v_cache, v.transpose(1, 2), fpt, batch_idx)
        if chunk_start_idx is not None:
            out = chunked_sdpa(
                q.transpose(1, 2).to(dt), k_cache.to(dt), v_cache.to(dt), page_table,
                int(chunk_start_idx.reshape(-1)[0]), scale, sliding_window,
            ).transpose(1, 2)
        else:
            out = sdpa(
                q.transpose(1, 2).to(dt), k.transpose(1, 2).to(dt), v.transpose(1, 2).to(dt),
                True, scale, sliding_window,
            ).transpose(1, 2)
    return out.reshape(-1, num_heads * head_size), k_cache, v_cache
