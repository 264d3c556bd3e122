"""Sliding-window ring caches: geometry, per-request sub-ring bookkeeping and the rotated page
table (host mirror of integrations/vllm_plugin/vllm_tt/swa_cache_utils.py and of the runner lines
that feed it, model_runner.py:1753-1815).

A sliding-window layer does not need the whole block pool: every request owns a small ring of
`window_blocks` physical blocks, logical block b of the request lives in ring position
`b % window_blocks`, and the attention ops are handed (a) a page table whose columns list the ring
positions of the last `window_blocks` logical blocks in logical order and (b) the newest token's
position counted from the first listed block.  With those two the unchanged decode kernel, given
`sliding_window`, reads exactly the window (the kernels take positions relative to the page table,
so nothing in them knows about the ring).

Pure integer / numpy code, same names and argument meaning as the reference helpers.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

# A page-table row of a sliding group holds window_blocks int32 ids and must be a multiple of
# 32 bytes long (swa_cache_utils.py:20-22), hence a multiple of 8 ids.
PAGE_TABLE_STICK_BLOCK_ALIGNMENT = 8


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def sliding_window_blocks(sliding_window: int, block_size: int, max_model_len: int) -> int:
    """Ring length in blocks (swa_cache_utils.py:25-42): enough blocks for a window that
    straddles a block boundary (one more than the window's own block count), rounded up to the
    page-table row alignment; a window longer than any request can get is cut to
    `max_model_len` first."""
    effective = sliding_window if sliding_window < max_model_len else max_model_len
    blocks = _ceil_div(effective, block_size) + 1
    a = PAGE_TABLE_STICK_BLOCK_ALIGNMENT
    return _ceil_div(blocks, a) * a


def sliding_ring_is_profitable(sliding_window: int, block_size: int, max_model_len: int) -> bool:
    """True when the ring is shorter than the blocks a full-length request would take from the
    pool (swa_cache_utils.py:45-57); otherwise the layer is better left in the pool."""
    full = _ceil_div(max_model_len, block_size)
    return sliding_window_blocks(sliding_window, block_size, max_model_len) < full


def sliding_ring_phys_blocks(window_blocks: int, max_num_reqs: int) -> int:
    """Blocks of one sliding layer's cache tensor: block 0 is the null block padded rows write
    to, then one sub-ring per batch slot (swa_cache_utils.py:60-63)."""
    return 1 + window_blocks * max_num_reqs


def sliding_ring_reserve_bytes(window_blocks: int, max_num_reqs: int, page_size_bytes: int) -> int:
    """Bytes of that tensor in the accounting unit of the block pool, i.e. with the un-sharded
    page size (swa_cache_utils.py:66-78)."""
    return page_size_bytes * sliding_ring_phys_blocks(window_blocks, max_num_reqs)


def sliding_page_table_width(window_blocks: int, base_width: int) -> int:
    """Columns of a sliding group's page table: the ring length, unless the full-attention
    buffer is narrower still (swa_cache_utils.py:81-84)."""
    return base_width if base_width < window_blocks else window_blocks


def assign_ring_slots(
    row_req_ids: Sequence[str],
    batch_req_ids: Sequence[str],
    req_ring_slot: Dict[str, int],
    free_ring_slots: List[int],
) -> np.ndarray:
    """Slot (sub-ring index) of every request in `row_req_ids` (swa_cache_utils.py:87-122).

    A request keeps one slot for life, whatever batch row it moves to.  Requests that are no
    longer anywhere in `batch_req_ids` give their slot back first; a request seen for the first
    time takes the lowest free slot.  Both containers are updated in place.  Raises IndexError
    when more requests are live than there are slots."""
    live = frozenset(batch_req_ids)
    gone = [rid for rid in req_ring_slot if rid not in live]
    for rid in gone:
        free_ring_slots.append(req_ring_slot.pop(rid))
    free_ring_slots.sort(reverse=True)            # lowest slot at the end, popped first
    out = np.empty(len(row_req_ids), dtype=np.int64)
    for i, rid in enumerate(row_req_ids):
        if rid not in req_ring_slot:
            req_ring_slot[rid] = free_ring_slots.pop()
        out[i] = req_ring_slot[rid]
    return out


def build_sliding_ring_page_table(
    start_block: np.ndarray, slots: np.ndarray, window_blocks: int, width: int
) -> np.ndarray:
    """[rows, width] page table into the sub-rings (swa_cache_utils.py:125-137): column c of row
    i is the physical block of logical block `start_block[i] + c`, which sits at ring position
    `(start_block[i] + c) % window_blocks` of sub-ring `slots[i]`; sub-ring s begins at physical
    block `1 + s * window_blocks`."""
    start_block = np.asarray(start_block, dtype=np.int64).reshape(-1, 1)
    base = 1 + np.asarray(slots, dtype=np.int64).reshape(-1, 1) * window_blocks
    ring_pos = np.mod(start_block + np.arange(width, dtype=np.int64).reshape(1, -1), window_blocks)
    return base + ring_pos


def ring_window_view(
    seq_lens: np.ndarray, block_size: int, window_blocks: int
) -> Tuple[np.ndarray, np.ndarray]:
    """(start_block, cache_position) of the rows of a sliding group (model_runner.py:1758-1761,
    1812-1815): the page table lists the last `min(blocks so far, window_blocks)` logical blocks,
    so it starts at `start_block`, and the newest token's position is counted from there.
    Contexts that still fit the ring give start_block 0 and the absolute position."""
    cur = np.asarray(seq_lens, dtype=np.int64) - 1
    cur_block = cur // block_size
    listed = np.minimum(cur_block + 1, window_blocks)
    start_block = cur_block - listed + 1
    return start_block, cur - start_block * block_size


def check_sliding_prefill_supported(
    start_block: np.ndarray, num_scheduled: np.ndarray, num_computed: np.ndarray
) -> None:
    """The reference fills a ring only from its beginning (model_runner.py:1762-1779): a row that
    writes more than one token must start at block 0 of its ring with nothing computed before.
    Same refusal, same message."""
    filling = np.asarray(num_scheduled) > 1
    bad = filling & ((np.asarray(start_block) > 0) | (np.asarray(num_computed) > 0))
    if np.any(bad):
        raise NotImplementedError(
            "sliding-window prefill for context > window or with "
            "prefix caching / chunked prefill (num_computed > 0) is "
            "not yet supported on TT"
        )
