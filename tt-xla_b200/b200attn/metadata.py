"""Step-metadata arithmetic of the plugin's runner, as pure functions, plus the one-launch GPU
builder that replaces the per-step host loop and host-to-device copies.

Mirrors the parts of integrations/vllm_plugin/vllm_tt/model_runner.py that decide what the
attention path receives:
    seq_lens = num_computed + num_scheduled                      (:1722-1725)
    cache_position = seq_lens - 1, -1 on unused rows             (:1734-1741)
    page_table[:n] = block_table rows, unused / parked rows -> 0 (:1945-1983)
    fill_page_table[i] = roll(page_table[i], -num_computed_i // block_size), narrowed to
        the step's width                                          (:1955-1993, :1255-1286)
    chunk_start_idx = the one shared num_computed - row_lead      (:1863-1887)
    _row_lead / _same_block_run                                  (:5284-5307)
and the slot addressing the live path implies (slot = page_table[u, p // bs] * bs + p % bs).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def row_lead(num_computed: np.ndarray, block_size: int) -> np.ndarray:
    """Tokens to re-feed so each row starts on its KV block boundary (model_runner.py:5301-5307)."""
    return (np.asarray(num_computed) % block_size).astype(np.int32)


def same_block_run(num_computed: np.ndarray, block_size: int) -> int:
    """Length of the leading run of requests sharing one KV block boundary
    (model_runner.py:5284-5298)."""
    num_computed = np.asarray(num_computed)
    if num_computed.size == 0:
        return 0
    boundary = num_computed // block_size
    differs = np.flatnonzero(boundary != boundary[0])
    return int(differs[0]) if differs.size else int(num_computed.size)


def fill_page_table_width(max_num_tokens: int, block_size: int, read_width: int) -> int:
    """Columns the fill page table needs: the step's token budget in blocks, rounded up to 8
    entries, capped at the read table's width (model_runner.py:1255-1286)."""
    width = cdiv(cdiv(max_num_tokens, block_size), 8) * 8
    fill_width = min(width, read_width)
    assert fill_width * block_size >= max_num_tokens, (
        f"fill page table ({fill_width} cols x block_size {block_size}) cannot cover a "
        f"{max_num_tokens}-token step"
    )
    return fill_width


@dataclass
class StepMetadata:
    cache_position: torch.Tensor     # [rows] i32
    page_table: torch.Tensor         # [rows, width] i32
    fill_page_table: torch.Tensor    # [rows, fill_width] i32
    slot_mapping: torch.Tensor       # [rows * tokens_per_row] i64, -1 on padding
    chunk_start_idx: Optional[torch.Tensor]   # [1] i32 or None


def build_step_metadata_host(
    num_computed: torch.Tensor,
    num_scheduled: torch.Tensor,
    block_table: torch.Tensor,
    block_size: int,
    rows: int,
    tokens_per_row: int,
    fill_width: int,
) -> StepMetadata:
    """Host statement of one pass of the runner's metadata build for `n = len(num_scheduled)`
    live requests padded to `rows` rows of `tokens_per_row` tokens.  CPU tensors in and out;
    this is what the GPU builder is checked against."""
    n = num_scheduled.numel()
    width = block_table.shape[1]
    seq_lens = (num_computed[:n] + num_scheduled).to(torch.int32)
    cache_position = torch.full((rows,), -1, dtype=torch.int32)
    cache_position[:n] = seq_lens - 1
    page_table = torch.zeros((rows, width), dtype=torch.int32)
    page_table[:n] = block_table[:n]
    parked = (num_scheduled == 0).nonzero().flatten()
    page_table[parked] = 0
    fill = page_table.clone()
    for i in range(n):
        off = int(num_computed[i]) // block_size
        if off > 0:
            fill[i] = torch.roll(page_table[i], shifts=-off)
    fill_page_table = fill[:, :fill_width].contiguous()
    slot = torch.full((rows, tokens_per_row), -1, dtype=torch.int64)
    for i in range(n):
        for t in range(int(num_scheduled[i])):
            p = int(num_computed[i]) + t
            slot[i, t] = int(page_table[i, p // block_size]) * block_size + p % block_size
    chunk_start = None
    if tokens_per_row > 1 and n > 0:
        lead = row_lead(num_computed[:n].numpy(), block_size)
        starts = num_computed[:n].numpy() - lead
        live = num_scheduled.numpy() > 0
        if live.any() and int(starts[live].max()) > 0:
            if len(set(starts[live].tolist())) != 1:
                raise ValueError("rows of one multi-token pass must share their chunk start")
            chunk_start = torch.tensor([int(starts[live][0])], dtype=torch.int32)
    return StepMetadata(cache_position, page_table, fill_page_table, slot.reshape(-1),
                        chunk_start)


def build_step_metadata(
    num_computed: torch.Tensor,
    num_scheduled: torch.Tensor,
    block_table: torch.Tensor,
    block_size: int,
    out: StepMetadata,
    tokens_per_row: int,
) -> None:
    """GPU builder: one launch fills the persistent buffers of `out` (cache_position, page_table,
    fill_page_table, slot_mapping) from device-resident `num_computed` / `num_scheduled` [n] and
    `block_table` [>= n, width].  Nothing is copied from the host."""
    for t in (num_computed, num_scheduled, block_table, out.cache_position, out.page_table,
              out.fill_page_table, out.slot_mapping):
        if not t.is_cuda:
            raise RuntimeError("build_step_metadata runs on CUDA tensors only")
    n = num_scheduled.numel()
    rows, width = out.page_table.shape
    if block_table.shape[1] != width or block_table.stride(1) != 1:
        raise ValueError("block_table must have the page table's width and dense rows")
    for t, dt in ((num_computed, torch.int32), (num_scheduled, torch.int32),
                  (block_table, torch.int32), (out.cache_position, torch.int32),
                  (out.page_table, torch.int32), (out.fill_page_table, torch.int32),
                  (out.slot_mapping, torch.int64)):
        if t.dtype != dt:
            raise ValueError("step metadata tensors are int32 (slot_mapping int64)")
    if out.slot_mapping.numel() != rows * tokens_per_row:
        raise ValueError("slot_mapping must hold rows * tokens_per_row entries")
    _lib.check(
        "b200attn_build_step_metadata",
        _lib.lib().b200attn_build_step_metadata(
            num_computed.data_ptr(), num_scheduled.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), n, rows, width, out.fill_page_table.shape[1], tokens_per_row,
            block_size, out.cache_position.data_ptr(), out.page_table.data_ptr(),
            out.fill_page_table.data_ptr(), out.slot_mapping.data_ptr(),
            torch.cuda.current_stream(num_computed.device).cuda_stream,
        ),
    )
