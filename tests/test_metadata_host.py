"""Runner-side metadata arithmetic (device free).  Cases follow the reference's device-free tests
tests/integrations/vllm_plugin/test_prepare_inputs_block_alignment.py and
test_fill_page_table_width.py."""
import numpy as np
import pytest
import torch

from b200attn import metadata as md
from oracle import restate
from oracle.inputs import randn_bf16

BLOCK = 32


def test_row_lead():
    assert md.row_lead(np.array([0, 32, 64, 256], dtype=np.int32), BLOCK).tolist() == [0, 0, 0, 0]
    assert md.row_lead(np.array([41, 44, 63, 65], dtype=np.int32), BLOCK).tolist() == [9, 12, 31, 1]
    assert md.row_lead(np.array([41], dtype=np.int64), BLOCK).dtype == np.int32


def test_same_block_run():
    assert md.same_block_run(np.array([33, 40, 63], dtype=np.int32), BLOCK) == 3
    assert md.same_block_run(np.array([41, 20], dtype=np.int32), BLOCK) == 1
    assert md.same_block_run(np.array([33, 40, 80, 41], dtype=np.int32), BLOCK) == 2
    assert md.same_block_run(np.array([41], dtype=np.int32), BLOCK) == 1
    assert md.same_block_run(np.array([], dtype=np.int32), BLOCK) == 0
    for computed in ([0, 1], [41, 20], [63, 64], [7]):
        assert md.same_block_run(np.array(computed, dtype=np.int32), BLOCK) >= 1
    computed = np.array([33, 40, 63, 80], dtype=np.int32)
    run = md.same_block_run(computed, BLOCK)
    starts = (computed - md.row_lead(computed, BLOCK))[:run]
    assert len(set(starts.tolist())) == 1


def test_fill_page_table_width():
    # the step's token budget in blocks, rounded to 8 entries, capped at the read width
    assert md.fill_page_table_width(512, 32, 2048) == 16
    assert md.fill_page_table_width(100, 32, 2048) == 8
    assert md.fill_page_table_width(2048, 32, 64) == 64
    with pytest.raises(AssertionError, match="cannot cover"):
        md.fill_page_table_width(8192, 32, 64)


def test_host_builder_decode_and_chunk_rows():
    bs, width = 32, 8
    bt = (torch.arange(3 * width, dtype=torch.int32) + 1).reshape(3, width)
    # decode pass: 3 live rows + 1 padding row, one parked (0 scheduled)
    m = md.build_step_metadata_host(torch.tensor([40, 63, 7], dtype=torch.int32),
                                    torch.tensor([1, 1, 0], dtype=torch.int32), bt, bs, rows=4,
                                    tokens_per_row=1, fill_width=8)
    assert m.cache_position.tolist() == [40, 63, 6, -1]
    assert m.page_table[2].abs().sum() == 0 and m.page_table[3].abs().sum() == 0
    assert m.slot_mapping.tolist() == [int(bt[0, 1]) * bs + 8, int(bt[1, 1]) * bs + 31, -1, -1]
    assert m.chunk_start_idx is None
    # chunk pass: two rows continuing at 64 computed tokens, 64 new tokens each
    m = md.build_step_metadata_host(torch.tensor([64, 64], dtype=torch.int32),
                                    torch.tensor([64, 40], dtype=torch.int32), bt, bs, rows=2,
                                    tokens_per_row=64, fill_width=8)
    assert m.chunk_start_idx.tolist() == [64]
    assert m.fill_page_table[0].tolist() == torch.roll(bt[0], -2).tolist()
    assert m.slot_mapping.view(2, 64)[1, 40:].eq(-1).all()
    with pytest.raises(ValueError, match="share their chunk start"):
        md.build_step_metadata_host(torch.tensor([64, 32], dtype=torch.int32),
                                    torch.tensor([64, 64], dtype=torch.int32), bt, bs, 2, 64, 8)


def test_fill_page_table_and_slot_mapping_address_the_same_cells():
    """paged_fill_cache through the rolled fill_page_table writes exactly the cells the slot
    mapping names (the two addressings of the live path agree)."""
    g = torch.Generator().manual_seed(0)
    bs, nkv, hd, width, T = 32, 2, 64, 6, 64
    bt = (torch.randperm(2 * width, generator=g) + 1).reshape(2, width).int()
    computed = torch.tensor([64, 64], dtype=torch.int32)
    m = md.build_step_metadata_host(computed, torch.tensor([T, T], dtype=torch.int32), bt, bs, 2, T,
                                    fill_width=6)
    cache = torch.zeros(2 * width + 1, nkv, bs, hd, dtype=torch.bfloat16)
    fill = randn_bf16((2, T, nkv, hd), g)
    a = restate.paged_fill_cache(cache, fill.transpose(1, 2), m.fill_page_table)
    b = cache.clone()
    for i, s in enumerate(m.slot_mapping.tolist()):
        b[s // bs, :, s % bs] = fill.reshape(2 * T, nkv, hd)[i]
    assert torch.equal(a, b)
