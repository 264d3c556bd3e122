"""Sliding-window ring helpers (host mirror of vllm_tt/swa_cache_utils.py): fixed expectations
taken from the definitions, and a sweep against the live reference functions where the reference
tree is mounted."""
import numpy as np
import pytest

from b200attn import swa
from oracle import reference_loader as ref


def test_window_blocks_alignment_slack_and_cap():
    for window in (1, 31, 32, 33, 512, 1000, 1024, 4096):
        for bs in (16, 32, 64, 128):
            wb = swa.sliding_window_blocks(window, bs, 1 << 20)
            need = -(-window // bs) + 1
            assert wb % 8 == 0 and need <= wb < need + 8
    assert swa.sliding_window_blocks(1024, 32, 1_000_000) == 40    # 33 blocks -> next multiple of 8
    assert swa.sliding_window_blocks(1024, 32, 128) == 8           # cut to the model length
    assert swa.sliding_window_blocks(1024, 32, 1024) == swa.sliding_window_blocks(1024, 32, 10**6)


def test_profitability_is_ring_shorter_than_full_context():
    assert not swa.sliding_ring_is_profitable(1024, 32, 1024)
    assert not swa.sliding_ring_is_profitable(1024, 32, 40 * 32)
    assert swa.sliding_ring_is_profitable(1024, 32, 40 * 32 + 1)
    assert swa.sliding_ring_is_profitable(1024, 32, 131072)


def test_physical_blocks_bytes_and_width():
    assert swa.sliding_ring_phys_blocks(40, 32) == 1281
    assert swa.sliding_ring_reserve_bytes(40, 32, 65536) == 1281 * 65536
    assert swa.sliding_page_table_width(40, 4096) == 40
    assert swa.sliding_page_table_width(40, 8) == 8


def test_slots_are_stable_reclaimed_and_lowest_first():
    mapping, free = {}, list(range(4))
    assert swa.assign_ring_slots(["a", "b", "c"], ["a", "b", "c"], mapping, free).tolist() == [0, 1, 2]
    # rows reordered after "a" left: survivors keep their slots
    assert swa.assign_ring_slots(["c", "b"], ["c", "b"], mapping, free).tolist() == [2, 1]
    assert "a" not in mapping and sorted(free) == [0, 3]
    # newcomers take the lowest free slot
    assert swa.assign_ring_slots(["c", "b", "d"], ["c", "b", "d"], mapping, free).tolist() == [2, 1, 0]
    # a pass over part of the batch frees nothing that is still in the batch
    assert swa.assign_ring_slots(["d"], ["c", "b", "d"], mapping, free).tolist() == [0]
    assert mapping == {"c": 2, "b": 1, "d": 0} and free == [3]
    swa.assign_ring_slots(["e"], ["c", "b", "d", "e"], mapping, free)
    with pytest.raises(IndexError):
        swa.assign_ring_slots(["f"], ["c", "b", "d", "e", "f"], mapping, free)


def test_page_table_rotation():
    wb, width = 8, 8
    # below the window: identity inside the request's own sub-ring
    pt = swa.build_sliding_ring_page_table(np.array([0]), np.array([1]), wb, width)
    assert pt.tolist() == [[1 + wb + i for i in range(width)]]
    # start block 3: wraps once
    pt = swa.build_sliding_ring_page_table(np.array([3]), np.array([0]), wb, width)
    assert pt.tolist() == [[1 + (3 + i) % wb for i in range(width)]]
    # every row is a permutation of its own sub-ring and never names the null block
    pt = swa.build_sliding_ring_page_table(np.array([5, 77]), np.array([2, 0]), wb, width)
    for row, slot in zip(pt, (2, 0)):
        assert sorted(row.tolist()) == list(range(1 + slot * wb, 1 + (slot + 1) * wb))


def test_ring_window_view_and_prefill_guard():
    bs, wb = 32, 8
    start, pos = swa.ring_window_view(np.array([1, 256, 257, 1000]), bs, wb)
    assert start.tolist() == [0, 0, 1, 24]
    assert pos.tolist() == [0, 255, 224, 231]
    swa.check_sliding_prefill_supported(np.array([0, 3]), np.array([64, 1]), np.array([0, 99]))
    with pytest.raises(NotImplementedError, match="sliding-window prefill"):
        swa.check_sliding_prefill_supported(np.array([1]), np.array([64]), np.array([0]))
    with pytest.raises(NotImplementedError, match="sliding-window prefill"):
        swa.check_sliding_prefill_supported(np.array([0]), np.array([64]), np.array([32]))


@pytest.mark.skipif(not ref.available(), reason="reference tree not mounted")
def test_against_live_reference_helpers():
    r = ref.load_swa_utils()
    rng = np.random.default_rng(0)
    for _ in range(300):
        window = int(rng.integers(1, 5000))
        bs = int(rng.choice([16, 32, 64, 128]))
        mml = int(rng.integers(1, 200000))
        assert swa.sliding_window_blocks(window, bs, mml) == r.sliding_window_blocks(window, bs, mml)
        assert swa.sliding_ring_is_profitable(window, bs, mml) == \
            r.sliding_ring_is_profitable(window, bs, mml)
        wb = swa.sliding_window_blocks(window, bs, mml)
        n = int(rng.integers(1, 64))
        assert swa.sliding_ring_phys_blocks(wb, n) == r.sliding_ring_phys_blocks(wb, n)
        assert swa.sliding_ring_reserve_bytes(wb, n, 4096) == r.sliding_ring_reserve_bytes(wb, n, 4096)
        bw = int(rng.integers(1, 300))
        assert swa.sliding_page_table_width(wb, bw) == r.sliding_page_table_width(wb, bw)
        rows = int(rng.integers(1, 9))
        start = rng.integers(0, 500, rows)
        slots = rng.permutation(16)[:rows]
        width = swa.sliding_page_table_width(wb, bw)
        assert np.array_equal(swa.build_sliding_ring_page_table(start, slots, wb, width),
                              r.build_sliding_ring_page_table(start, slots, wb, width))
    # slot bookkeeping through a random arrival / departure sequence
    ours, theirs = ({}, list(range(6))), ({}, list(range(6)))
    live = []
    for step in range(200):
        if live and rng.random() < 0.4:
            live.pop(int(rng.integers(len(live))))
        while len(live) < 6 and rng.random() < 0.6:
            live.append(f"r{step}_{len(live)}")
        rows = [x for x in live if rng.random() < 0.7]
        a = swa.assign_ring_slots(rows, live, *ours)
        b = r.assign_ring_slots(rows, live, *theirs)
        assert a.tolist() == b.tolist() and ours[0] == theirs[0] and sorted(ours[1]) == sorted(theirs[1])
