"""The decode split-count cost model (`b200attn_decode_auto_splits`, host code: no GPU needed)
against the sweep it was fitted to (tests/golden/decode_split_sweep.json: microseconds per
decode call on a B200 for 20 batch shapes at several split counts, written by
tests/golden/make_decode_split_sweep.py)."""
import json
import os

import pytest

from b200attn import _lib

SWEEP = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decode_split_sweep.json")


def _rows():
    with open(SWEEP) as f:
        return json.load(f)


def _regret(row, pick):
    times = {int(k): v for k, v in row["times"].items()}
    nearest = min(times, key=lambda s: (abs(s - pick), s))     # the sweep is a grid: nearest point
    return times[nearest] / min(times.values()) - 1.0


def test_model_stays_close_to_the_best_measured_split():
    L = _lib.lib()
    regrets = {}
    for row in _rows():
        pick = L.b200attn_decode_auto_splits(row["users"], row["nkv"], row["hd"], row["hint"])
        tiles = (row["hint"] + 63) // 64
        assert 1 <= pick <= min(tiles, 128), row["name"]
        regrets[row["name"]] = _regret(row, pick)
    worst = max(regrets, key=regrets.get)
    mean = sum(regrets.values()) / len(regrets)
    assert regrets[worst] <= 0.12, f"{worst}: {regrets[worst]:.3f} over the best measured split"
    assert mean <= 0.03, f"mean regret {mean:.4f}"


@pytest.mark.parametrize("users,nkv,hd,ctx,want", [
    (32, 8, 128, 32768, 3),      # config 4 on one GPU
    (32, 1, 128, 32768, 9),      # ... its per-rank shard on eight
    (64, 8, 128, 2048, 1),       # config 5 decode: plenty of CTAs already
    (8, 8, 64, 1024, 4),         # config 1: short contexts, few users
])
def test_picks_for_the_benchmark_shapes(users, nkv, hd, ctx, want):
    assert _lib.lib().b200attn_decode_auto_splits(users, nkv, hd, ctx) == want


def test_degenerate_arguments_give_one_split():
    L = _lib.lib()
    assert L.b200attn_decode_auto_splits(0, 8, 128, 1024) == 1
    assert L.b200attn_decode_auto_splits(8, 8, 128, 0) == 1
    assert L.b200attn_decode_auto_splits(8, 8, 128, 1) == 1
