"""The oracle restatement against the golden vectors produced by the unmodified reference
(tests/golden/make_golden.py).  CPU only."""
import pytest
import torch

from oracle import restate
from tests.golden.golden_io import load_case


def test_update_cache_matches_reference():
    c = load_case("update_cache")
    out_k = restate.paged_update_cache(c["k_cache"], c["k"], c["update_indices"], c["page_table"])
    out_v = restate.paged_update_cache(c["v_cache"], c["v"], c["update_indices"], c["page_table"])
    assert torch.equal(out_k, c["out_k"]) and torch.equal(out_v, c["out_v"])
    # the padded row (-1) lands in the last page-table column at the last offset
    blk = int(c["page_table"][3, -1])
    assert torch.equal(c["out_k"][blk, :, -1, :], c["k"][0, 3])


@pytest.mark.parametrize("T", [10, 32, 50, 70])
def test_fill_cache_matches_reference(T):
    c = load_case(f"fill_cache_T{T}")
    out = restate.paged_fill_cache(
        c["cache"], c["fill"].transpose(1, 2), c["page_table"], c["batch_idx"]
    )
    assert torch.equal(out, c["out"])


@pytest.mark.parametrize("name", ["decode_mha", "decode_gqa4_hd64", "decode_gqa8_hd128"])
def test_decode_matches_reference(name):
    c = load_case(name)
    scale = float(c["scale"])
    o32 = restate.paged_sdpa_decode(
        c["q"].float(), c["k_cache"].float(), c["v_cache"].float(), c["page_table"],
        c["cur_pos"], scale,
    )
    assert torch.allclose(o32, c["out_fp32"], atol=1e-5, rtol=1e-5)
    o16 = restate.paged_sdpa_decode(
        c["q"], c["k_cache"], c["v_cache"], c["page_table"], c["cur_pos"], scale
    )
    # bf16 arithmetic: same operations, so agreement to bf16 rounding of the result
    assert (o16.float() - c["out_bf16"].float()).abs().max() <= 2e-2


def test_sdpa_matches_reference():
    c = load_case("sdpa_gqa")
    o32 = restate.sdpa(c["q"].float(), c["k"].float(), c["v"].float(), True, float(c["scale"]))
    assert torch.allclose(o32, c["out_fp32"], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("start", [0, 64, 96])
def test_chunked_matches_reference(start):
    c = load_case(f"chunked_start{start}")
    o32 = restate.chunked_sdpa(
        c["q"].float(), c["k_cache"].float(), c["v_cache"].float(), c["page_table"],
        int(c["chunk_start"]), float(c["scale"]),
    )
    assert torch.allclose(o32, c["out_fp32"], atol=1e-5, rtol=1e-5)


def _impl_args(c, users, **kw):
    nq, nkv = int(c["nq"]), int(c["nkv"])
    return dict(num_heads=nq, num_kv_heads=nkv, head_size=64, scale=64 ** -0.5, num_users=users,
                **kw)


def test_impl_decode_matches_reference_forward():
    c = load_case("impl_decode_mha")
    out, k2, v2 = restate.impl_forward(
        c["q"], c["k"], c["v"], c["k_cache"], c["v_cache"],
        **_impl_args(c, 4, cache_position=c["cache_position"], page_table=c["page_table"]),
    )
    assert torch.equal(k2, c["out_k"]) and torch.equal(v2, c["out_v"])
    assert (out.float() - c["out_bf16"].float()).abs().max() <= 2e-2


def test_impl_prefill_matches_reference_forward():
    c = load_case("impl_prefill_gqa")
    nb, bs = int(c["nb"]), int(c["bs"])
    zeros = torch.zeros((nb, int(c["nkv"]), bs, 64), dtype=torch.bfloat16)
    T = c["q"].shape[0]
    out, k2, v2 = restate.impl_forward(
        c["q"], c["k"], c["v"], zeros, zeros.clone(),
        **_impl_args(c, 1, cache_position=torch.tensor([T - 1], dtype=torch.int32),
                     page_table=c["page_table"], batch_idx=torch.zeros(1, dtype=torch.int32),
                     compute_dtype=torch.float32),
    )
    assert torch.equal(k2, c["out_k"]) and torch.equal(v2, c["out_v"])
    assert (out - c["out_bf16"].float()).abs().max() <= 2e-2


def test_impl_chunk_matches_reference_forward():
    c = load_case("impl_chunk_gqa")
    T = c["q"].shape[0]
    start = int(c["chunk_start"])
    out, k2, v2 = restate.impl_forward(
        c["q"], c["k"], c["v"], c["k_cache"], c["v_cache"],
        **_impl_args(c, 1, cache_position=torch.tensor([start + T - 1], dtype=torch.int32),
                     page_table=c["page_table"], fill_page_table=c["fill_page_table"],
                     batch_idx=torch.zeros(1, dtype=torch.int32),
                     chunk_start_idx=torch.tensor([start], dtype=torch.int32),
                     compute_dtype=torch.float32),
    )
    assert torch.equal(k2, c["out_k"]) and torch.equal(v2, c["out_v"])
    assert (out - c["out_bf16"].float()).abs().max() <= 2e-2


@pytest.mark.parametrize("name", ["rotary_hd64", "rotary_hd128", "rotary_hd64_partial32"])
def test_rotary_matches_reference(name):
    c = load_case(name)
    q, k = restate.rotary_embedding(c["positions"], c["q"], c["k"], c["inv_freq"],
                                    int(c["head_size"]), int(c["rotary_dim"]))
    assert torch.equal(q, c["out_q"]) and torch.equal(k, c["out_k"])
