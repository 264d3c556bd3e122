"""B200AttentionBackendImpl.forward against the reference backend's forward (golden vectors from
the unmodified TTAttentionBackendImpl on CPU) and against the oracle's restated forward:
cache contents bit-exact, outputs within the bf16 budget."""
import pytest
import torch

from oracle import restate
from oracle.inputs import config1, make_prefill_case
from tests.conftest import assert_attention_close
from tests.golden.golden_io import load_case

pytestmark = pytest.mark.gpu


def make_impl(nq, nkv, hd):
    from b200attn import B200AttentionBackendImpl

    return B200AttentionBackendImpl(nq, hd, hd ** -0.5, nkv, None, None, "auto")


def test_impl_decode_golden(clean_error_word):
    from b200attn import B200Metadata

    c = load_case("impl_decode_mha")
    nq, nkv, users = int(c["nq"]), int(c["nkv"]), 4
    impl = make_impl(nq, nkv, 64)
    kv = [c["k_cache"].cuda(), c["v_cache"].cuda()]
    ids = [t.data_ptr() for t in kv]
    md = B200Metadata(cache_position=c["cache_position"].cuda(), page_table=c["page_table"].cuda(),
                      batch_idx=torch.arange(users, dtype=torch.int32).cuda(), num_users=users)
    out = torch.empty(users, nq * 64, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, c["q"].cuda(), c["k"].cuda(), c["v"].cuda(), kv, md, output=out)
    assert [t.data_ptr() for t in kv] == ids, "cache tensors keep their identity"
    assert torch.equal(kv[0].cpu(), c["out_k"]) and torch.equal(kv[1].cpu(), c["out_v"])
    assert_attention_close(out, c["out_bf16"].float(), "impl decode golden")


def test_impl_prefill_golden(clean_error_word):
    from b200attn import B200Metadata

    c = load_case("impl_prefill_gqa")
    nq, nkv, nb, bs = int(c["nq"]), int(c["nkv"]), int(c["nb"]), int(c["bs"])
    T = c["q"].shape[0]
    impl = make_impl(nq, nkv, 64)
    kv = [torch.zeros(nb, nkv, bs, 64, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    md = B200Metadata(cache_position=torch.tensor([T - 1], dtype=torch.int32).cuda(),
                      page_table=c["page_table"].cuda(), fill_page_table=c["page_table"].cuda(),
                      batch_idx=torch.zeros(1, dtype=torch.int32).cuda(), num_users=1)
    out = torch.empty(T, nq * 64, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, c["q"].cuda(), c["k"].cuda(), c["v"].cuda(), kv, md, output=out)
    assert torch.equal(kv[0].cpu(), c["out_k"]) and torch.equal(kv[1].cpu(), c["out_v"])
    assert_attention_close(out, c["out_bf16"].float(), "impl prefill golden")


def test_impl_chunk_golden(clean_error_word):
    from b200attn import B200Metadata

    c = load_case("impl_chunk_gqa")
    nq, nkv = int(c["nq"]), int(c["nkv"])
    T, start = c["q"].shape[0], int(c["chunk_start"])
    impl = make_impl(nq, nkv, 64)
    kv = [c["k_cache"].cuda(), c["v_cache"].cuda()]
    md = B200Metadata(cache_position=torch.tensor([start + T - 1], dtype=torch.int32).cuda(),
                      page_table=c["page_table"].cuda(),
                      fill_page_table=c["fill_page_table"].cuda(),
                      chunk_start_idx=torch.tensor([start], dtype=torch.int32).cuda(),
                      batch_idx=torch.zeros(1, dtype=torch.int32).cuda(), num_users=1)
    out = torch.empty(T, nq * 64, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, c["q"].cuda(), c["k"].cuda(), c["v"].cuda(), kv, md, output=out)
    assert torch.equal(kv[0].cpu(), c["out_k"]) and torch.equal(kv[1].cpu(), c["out_v"])
    assert_attention_close(out, c["out_bf16"].float(), "impl chunk golden")


def test_impl_decode_config1(clean_error_word):
    """benchmark config 1 end to end through forward: scatter bit-exact, attention in budget."""
    from b200attn import B200Metadata

    case = config1()
    users = case.users
    impl = make_impl(case.nq, case.nkv, case.hd)
    want_out, want_k, want_v = restate.impl_forward(
        case.q, case.k, case.v, case.k_cache, case.v_cache, num_heads=case.nq,
        num_kv_heads=case.nkv, head_size=case.hd, scale=case.scale, num_users=users,
        cache_position=case.cache_position, page_table=case.page_table,
        compute_dtype=torch.float32,
    )
    kv = [case.k_cache.cuda(), case.v_cache.cuda()]
    md = B200Metadata(cache_position=case.cache_position.cuda(), page_table=case.page_table.cuda(),
                      batch_idx=torch.arange(users, dtype=torch.int32).cuda(), num_users=users)
    out = torch.empty(users, case.nq * case.hd, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, case.q.cuda(), case.k.cuda(), case.v.cuda(), kv, md, output=out)
    assert torch.equal(kv[0].cpu(), want_k) and torch.equal(kv[1].cpu(), want_v)
    assert_attention_close(out, want_out, "config 1 forward")


@pytest.mark.parametrize("start", [0, 128])
def test_impl_prefill_multi_user_gqa(start, clean_error_word):
    """Multi-user GQA prefill / continuation chunk (not pinned by any CPU-runnable reference
    test; the oracle loops the reference semantics per user)."""
    from b200attn import B200Metadata

    case = make_prefill_case(nq=32, nkv=8, hd=128, bs=64, users=3, T=256, chunk_start=start,
                             seed=21 + start)
    impl = make_impl(case.nq, case.nkv, case.hd)
    bidx = torch.arange(case.users, dtype=torch.int32)
    cs = torch.tensor([start], dtype=torch.int32) if start else None
    want_out, want_k, want_v = restate.impl_forward(
        case.q, case.k, case.v, case.k_cache, case.v_cache, num_heads=case.nq,
        num_kv_heads=case.nkv, head_size=case.hd, scale=case.scale, num_users=case.users,
        cache_position=torch.full((case.users,), start + case.T - 1, dtype=torch.int32),
        page_table=case.page_table, fill_page_table=case.fill_page_table, batch_idx=bidx,
        chunk_start_idx=cs, compute_dtype=torch.float32,
    )
    kv = [case.k_cache.cuda(), case.v_cache.cuda()]
    md = B200Metadata(
        cache_position=torch.full((case.users,), start + case.T - 1, dtype=torch.int32).cuda(),
        page_table=case.page_table.cuda(), fill_page_table=case.fill_page_table.cuda(),
        chunk_start_idx=cs.cuda() if cs is not None else None, batch_idx=bidx.cuda(),
        num_users=case.users)
    out = torch.empty(case.users * case.T, case.nq * case.hd, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, case.q.cuda(), case.k.cuda(), case.v.cuda(), kv, md, output=out)
    assert torch.equal(kv[0].cpu(), want_k) and torch.equal(kv[1].cpu(), want_v)
    assert_attention_close(out, want_out, "multi-user prefill")
