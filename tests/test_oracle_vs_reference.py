"""The oracle restatement against the LIVE unmodified reference ops on fresh seeds, plus the
parametrisation of the reference's own CPU test (tests/torch/ops/test_chunked_sdpa_op_cpu.py)
re-run on both.  Needs the reference tree; skipped where it is not mounted (the golden vectors
carry the pin there)."""
import pytest
import torch

from oracle import reference_loader as ref
from oracle import restate
from oracle.inputs import config1, randn_bf16

pytestmark = pytest.mark.skipif(not ref.available(), reason="reference tree not mounted")


def _dense_offset_causal(q, k, v, start, scale):
    """Independent dense check in the style of the reference test: full K/V, explicit mask."""
    rep = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    T, S = q.shape[2], k.shape[2]
    mask = torch.arange(S)[None, :] <= (start + torch.arange(T))[:, None]
    w = (q @ k.transpose(-1, -2)) * scale
    w = w.masked_fill(~mask, float("-inf")).softmax(-1)
    return w @ v


@pytest.mark.parametrize("nq,nkv", [(4, 4), (8, 2), (32, 8)])
@pytest.mark.parametrize("start", [0, 64, 96])
def test_chunked_reference_parametrisation(nq, nkv, start):
    g = torch.Generator().manual_seed(nq + start)
    hd, bs, T, users = 64, 32, 64, 2
    nblk = (start + T) // bs
    nb = users * nblk + 1
    kc = torch.randn(nb, nkv, bs, hd, generator=g)
    vc = torch.randn(nb, nkv, bs, hd, generator=g)
    pt = (torch.randperm(nb - 1, generator=g)[: users * nblk] + 1).reshape(users, nblk).int()
    q = torch.randn(users, nq, T, hd, generator=g)
    scale = hd ** -0.5
    want = ref.ref_chunked_sdpa(q, kc, vc, pt, start, scale)
    got = restate.chunked_sdpa(q, kc, vc, pt, start, scale)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    # the independent dense form, as the reference test builds it
    for u in range(users):
        ku = kc[pt[u].long()].transpose(0, 1).reshape(1, nkv, nblk * bs, hd)
        vu = vc[pt[u].long()].transpose(0, 1).reshape(1, nkv, nblk * bs, hd)
        dense = _dense_offset_causal(q[u:u + 1], ku, vu, start, scale)
        assert torch.allclose(got[u:u + 1], dense, atol=1e-4, rtol=1e-4)


def test_one_token_remainder_chunk():
    g = torch.Generator().manual_seed(3)
    nq, nkv, hd, bs, start, T = 8, 2, 64, 32, 64, 1
    nblk = 3
    kc = torch.randn(nblk + 1, nkv, bs, hd, generator=g)
    vc = torch.randn(nblk + 1, nkv, bs, hd, generator=g)
    pt = torch.tensor([[1, 2, 3]], dtype=torch.int32)
    q = torch.randn(1, nq, T, hd, generator=g)
    want = ref.ref_chunked_sdpa(q, kc, vc, pt, start, hd ** -0.5)
    got = restate.chunked_sdpa(q, kc, vc, pt, start, hd ** -0.5)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)


def test_config1_decode_step_live():
    """benchmark config 1 through the live reference ops (GQA via the per-group loop) vs the oracle:
    cache writes bit-exact, attention equal in fp32 and in native bf16."""
    c = config1()
    users = c.users
    k = c.k.reshape(1, users, c.nkv, c.hd)
    v = c.v.reshape(1, users, c.nkv, c.hd)
    q = c.q.reshape(1, users, c.nq, c.hd)
    pos = c.cache_position
    rk = ref.ref_paged_update_cache(c.k_cache, k, pos, c.page_table)
    rv = ref.ref_paged_update_cache(c.v_cache, v, pos, c.page_table)
    ok = restate.paged_update_cache(c.k_cache, k, pos, c.page_table)
    ov = restate.paged_update_cache(c.v_cache, v, pos, c.page_table)
    assert torch.equal(rk, ok) and torch.equal(rv, ov)
    want = ref.ref_paged_decode(q.float(), rk.float(), rv.float(), c.page_table, pos, c.scale)
    got = restate.paged_sdpa_decode(q.float(), ok.float(), ov.float(), c.page_table, pos, c.scale)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
    mla = ref.ref_paged_decode_mla_branch(q.float(), rk.float(), rv.float(), c.page_table, pos,
                                          c.scale)
    assert torch.allclose(got, mla, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("T", [10, 20, 32, 50, 70])   # tests/torch/ops/test_custom_ops.py:171-203
def test_fill_cache_reference_lengths(T):
    g = torch.Generator().manual_seed(T)
    nb, nkv, bs, hd, users = 12, 8, 32, 128, 2
    cache = randn_bf16((nb, nkv, bs, hd), g)
    pt = torch.randperm(nb, generator=g)[: users * 3].reshape(users, 3).int()
    fill = randn_bf16((users, nkv, T, hd), g)
    want = ref.ref_paged_fill_cache(cache, fill, pt)
    got = restate.paged_fill_cache(cache, fill, pt)
    assert torch.equal(got, want)


def test_sdpa_gqa_12_4():                              # tests/torch/ops/test_custom_ops.py:52-95
    g = torch.Generator().manual_seed(8)
    q = torch.randn(1, 12, 64, 64, generator=g)
    k = torch.randn(1, 4, 64, 64, generator=g)
    v = torch.randn(1, 4, 64, 64, generator=g)
    want = ref.ref_sdpa(q, k, v, 0.125)
    got = restate.sdpa(q, k, v, True, 0.125)
    assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
