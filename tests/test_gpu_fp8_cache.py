"""fp8 (e4m3) KV cache: the plugin's kv_cache_dtype "fp8" / "fp8_e4m3" (attention.py:42-51).
Cache writes are checked bit for bit against the reference's write arithmetic (clamp to the finite
range, cast: attention.py:692-700, restated in oracle.restate.quantize_kv_fp8); decode attention
over the fp8 cache against the oracle run on the same fp8 tensors in fp32 arithmetic, bf16
tolerance (max abs <= 2e-2, mean abs <= 2e-3).  The reference's live CPU cache ops cannot take an
fp8 cache (index_put needs matching dtypes), so parity here rests on that published arithmetic."""
import pytest
import torch

from oracle import restate
from oracle.inputs import make_decode_case, randn_bf16
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _bits(t):
    """Byte image with the two NaN encodings of e4m3 (0x7f, 0xff) folded together: which one a
    conversion produces for a NaN input carries no information."""
    b = t.view(torch.uint8).clone()
    b[b == 0xFF] = 0x7F
    return b


def _special_rows(shape, g):
    """N(0,1) rows with the awkward values mixed in: saturating, subnormal, tiny, signed zero, NaN."""
    x = torch.randn(shape, generator=g) * 3
    flat = x.view(-1)
    specials = torch.tensor([1000.0, -1000.0, 448.0, 449.0, 464.0, -480.0, 2 ** -6, 2 ** -7, 2 ** -9,
                             2 ** -10, 3 * 2 ** -10, 1e-9, -0.0, 0.0, float("nan"), 0.0703125,
                             0.0664, 17.0, 18.0, 19.0, 240.0, 250.0, float("inf"), -float("inf")])
    idx = torch.randperm(flat.numel(), generator=g)[: specials.numel() * 4]
    flat[idx] = specials.repeat(4)
    return x.to(torch.bfloat16)


def test_update_cache_fp8_bit_exact(clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(1)
    nb, nkv, bs, hd, users = 24, 4, 32, 128, 9
    kc = (torch.randn(nb, nkv, bs, hd, generator=g)).to(FP8)
    vc = (torch.randn(nb, nkv, bs, hd, generator=g)).to(FP8)
    pt = torch.randperm(nb, generator=g)[: users * 2].reshape(users, 2).to(torch.int32)
    pos = torch.randint(0, 2 * bs, (users,), generator=g).to(torch.int32)
    k = _special_rows((1, users, nkv, hd), g)
    v = _special_rows((1, users, nkv, hd), g)
    want_k = restate.paged_update_cache(kc, k, pos, pt)
    want_v = restate.paged_update_cache(vc, v, pos, pt)
    kd, vd = kc.cuda(), vc.cuda()
    ops.paged_update_cache(kd, vd, k[0].cuda(), v[0].cuda(), pos.cuda(), pt.cuda())
    assert torch.equal(_bits(kd.cpu()), _bits(want_k)) and torch.equal(_bits(vd.cpu()), _bits(want_v))


@pytest.mark.parametrize("T", [10, 32, 70])
def test_fill_cache_fp8_bit_exact(T, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(T)
    nb, nkv, bs, hd, users = 16, 2, 32, 128, 3
    kc = torch.zeros(nb, nkv, bs, hd).to(FP8)
    vc = torch.zeros(nb, nkv, bs, hd).to(FP8)
    pt = (torch.randperm(nb - 1, generator=g)[: users * 3] + 1).reshape(users, 3).to(torch.int32)
    k = _special_rows((users, T, nkv, hd), g)
    v = _special_rows((users, T, nkv, hd), g)
    want_k = restate.paged_fill_cache(kc, k.transpose(1, 2), pt)
    want_v = restate.paged_fill_cache(vc, v.transpose(1, 2), pt)
    kd, vd = kc.cuda(), vc.cuda()
    ops.paged_fill_cache(kd, vd, k.cuda(), v.cuda(), pt.cuda(),
                         torch.arange(users, dtype=torch.int32).cuda())
    assert torch.equal(_bits(kd.cpu()), _bits(want_k)) and torch.equal(_bits(vd.cpu()), _bits(want_v))


def test_slot_scatter_fp8_bit_exact(clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(5)
    nb, nkv, bs, hd, n = 10, 8, 64, 128, 50
    kc = torch.zeros(nb, nkv, bs, hd).to(FP8)
    vc = torch.zeros(nb, nkv, bs, hd).to(FP8)
    slots = torch.randperm(nb * bs, generator=g)[:n].to(torch.int64)
    slots[7] = -1
    k = _special_rows((n, nkv, hd), g)
    v = _special_rows((n, nkv, hd), g)
    want_k, want_v = kc.clone(), vc.clone()
    for i, s in enumerate(slots.tolist()):
        if s >= 0:
            want_k[s // bs, :, s % bs] = restate.quantize_kv_fp8(k[i])
            want_v[s // bs, :, s % bs] = restate.quantize_kv_fp8(v[i])
    kd, vd = kc.cuda(), vc.cuda()
    ops.kv_scatter_slots(kd, vd, k.cuda(), v.cuda(), slots.cuda())
    assert torch.equal(_bits(kd.cpu()), _bits(want_k)) and torch.equal(_bits(vd.cpu()), _bits(want_v))


def _fp8_case(**kw):
    case = make_decode_case(**kw)
    case.k_cache = restate.quantize_kv_fp8(case.k_cache)
    case.v_cache = restate.quantize_kv_fp8(case.v_cache)
    return case


def _decode(case, splits=0, window=0, sinks=None):
    from b200attn import ops

    u = case.users
    return ops.paged_decode(
        case.q.reshape(u, case.nq, case.hd).cuda(), case.k_cache.cuda(), case.v_cache.cuda(),
        case.page_table.cuda(), case.cache_position.cuda(), scale=case.scale, num_splits=splits,
        sliding_window=window, sinks=None if sinks is None else sinks.cuda()).cpu()


def _oracle(case, window=None, sinks=None):
    u = case.users
    return restate.paged_sdpa_decode(
        case.q.reshape(1, u, case.nq, case.hd).float(), case.k_cache, case.v_cache, case.page_table,
        case.cache_position, case.scale, window, sinks)[0]


@pytest.mark.parametrize("nq,nkv", [(8, 2), (32, 8), (64, 8), (16, 1), (4, 4)])
@pytest.mark.parametrize("bs", [32, 64])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_decode_over_fp8_cache(nq, nkv, bs, splits, clean_error_word):
    case = _fp8_case(nq=nq, nkv=nkv, hd=128, bs=bs, users=5, ctx_lo=1, ctx_hi=700, seed=nq + bs)
    assert_attention_close(_decode(case, splits), _oracle(case), f"{nq}/{nkv}/{bs} splits={splits}")


@pytest.mark.parametrize("bs", [32, 64])
def test_fp8_every_context_length_in_three_tiles(bs, clean_error_word):
    users = 192
    case = _fp8_case(nq=8, nkv=2, hd=128, bs=bs, users=users, ctx_lo=192, ctx_hi=192, seed=3)
    case.ctx_lens = torch.arange(1, users + 1)
    for splits in (1, 2):
        assert_attention_close(_decode(case, splits), _oracle(case), f"splits={splits}")


def test_fp8_decode_with_window_and_sinks(clean_error_word):
    case = _fp8_case(nq=16, nkv=2, hd=128, bs=64, users=6, ctx_lo=1, ctx_hi=900, seed=21)
    g = torch.Generator().manual_seed(5)
    sinks = torch.randn(16, generator=g) * 2.0
    for splits in (0, 1, 4):
        assert_attention_close(_decode(case, splits, 100, sinks), _oracle(case, 100, sinks),
                               f"window+sinks splits={splits}")


def test_fp8_decode_of_values_beyond_f16_range_of_products(clean_error_word):
    """Largest representable cache values (+-448) with large queries: the MMAs take f16 operands,
    so this checks that nothing overflows on the way (accumulation is fp32)."""
    case = _fp8_case(nq=8, nkv=2, hd=128, bs=64, users=3, ctx_lo=100, ctx_hi=300, seed=2)
    case.k_cache = (case.k_cache.float() * 200).clamp(-448, 448).to(FP8)
    case.v_cache = (case.v_cache.float() * 200).clamp(-448, 448).to(FP8)
    case.q = (case.q.float() * 30).to(torch.bfloat16)
    out, ref = _decode(case, 2), _oracle(case)
    assert torch.isfinite(out.float()).all()
    # outputs are O(100): compare relatively (one bf16 ulp of the magnitude)
    assert ((out.float() - ref).abs() <= ref.abs() * 2 ** -6 + 1.0).all()


def test_fp8_needs_head_size_128_and_matching_caches():
    from b200attn import ops

    kc = torch.zeros(4, 2, 32, 64, device="cuda").to(FP8)
    q = torch.zeros(1, 8, 64, dtype=torch.bfloat16, device="cuda")
    pt = torch.zeros(1, 4, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="unsupported"):
        ops.paged_decode(q, kc, kc, pt, torch.zeros(1, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError, match="both"):
        ops.paged_decode(q, kc, kc.to(torch.bfloat16), pt,
                         torch.zeros(1, dtype=torch.int32, device="cuda"))


def test_impl_forward_fp8_cache(clean_error_word):
    """Through the Impl with kv_cache_dtype="fp8": fresh-K/V prefill writes the quantised cache and
    attends the bf16 K/V (as the reference does, attention.py:575-598), then a decode step reads
    the fp8 cache."""
    from b200attn import B200AttentionBackendImpl, B200Metadata

    nq, nkv, hd, bs, users, T = 8, 2, 128, 64, 2, 128
    g = torch.Generator().manual_seed(4)
    nb = 8
    kc = torch.zeros(nb, nkv, bs, hd).to(FP8)
    vc = torch.zeros(nb, nkv, bs, hd).to(FP8)
    pt = torch.tensor([[1, 2, 3], [4, 5, 6]], dtype=torch.int32)
    q = randn_bf16((users * T, nq * hd), g)
    k = randn_bf16((users * T, nkv * hd), g)
    v = randn_bf16((users * T, nkv * hd), g)
    impl = B200AttentionBackendImpl(nq, hd, hd ** -0.5, nkv, None, None, "fp8")
    kd, vd = kc.cuda(), vc.cuda()
    md = B200Metadata(cache_position=torch.zeros(users, dtype=torch.int32, device="cuda"),
                      page_table=pt.cuda(), num_users=users,
                      batch_idx=torch.arange(users, dtype=torch.int32, device="cuda"))
    out = torch.empty(users * T, nq * hd, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, q.cuda(), k.cuda(), v.cuda(), [kd, vd], md, output=out)
    want, kc_o, vc_o = restate.impl_forward(
        q, k, v, kc, vc, num_heads=nq, num_kv_heads=nkv, head_size=hd, scale=hd ** -0.5,
        num_users=users, cache_position=torch.zeros(users, dtype=torch.int32), page_table=pt,
        batch_idx=torch.arange(users), compute_dtype=torch.float32)
    assert torch.equal(_bits(kd.cpu()), _bits(kc_o)) and torch.equal(_bits(vd.cpu()), _bits(vc_o))
    assert_attention_close(out.cpu(), want, "fp8 impl prefill")
    q1 = randn_bf16((users, nq * hd), g)
    k1 = randn_bf16((users, nkv * hd), g)
    v1 = randn_bf16((users, nkv * hd), g)
    pos = torch.tensor([T, 70], dtype=torch.int32)
    md1 = B200Metadata(cache_position=pos.cuda(), page_table=pt.cuda(), num_users=users)
    out1 = torch.empty(users, nq * hd, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, q1.cuda(), k1.cuda(), v1.cuda(), [kd, vd], md1, output=out1)
    want1, kc_1, vc_1 = restate.impl_forward(
        q1, k1, v1, kc_o, vc_o, num_heads=nq, num_kv_heads=nkv, head_size=hd, scale=hd ** -0.5,
        num_users=users, cache_position=pos, page_table=pt, compute_dtype=torch.float32)
    assert torch.equal(_bits(kd.cpu()), _bits(kc_1)) and torch.equal(_bits(vd.cpu()), _bits(vc_1))
    assert_attention_close(out1.cpu(), want1, "fp8 impl decode")
    # a chunk of 64 tokens on top of the T-token prefix, attended over the fp8 pages
    # (chunked prefill: attention.py:545-560)
    n = users * 64
    md2 = B200Metadata(cache_position=torch.tensor([T + 63, T + 63], dtype=torch.int32).cuda(),
                       page_table=pt.cuda(), num_users=users,
                       chunk_start_idx=torch.tensor([T], dtype=torch.int32).cuda(),
                       batch_idx=torch.arange(users, dtype=torch.int32, device="cuda"),
                       fill_page_table=torch.roll(pt, -2, dims=1).contiguous().cuda())
    # decode step above wrote position T of user 0 and 70 of user 1; start from the prefill state
    kd, vd = kc_o.cuda(), vc_o.cuda()
    impl.forward(None, q[:n].cuda(), k[:n].cuda(), v[:n].cuda(), [kd, vd], md2, output=out[:n])
    want2, kc_2, vc_2 = restate.impl_forward(
        q[:n], k[:n], v[:n], kc_o, vc_o, num_heads=nq, num_kv_heads=nkv, head_size=hd,
        scale=hd ** -0.5, num_users=users,
        cache_position=torch.tensor([T + 63, T + 63], dtype=torch.int32), page_table=pt,
        fill_page_table=torch.roll(pt, -2, dims=1).contiguous(), batch_idx=torch.arange(users),
        chunk_start_idx=torch.tensor([T], dtype=torch.int32), compute_dtype=torch.float32)
    assert torch.equal(_bits(kd.cpu()), _bits(kc_2)) and torch.equal(_bits(vd.cpu()), _bits(vc_2))
    assert_attention_close(out[:n].cpu(), want2, "fp8 impl chunked prefill")


@pytest.mark.parametrize("bs", [32, 64])
def test_chunked_prefill_over_fp8_pages(bs, clean_error_word):
    """Ragged sequences with different prefixes over an e4m3 cache: the pages each sequence reads
    are widened (exactly) into a bf16 pool and attended there; expected = the oracle's chunked op
    on the same e4m3 values in fp32.  Unwidened slots of the pool hold NaN to show they are never
    read into a result."""
    from b200attn import ops

    g = torch.Generator().manual_seed(70 + bs)
    nq, nkv, hd = 8, 2, 128
    q_lens = [1, 37, 128, 200]
    starts = [300, 64, 0, 128]
    nblks = [(s + t + bs - 1) // bs for s, t in zip(starts, q_lens)]
    width = max(nblks) + 2
    nb = sum(nblks) + 1
    perm = torch.randperm(nb - 1, generator=g) + 1
    pt = torch.zeros(len(q_lens), width, dtype=torch.int32)
    o = 0
    for i, n_ in enumerate(nblks):
        pt[i, :n_] = perm[o:o + n_].int()
        o += n_
    kc = restate.quantize_kv_fp8(randn_bf16((nb, nkv, bs, hd), g))
    vc = restate.quantize_kv_fp8(randn_bf16((nb, nkv, bs, hd), g))
    total = sum(q_lens)
    q = randn_bf16((total, nq, hd), g)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    # poison a scratch pool of the size the op will ask for, so stale contents would show
    ops._fp8_scratch.clear()
    out = ops.prefill(q.cuda(), kc.cuda(), vc.cuda(), cu_q, scale=hd ** -0.5, page_table=pt.cuda(),
                      q_start=torch.tensor(starts, dtype=torch.int32).cuda())
    for pool in list(ops._fp8_scratch.values())[0][:2]:
        pool.fill_(float("nan"))
    out = ops.prefill(q.cuda(), kc.cuda(), vc.cuda(), cu_q, scale=hd ** -0.5, page_table=pt.cuda(),
                      q_start=torch.tensor(starts, dtype=torch.int32).cuda()).cpu()
    for i, (t, s_) in enumerate(zip(q_lens, starts)):
        qi = q[cu_q[i]:cu_q[i + 1]].transpose(0, 1)[None].float()
        want = restate.chunked_sdpa(qi, kc.float(), vc.float(), pt[i:i + 1, :nblks[i]], s_,
                                    hd ** -0.5)[0].transpose(0, 1)
        assert_attention_close(out[cu_q[i]:cu_q[i + 1]], want, f"seq {i}")
