"""Sliding-window attention and attention sinks (the ops' `sliding_window_size` /
`attention_sink` arguments, custom_ops.py:635-646, 1198-1208) against the oracle's restatement of
their published definitions.  The reference's CPU branches ignore both arguments, so these cases
have no reference output behind them; window 0 / no sinks must reproduce the plain kernels
bit for bit.  Tolerance: max abs <= 2e-2, mean abs <= 2e-3 against fp32 arithmetic."""
import pytest
import torch

from oracle import restate
from oracle.inputs import make_decode_case, make_prefill_case, randn_bf16
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def _decode(case, window=0, sinks=None, splits=0):
    from b200attn import ops

    u = case.users
    return ops.paged_decode(
        case.q.reshape(u, case.nq, case.hd).cuda(), case.k_cache.cuda(), case.v_cache.cuda(),
        case.page_table.cuda(), case.cache_position.cuda(), scale=case.scale, num_splits=splits,
        sliding_window=window, sinks=None if sinks is None else sinks.cuda(),
    ).cpu()


def _decode_oracle(case, window=None, sinks=None):
    u = case.users
    return restate.paged_sdpa_decode(
        case.q.reshape(1, u, case.nq, case.hd).float(), case.k_cache.float(),
        case.v_cache.float(), case.page_table, case.cache_position, case.scale, window, sinks,
    )[0]


@pytest.mark.parametrize("window", [1, 17, 64, 100, 128, 1000])
@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("hd,bs", [(64, 32), (128, 64)])
def test_decode_sliding_window(window, splits, hd, bs, clean_error_word):
    case = make_decode_case(nq=8, nkv=2, hd=hd, bs=bs, users=7, ctx_lo=1, ctx_hi=600,
                            seed=window + hd)
    assert_attention_close(_decode(case, window, None, splits), _decode_oracle(case, window),
                           f"window={window} splits={splits}")


@pytest.mark.parametrize("splits", [0, 1, 4])
@pytest.mark.parametrize("window", [0, 128])
def test_decode_sinks(window, splits, clean_error_word):
    case = make_decode_case(nq=16, nkv=2, hd=64, bs=32, users=6, ctx_lo=1, ctx_hi=900, seed=21)
    g = torch.Generator().manual_seed(5)
    sinks = torch.randn(16, generator=g) * 2.0
    assert_attention_close(_decode(case, window, sinks, splits),
                           _decode_oracle(case, window or None, sinks),
                           f"sinks window={window} splits={splits}")


def test_decode_window_every_context_length(clean_error_word):
    """Every context length 1..256 with a 70-key window: the window edge crosses tile and page
    boundaries at every offset."""
    users = 256
    case = make_decode_case(nq=4, nkv=1, hd=128, bs=64, users=users, ctx_lo=256, ctx_hi=256, seed=4)
    case.ctx_lens = torch.arange(1, users + 1)
    for splits in (1, 2):
        assert_attention_close(_decode(case, 70, None, splits), _decode_oracle(case, 70),
                               f"splits={splits}")


def test_decode_defaults_are_bit_identical(clean_error_word):
    """window 0 / no sinks through the extended entry point equals the plain entry point; a
    window at least as long as every context changes nothing either."""
    from b200attn import _lib, ops

    case = make_decode_case(nq=8, nkv=2, hd=128, bs=64, users=5, ctx_lo=1, ctx_hi=500, seed=8)
    base = _decode(case, splits=2)
    assert torch.equal(base, _decode(case, window=4096, splits=2))
    u = case.users
    q = case.q.reshape(u, case.nq, case.hd).cuda()
    kc, vc = case.k_cache.cuda(), case.v_cache.cuda()
    pt, pos = case.page_table.cuda(), case.cache_position.cuda()
    out = torch.empty_like(q)
    ws = torch.zeros(ops.decode_workspace_bytes(u, case.nq, case.hd, 2), dtype=torch.uint8,
                     device="cuda")
    L = _lib.lib()
    rc = L.b200attn_paged_decode(
        out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
        pt.data_ptr(), pt.stride(0), pt.shape[1], pos.data_ptr(), u, case.nq, case.nkv, case.hd,
        case.bs, kc.shape[0], case.scale, 0, 2, ws.data_ptr(), ws.numel(),
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), base)


def test_decode_bad_window_and_sinks_are_refused():
    from b200attn import ops

    case = make_decode_case(nq=8, nkv=2, hd=64, bs=32, users=2, ctx_lo=5, ctx_hi=50, seed=1)
    with pytest.raises(RuntimeError, match="BAD_ARGUMENT|bad argument"):
        _decode(case, window=-3)
    with pytest.raises(ValueError, match="sinks"):
        _decode(case, sinks=torch.zeros(4))
    with pytest.raises(ValueError, match="sinks"):
        ops.paged_decode(
            case.q.reshape(2, 8, 64).cuda(), case.k_cache.cuda(), case.v_cache.cuda(),
            case.page_table.cuda(), case.cache_position.cuda(), scale=case.scale,
            sinks=torch.zeros(8, dtype=torch.bfloat16, device="cuda"))


# ---------------------------------------------------------------------------------- prefill
def _cu(users, T):
    return torch.arange(users + 1, dtype=torch.int32) * T


@pytest.mark.parametrize("window", [1, 50, 128, 129, 300, 1024])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("T", [96, 512, 700])
def test_prefill_fresh_sliding_window(window, hd, T, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(T + hd + window)
    B, nq, nkv = 2, 4, 2
    q = randn_bf16((B, T, nq, hd), g)
    k = randn_bf16((B, T, nkv, hd), g)
    v = randn_bf16((B, T, nkv, hd), g)
    want = restate.sdpa(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                        v.transpose(1, 2).float(), True, hd ** -0.5, window).transpose(1, 2)
    out = ops.prefill(q.reshape(B * T, nq, hd).cuda(), k.reshape(B * T, nkv, hd).cuda(),
                      v.reshape(B * T, nkv, hd).cuda(), _cu(B, T), scale=hd ** -0.5,
                      sliding_window=window)
    assert_attention_close(out.reshape(B, T, nq, hd), want, f"fresh window={window}")


@pytest.mark.parametrize("window", [33, 128, 256, 500])
@pytest.mark.parametrize("hd,bs", [(64, 32), (128, 64)])
@pytest.mark.parametrize("T,start", [(64, 448), (320, 640), (200, 0)])
def test_prefill_chunked_sliding_window(window, hd, bs, T, start, clean_error_word):
    from b200attn import ops

    nq, nkv = 8, 2
    case = make_prefill_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=2, T=T, chunk_start=start,
                             seed=window + T)
    k = case.k.reshape(2, T, nkv, hd)
    v = case.v.reshape(2, T, nkv, hd)
    kc = restate.paged_fill_cache(case.k_cache, k.transpose(1, 2), case.fill_page_table)
    vc = restate.paged_fill_cache(case.v_cache, v.transpose(1, 2), case.fill_page_table)
    q4 = case.q.reshape(2, T, nq, hd)
    want = restate.chunked_sdpa(q4.transpose(1, 2).float(), kc.float(), vc.float(),
                                case.page_table, start, case.scale, window).transpose(1, 2)
    out = ops.prefill(
        case.q.reshape(2 * T, nq, hd).cuda(), kc.cuda(), vc.cuda(), _cu(2, T), scale=case.scale,
        page_table=case.page_table.cuda(),
        q_start=torch.full((2,), start, dtype=torch.int32, device="cuda"),
        sliding_window=window,
    )
    assert_attention_close(out.reshape(2, T, nq, hd), want, f"chunked window={window}")


def test_prefill_window_ragged_batch(clean_error_word):
    """Ragged query lengths and prefix lengths under one window: per sequence equal to its own
    oracle call."""
    from b200attn import ops

    g = torch.Generator().manual_seed(31)
    nq, nkv, hd, bs, window = 8, 2, 128, 64, 150
    q_lens = [1, 37, 300, 129]
    starts = [500, 64, 0, 384]
    nblks = [(s + t + bs - 1) // bs for s, t in zip(starts, q_lens)]
    nb = sum(nblks) + 1
    perm = torch.randperm(nb - 1, generator=g) + 1
    pt = torch.zeros(len(q_lens), max(nblks), dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblks):
        pt[i, :n] = perm[o:o + n].int()
        o += n
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    q = randn_bf16((sum(q_lens), nq, hd), g)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    out = ops.prefill(q.cuda(), kc.cuda(), vc.cuda(), cu_q, scale=hd ** -0.5,
                      page_table=pt.cuda(), q_start=torch.tensor(starts, dtype=torch.int32).cuda(),
                      sliding_window=window).cpu()
    for i, (t, s) in enumerate(zip(q_lens, starts)):
        qi = q[cu_q[i]:cu_q[i + 1]].transpose(0, 1)[None].float()
        want = restate.chunked_sdpa(qi, kc.float(), vc.float(), pt[i:i + 1, :nblks[i]], s,
                                    hd ** -0.5, window)[0].transpose(0, 1)
        assert_attention_close(out[cu_q[i]:cu_q[i + 1]], want, f"seq {i}")


def test_prefill_wide_window_is_bit_identical(clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(12)
    T, nq, nkv, hd = 640, 8, 2, 128
    q = randn_bf16((T, nq, hd), g).cuda()
    k = randn_bf16((T, nkv, hd), g).cuda()
    v = randn_bf16((T, nkv, hd), g).cuda()
    base = ops.prefill(q, k, v, _cu(1, T), scale=hd ** -0.5)
    wide = ops.prefill(q, k, v, _cu(1, T), scale=hd ** -0.5, sliding_window=T)
    assert torch.equal(base, wide)


def test_impl_forward_window_and_sinks(clean_error_word):
    """Through the plugin-facing Impl: windowed prefill then windowed decode with sinks; prefill
    with sinks is refused as in the reference (attention.py:321)."""
    from b200attn import B200AttentionBackendImpl, B200Metadata

    nq, nkv, hd, bs, users, T, window = 8, 2, 64, 32, 2, 96, 40
    case = make_prefill_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=users, T=T, seed=3)
    g = torch.Generator().manual_seed(2)
    sinks = torch.randn(nq, generator=g)
    kc, vc = case.k_cache.cuda(), case.v_cache.cuda()
    pt = case.page_table.cuda()
    # ---- prefill (no sinks)
    impl = B200AttentionBackendImpl(nq, hd, case.scale, nkv, None, window, "auto")
    md = B200Metadata(cache_position=torch.zeros(users, dtype=torch.int32, device="cuda"),
                      attn_mask=None, page_table=pt, is_causal=True, num_users=users,
                      batch_idx=torch.arange(users, dtype=torch.int32, device="cuda"))
    out = torch.empty(users * T, nq * hd, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, case.q.cuda(), case.k.cuda(), case.v.cuda(), [kc, vc], md, output=out)
    want, kc_o, vc_o = restate.impl_forward(
        case.q, case.k, case.v, case.k_cache, case.v_cache, num_heads=nq, num_kv_heads=nkv,
        head_size=hd, scale=case.scale, num_users=users,
        cache_position=torch.zeros(users, dtype=torch.int32), page_table=case.page_table,
        batch_idx=torch.arange(users), compute_dtype=torch.float32, sliding_window=window)
    assert_attention_close(out.cpu(), want, "impl prefill window")
    assert torch.equal(kc.cpu(), kc_o) and torch.equal(vc.cpu(), vc_o)
    # ---- decode with sinks
    impl_s = B200AttentionBackendImpl(nq, hd, case.scale, nkv, None, window, "auto",
                                      sinks=sinks.to(torch.bfloat16).cuda())
    q1 = randn_bf16((users, nq * hd), g)
    k1 = randn_bf16((users, nkv * hd), g)
    v1 = randn_bf16((users, nkv * hd), g)
    pos = torch.tensor([T - 1, 17], dtype=torch.int32)
    md1 = B200Metadata(cache_position=pos.cuda(), attn_mask=None, page_table=pt, is_causal=True,
                       num_users=users)
    out1 = torch.empty(users, nq * hd, dtype=torch.bfloat16, device="cuda")
    impl_s.forward(None, q1.cuda(), k1.cuda(), v1.cuda(), [kc, vc], md1, output=out1)
    want1, _, _ = restate.impl_forward(
        q1, k1, v1, kc_o, vc_o, num_heads=nq, num_kv_heads=nkv, head_size=hd, scale=case.scale,
        num_users=users, cache_position=pos, page_table=case.page_table,
        compute_dtype=torch.float32, sliding_window=window,
        sinks=sinks.to(torch.bfloat16).float())
    assert_attention_close(out1.cpu(), want1, "impl decode window+sinks")
    with pytest.raises(AssertionError, match="unsupported in SDPA prefill"):
        impl_s.forward(None, case.q.cuda(), case.k.cuda(), case.v.cuda(), [kc, vc], md,
                       output=out)


@pytest.mark.parametrize("hd,bs", [(64, 32), (128, 64)])
def test_decode_on_ring_cache_equals_windowed_decode_on_full_cache(hd, bs, clean_error_word):
    """The reference's sliding-window ring (swa_cache_utils.py, model_runner.py:1753-1815): each
    request keeps only `window_blocks` physical blocks, the page table lists them rotated into
    logical order and the position is counted from the first listed block.  Decoding on that
    ring must give what windowed decode over the whole context gives."""
    import numpy as np

    from b200attn import ops, swa

    window, users = 100, 6
    case = make_decode_case(nq=8, nkv=2, hd=hd, bs=bs, users=users, ctx_lo=1, ctx_hi=900, seed=13)
    want = _decode_oracle(case, window)
    wb = swa.sliding_window_blocks(window, bs, 1 << 20)
    slots = np.array([3, 0, 5, 1, 4, 2])
    start, pos_rel = swa.ring_window_view(case.ctx_lens.numpy(), bs, wb)
    ring_pt = swa.build_sliding_ring_page_table(start, slots, wb, wb)
    g = torch.Generator().manual_seed(99)
    nb_ring = swa.sliding_ring_phys_blocks(wb, users)
    ring_k = randn_bf16((nb_ring, 2, bs, hd), g)      # stale contents everywhere else
    ring_v = randn_bf16((nb_ring, 2, bs, hd), g)
    for u in range(users):
        cur_block = (int(case.ctx_lens[u]) - 1) // bs
        for b in range(int(start[u]), cur_block + 1):
            phys = 1 + int(slots[u]) * wb + b % wb
            assert phys == ring_pt[u, b - int(start[u])]
            ring_k[phys] = case.k_cache[int(case.page_table[u, b])]
            ring_v[phys] = case.v_cache[int(case.page_table[u, b])]
    out = ops.paged_decode(
        case.q.reshape(users, 8, hd).cuda(), ring_k.cuda(), ring_v.cuda(),
        torch.from_numpy(ring_pt.astype(np.int32)).cuda(),
        torch.from_numpy(pos_rel.astype(np.int32)).cuda(), scale=case.scale,
        sliding_window=window,
    ).cpu()
    assert_attention_close(out, want, "ring decode")
