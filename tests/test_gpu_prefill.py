"""Causal / chunked prefill kernel (tcgen05) against the oracle and the reference golden vectors
(bf16 tolerance: max abs <= 2e-2, mean abs <= 2e-3 against fp32 arithmetic)."""
import pytest
import torch

from oracle import restate
from oracle.inputs import make_prefill_case, randn_bf16
from tests.conftest import assert_attention_close
from tests.golden.golden_io import load_case

pytestmark = pytest.mark.gpu


def cu(users, T):
    return torch.arange(users + 1, dtype=torch.int32) * T


def test_sdpa_golden(clean_error_word):
    from b200attn import ops

    c = load_case("sdpa_gqa")
    B, nq, T, hd = c["q"].shape
    nkv = c["k"].shape[1]
    q = c["q"].transpose(1, 2).reshape(B * T, nq, hd).contiguous().cuda()
    k = c["k"].transpose(1, 2).reshape(B * T, nkv, hd).contiguous().cuda()
    v = c["v"].transpose(1, 2).reshape(B * T, nkv, hd).contiguous().cuda()
    out = ops.prefill(q, k, v, cu(B, T), scale=float(c["scale"]))
    got = out.reshape(B, T, nq, hd).transpose(1, 2)
    assert_attention_close(got, c["out_fp32"], "sdpa golden")


@pytest.mark.parametrize("start", [0, 64, 96])
def test_chunked_golden(start, clean_error_word):
    from b200attn import ops

    c = load_case(f"chunked_start{start}")
    users, nq, T, hd = c["q"].shape
    q = c["q"].transpose(1, 2).reshape(users * T, nq, hd).contiguous().cuda()
    out = ops.prefill(
        q, c["k_cache"].cuda(), c["v_cache"].cuda(), cu(users, T), scale=float(c["scale"]),
        page_table=c["page_table"].cuda(),
        q_start=torch.full((users,), start, dtype=torch.int32, device="cuda"),
    )
    got = out.reshape(users, T, nq, hd).transpose(1, 2)
    assert_attention_close(got, c["out_fp32"], f"chunked golden start={start}")


# reference CPU test parametrisation (tests/torch/ops/test_chunked_sdpa_op_cpu.py): MHA, GQA 8/2
# and 32/8, chunk_start 0 / 64 / 96, plus the supported larger geometries
@pytest.mark.parametrize("nq,nkv", [(4, 4), (8, 2), (32, 8)])
@pytest.mark.parametrize("hd,bs", [(64, 32), (128, 64)])
@pytest.mark.parametrize("T,start", [(64, 0), (64, 64), (32, 96), (256, 0), (192, 320)])
def test_chunked_vs_oracle(nq, nkv, hd, bs, T, start, clean_error_word):
    from b200attn import ops

    if start % bs:
        pytest.skip("chunks start on a block boundary")
    case = make_prefill_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=2, T=T, chunk_start=start,
                             seed=nq * 3 + T + start)
    # write the chunk's K/V into the cache on the CPU with the oracle, then attend on the GPU
    k = case.k.reshape(2, T, nkv, hd)
    v = case.v.reshape(2, T, nkv, hd)
    kc = restate.paged_fill_cache(case.k_cache, k.transpose(1, 2), case.fill_page_table)
    vc = restate.paged_fill_cache(case.v_cache, v.transpose(1, 2), case.fill_page_table)
    q4 = case.q.reshape(2, T, nq, hd)
    want = restate.chunked_sdpa(q4.transpose(1, 2).float(), kc.float(), vc.float(),
                                case.page_table, start, case.scale).transpose(1, 2)
    out = ops.prefill(
        case.q.reshape(2 * T, nq, hd).cuda(), kc.cuda(), vc.cuda(), cu(2, T), scale=case.scale,
        page_table=case.page_table.cuda(),
        q_start=torch.full((2,), start, dtype=torch.int32, device="cuda"),
    )
    assert_attention_close(out.reshape(2, T, nq, hd), want, "chunked vs oracle")


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("T", [32, 128, 160, 512])
def test_fresh_kv_causal_vs_oracle(hd, T, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(T + hd)
    B, nq, nkv = 3, 8, 2
    q = randn_bf16((B, T, nq, hd), g)
    k = randn_bf16((B, T, nkv, hd), g)
    v = randn_bf16((B, T, nkv, hd), g)
    want = restate.sdpa(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                        v.transpose(1, 2).float(), True, hd ** -0.5).transpose(1, 2)
    out = ops.prefill(q.reshape(B * T, nq, hd).cuda(), k.reshape(B * T, nkv, hd).cuda(),
                      v.reshape(B * T, nkv, hd).cuda(), cu(B, T), scale=hd ** -0.5)
    assert_attention_close(out.reshape(B, T, nq, hd), want, "fresh causal")


def test_varlen_ragged_lengths_and_starts(clean_error_word):
    """Sequences of different query lengths and different prefix lengths in one call (a superset
    of the reference's single shared chunk_start): each sequence equals its own oracle call."""
    from b200attn import ops

    g = torch.Generator().manual_seed(77)
    nq, nkv, hd, bs = 8, 2, 128, 64
    q_lens = [1, 37, 128, 200]
    starts = [300, 64, 0, 128]
    nblks = [(s + t + bs - 1) // bs for s, t in zip(starts, q_lens)]
    width = max(nblks)
    nb = sum(nblks) + 1
    perm = torch.randperm(nb - 1, generator=g) + 1
    pt = torch.zeros(len(q_lens), width, dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblks):
        pt[i, :n] = perm[o:o + n].int()
        o += n
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    total = sum(q_lens)
    q = randn_bf16((total, nq, hd), g)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    out = ops.prefill(q.cuda(), kc.cuda(), vc.cuda(), cu_q, scale=hd ** -0.5,
                      page_table=pt.cuda(),
                      q_start=torch.tensor(starts, dtype=torch.int32).cuda()).cpu()
    for i, (t, s) in enumerate(zip(q_lens, starts)):
        qi = q[cu_q[i]:cu_q[i + 1]].transpose(0, 1)[None].float()      # [1,nq,t,hd]
        want = restate.chunked_sdpa(qi, kc.float(), vc.float(), pt[i:i + 1, :nblks[i]], s,
                                    hd ** -0.5)[0].transpose(0, 1)
        assert_attention_close(out[cu_q[i]:cu_q[i + 1]], want, f"seq {i}")


def test_paged_and_fresh_forms_agree_at_config2_shape(clean_error_word):
    """benchmark config 2 geometry (nq 32, nkv 8, hd 128, bs 64, T 2048) on one sequence: the
    paged form with chunk_start 0 and the fresh-KV form give the same bits, and rows are
    checked against the oracle on a strided subset of heads."""
    from b200attn import ops

    case = make_prefill_case(nq=32, nkv=8, hd=128, bs=64, users=1, T=2048, seed=2)
    T, nq, nkv, hd = case.T, case.nq, case.nkv, case.hd
    q = case.q.reshape(T, nq, hd).cuda()
    k = case.k.reshape(T, nkv, hd).cuda()
    v = case.v.reshape(T, nkv, hd).cuda()
    kc, vc = case.k_cache.cuda(), case.v_cache.cuda()
    ops.paged_fill_cache(kc, vc, k[None], v[None], case.fill_page_table.cuda())
    fresh = ops.prefill(q, k, v, cu(1, T), scale=case.scale)
    paged = ops.prefill(q, kc, vc, cu(1, T), scale=case.scale, page_table=case.page_table.cuda(),
                        q_start=torch.zeros(1, dtype=torch.int32, device="cuda"))
    assert torch.equal(fresh, paged)
    heads = [0, 5, 31]
    kv_heads = [h // (nq // nkv) for h in heads]
    qh = case.q.reshape(T, nq, hd)[:, heads].transpose(0, 1)[None].float()
    for i, (h, kh) in enumerate(zip(heads, kv_heads)):
        want = restate.sdpa(qh[:, i:i + 1], case.k.reshape(T, nkv, hd)[:, kh][None, None].float(),
                            case.v.reshape(T, nkv, hd)[:, kh][None, None].float(), True,
                            case.scale)[0, 0]
        assert_attention_close(fresh[:, h], want, f"head {h}")


def _fresh_inputs(users, T, nq, nkv, hd, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda h: torch.randn(users * T, h, hd, generator=g, device="cuda").bfloat16()
    return mk(nq), mk(nkv), mk(nkv)


def test_a_captured_launch_replays_with_a_fresh_item_counter(clean_error_word):
    """The CTAs draw their work items from a counter word that carries the launch's tag; a CUDA
    graph replays the launch with the SAME tag, so the word has to be back at zero after every
    run.  Replays on new inputs must give the bits of an eager call on those inputs."""
    from b200attn import ops

    users, T, nq, nkv, hd = 3, 640, 8, 2, 128
    cu_host = cu(users, T)
    cu_dev = cu_host.cuda()
    q, k, v = _fresh_inputs(users, T, nq, nkv, hd, 1)
    out = torch.empty_like(q)
    ops.prefill(q, k, v, cu_host, scale=hd ** -0.5, out=out, cu_q=cu_dev)      # warm-up, eager
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            ops.prefill(q, k, v, cu_host, scale=hd ** -0.5, out=out, cu_q=cu_dev)
    torch.cuda.current_stream().wait_stream(side)
    for seed in (2, 3, 4, 5):
        q2, k2, v2 = _fresh_inputs(users, T, nq, nkv, hd, seed)
        want = ops.prefill(q2, k2, v2, cu_host, scale=hd ** -0.5, cu_q=cu_dev)
        q.copy_(q2), k.copy_(k2), v.copy_(v2)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want), f"replay with seed {seed}"
    assert ops.read_error_word() == 0


def test_launches_on_two_streams_keep_their_item_lists_apart(clean_error_word):
    """Two prefill launches in flight at once (one per stream) draw from different counter
    words; each must cover all of its own items."""
    from b200attn import ops

    users, T, nq, nkv, hd = 4, 1024, 16, 4, 128
    cu_host = cu(users, T)
    cu_dev = cu_host.cuda()
    a = _fresh_inputs(users, T, nq, nkv, hd, 11)
    b = _fresh_inputs(users, T, nq, nkv, hd, 12)
    want_a = ops.prefill(*a, cu_host, scale=hd ** -0.5, cu_q=cu_dev)
    want_b = ops.prefill(*b, cu_host, scale=hd ** -0.5, cu_q=cu_dev)
    out_a, out_b = torch.empty_like(want_a), torch.empty_like(want_b)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    for _ in range(8):
        out_a.zero_(), out_b.zero_()
        torch.cuda.synchronize()
        with torch.cuda.stream(s1):
            ops.prefill(*a, cu_host, scale=hd ** -0.5, out=out_a, cu_q=cu_dev)
        with torch.cuda.stream(s2):
            ops.prefill(*b, cu_host, scale=hd ** -0.5, out=out_b, cu_q=cu_dev)
        torch.cuda.synchronize()
        assert torch.equal(out_a, want_a) and torch.equal(out_b, want_b)
    assert ops.read_error_word() == 0


@pytest.mark.parametrize("bs,hd", [(64, 128), (32, 64)])
def test_non_finite_cache_slots_past_the_context_do_not_leak(bs, hd, clean_error_word):
    """A live cache holds stale data in the slots of the last page that were never written, and
    in pages listed beyond the context.  NaN / Inf there must not reach any output row (their
    weights are zero, but 0 x NaN is NaN unless the rows are neutralised)."""
    from b200attn import ops

    g = torch.Generator().manual_seed(31 + bs)
    nq, nkv = 8, 2
    q_lens, starts = [70, 129, 200], [64, 0, 128]
    nblks = [(s + t + bs - 1) // bs for s, t in zip(starts, q_lens)]
    width = max(nblks) + 1
    nb = sum(nblks) + 2
    perm = torch.randperm(nb - 1, generator=g) + 1
    pt = torch.zeros(len(q_lens), width, dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblks):
        pt[i, :n] = perm[o:o + n].int()
        o += n
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    total = sum(q_lens)
    q = randn_bf16((total, nq, hd), g)
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    wants = []
    for i, (t, s) in enumerate(zip(q_lens, starts)):
        qi = q[cu_q[i]:cu_q[i + 1]].transpose(0, 1)[None].float()
        wants.append(restate.chunked_sdpa(qi, kc.float(), vc.float(), pt[i:i + 1, :nblks[i]], s,
                                          hd ** -0.5)[0].transpose(0, 1))
    # now poison everything past each context: the tail of the last page, and block 0 (which the
    # unused page-table columns point at)
    kc[0], vc[0] = float("nan"), float("inf")
    for i, (t, s) in enumerate(zip(q_lens, starts)):
        ctx = s + t
        if ctx % bs:
            blk = int(pt[i, ctx // bs])
            kc[blk, :, ctx % bs:] = float("nan")
            vc[blk, :, ctx % bs:] = float("-inf")
    out = ops.prefill(q.cuda(), kc.cuda(), vc.cuda(), cu_q, scale=hd ** -0.5, page_table=pt.cuda(),
                      q_start=torch.tensor(starts, dtype=torch.int32).cuda()).cpu()
    for i in range(len(q_lens)):
        assert_attention_close(out[cu_q[i]:cu_q[i + 1]], wants[i], f"seq {i}")


def test_query_offsets_must_start_at_zero_and_stay_inside_q():
    """Rows are addressed absolutely (cu_q[s] + row): offsets that start above 0 or end past the
    query tensor are refused before anything is launched."""
    from b200attn import _lib, ops

    q = torch.zeros(64, 4, 64, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(64, 2, 64, dtype=torch.bfloat16, device="cuda")
    for bad in ([32, 64], [0, 96]):
        with pytest.raises(_lib.B200AttnError, match="bad argument"):
            ops.prefill(q, k, k, torch.tensor(bad, dtype=torch.int32), scale=0.125)
    assert ops.prefill(q, k, k, torch.tensor([0, 64], dtype=torch.int32), scale=0.125).shape == q.shape
