"""Layers that share another layer's KV cache (`kv_sharing_target_layer_name`: prefill reads the
target's pages and writes nothing, decode writes nothing; attention.py:309-314, 562-574, 600-632),
the layer wrapper for callers outside vLLM (attention.py:774-856) on caches made by
`allocate_kv_caches`, and the per-step watch on the diagnostics word."""
import pytest
import torch

from oracle import restate
from oracle.inputs import make_decode_case, make_prefill_case, randn_bf16
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def gather_paged_to_dense(cache, page_table, num_tokens):
    """The reference's `_gather_paged_to_dense` (attention.py:600-632) in one expression:
    [users, nkv, num_tokens, hd] from a paged cache."""
    users, nblk = page_table.shape
    nb, nkv, bs, hd = cache.shape
    g = cache[page_table.reshape(-1).long()].view(users, nblk, nkv, bs, hd)
    return g.permute(0, 2, 1, 3, 4).reshape(users, nkv, nblk * bs, hd)[:, :, :num_tokens]


@pytest.mark.parametrize("hd,bs,T", [(64, 32, 96), (128, 64, 256)])
def test_shared_kv_prefill_reads_target_pages_and_writes_nothing(hd, bs, T, clean_error_word):
    from b200attn import B200AttentionBackendImpl, B200Metadata

    pc = make_prefill_case(nq=8, nkv=2, hd=hd, bs=bs, users=2, T=T, seed=hd + T)
    users, nq, nkv = pc.users, pc.nq, pc.nkv
    # the target layer's cache already holds the K / V of these tokens
    k4 = pc.k.view(users, T, nkv, hd)
    v4 = pc.v.view(users, T, nkv, hd)
    kc = restate.paged_fill_cache(pc.k_cache, k4.transpose(1, 2), pc.fill_page_table)
    vc = restate.paged_fill_cache(pc.v_cache, v4.transpose(1, 2), pc.fill_page_table)
    want = restate.sdpa(pc.q.view(users, T, nq, hd).transpose(1, 2).float(),
                        gather_paged_to_dense(kc, pc.page_table, T).float(),
                        gather_paged_to_dense(vc, pc.page_table, T).float(), True,
                        pc.scale).transpose(1, 2)

    impl = B200AttentionBackendImpl(nq, hd, pc.scale, nkv, None, None, "auto",
                                    kv_sharing_target_layer_name="layers.0.attn")
    kv = [kc.cuda(), vc.cuda()]
    md = B200Metadata(cache_position=torch.full((users,), T - 1, dtype=torch.int32).cuda(),
                      page_table=pc.page_table.cuda(), fill_page_table=pc.fill_page_table.cuda(),
                      batch_idx=torch.arange(users, dtype=torch.int32).cuda(), num_users=users)
    out = torch.empty(users * T, nq * hd, dtype=torch.bfloat16, device="cuda")
    # this layer's own key / value are not used by a sharing layer: hand it garbage
    junk = torch.full_like(pc.k, float("nan")).cuda()
    impl.forward(None, pc.q.cuda(), junk, junk, kv, md, output=out)
    assert torch.equal(kv[0].cpu(), kc) and torch.equal(kv[1].cpu(), vc)
    assert_attention_close(out.view(users, T, nq, hd), want, "shared-KV prefill")


def test_shared_kv_decode_writes_nothing(clean_error_word):
    from b200attn import B200AttentionBackendImpl, B200Metadata

    case = make_decode_case(nq=8, nkv=2, hd=128, bs=64, users=4, ctx_lo=30, ctx_hi=400, seed=5)
    want = restate.paged_sdpa_decode(case.q.view(1, 4, 8, 128).float(), case.k_cache.float(),
                                     case.v_cache.float(), case.page_table, case.cache_position,
                                     case.scale)[0]
    kv = [case.k_cache.cuda(), case.v_cache.cuda()]
    md = B200Metadata(cache_position=case.cache_position.cuda(),
                      page_table=case.page_table.cuda(), num_users=4)
    out = torch.empty(4, 8 * 128, dtype=torch.bfloat16, device="cuda")
    for form in ("plugin", "varlen"):
        impl = B200AttentionBackendImpl(8, 128, case.scale, 2, None, None, "auto",
                                        kv_sharing_target_layer_name="layers.3.attn")
        if form == "varlen":
            from b200attn.backend import build_varlen_metadata

            qsl = torch.arange(5, dtype=torch.int32)
            slots = torch.tensor([int(case.page_table[u, int(p) // 64]) * 64 + int(p) % 64
                                  for u, p in enumerate(case.cache_position)])
            md = build_varlen_metadata(qsl.cuda(), qsl, case.ctx_lens.int().cuda(),
                                       case.page_table.cuda(), slots.cuda())
        impl.forward(None, case.q.cuda(), case.k.cuda(), case.v.cuda(), kv, md, output=out)
        assert torch.equal(kv[0].cpu(), case.k_cache) and torch.equal(kv[1].cpu(), case.v_cache)
        assert_attention_close(out.view(4, 8, 128), want, f"shared-KV decode ({form})")


def test_layer_wrapper_on_allocated_caches(clean_error_word):
    """4-D prefill inputs, then a 3-D decode step, through B200Attention on caches from
    allocate_kv_caches; the result keeps the query's shape and matches the oracle's forward."""
    from b200attn import B200Attention, B200Metadata, sharding

    nq, nkv, hd, bs, users, T = 8, 2, 128, 64, 2, 96
    pc = make_prefill_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=users, T=T, seed=8)
    layer = B200Attention(nq, hd, pc.scale, num_kv_heads=nkv)
    caches = sharding.allocate_kv_caches(["attn"], pc.nb, nkv, bs, hd, device="cuda")
    sharding.bind_kv_caches({"attn": layer}, caches)
    bidx = torch.arange(users, dtype=torch.int32)
    md = B200Metadata(cache_position=torch.full((users,), T - 1, dtype=torch.int32).cuda(),
                      page_table=pc.page_table.cuda(), fill_page_table=pc.fill_page_table.cuda(),
                      batch_idx=bidx.cuda(), num_users=users)
    want, want_k, want_v = restate.impl_forward(
        pc.q, pc.k, pc.v, pc.k_cache, pc.v_cache, num_heads=nq, num_kv_heads=nkv, head_size=hd,
        scale=pc.scale, num_users=users,
        cache_position=torch.full((users,), T - 1, dtype=torch.int32), page_table=pc.page_table,
        fill_page_table=pc.fill_page_table, batch_idx=bidx, compute_dtype=torch.float32)
    q4 = pc.q.view(users, T, nq, hd).cuda()
    out = layer(q4, pc.k.view(users, T, nkv, hd).cuda(), pc.v.view(users, T, nkv * hd).cuda(),
                attn_metadata=md)
    assert out.shape == q4.shape
    assert torch.equal(caches["attn"][0].cpu(), want_k) and torch.equal(caches["attn"][1].cpu(), want_v)
    assert_attention_close(out.reshape(users * T, nq * hd), want, "wrapper prefill")

    # one decode step on top: position T, 3-D inputs [users, heads, hd]
    g = torch.Generator().manual_seed(1)
    q, k, v = (randn_bf16((users, h, hd), g) for h in (nq, nkv, nkv))
    pos = torch.full((users,), T, dtype=torch.int32)
    layer.set_metadata(B200Metadata(cache_position=pos.cuda(), page_table=pc.page_table.cuda(),
                                    num_users=users))
    want, want_k2, want_v2 = restate.impl_forward(
        q.reshape(users, -1), k.reshape(users, -1), v.reshape(users, -1), want_k, want_v,
        num_heads=nq, num_kv_heads=nkv, head_size=hd, scale=pc.scale, num_users=users,
        cache_position=pos, page_table=pc.page_table, compute_dtype=torch.float32)
    out = layer(q.cuda(), k.cuda(), v.cuda())
    assert out.shape == q.shape
    assert torch.equal(caches["attn"][0].cpu(), want_k2)
    assert_attention_close(out.reshape(users, nq * hd), want, "wrapper decode")


def test_error_watch_reports_a_bad_page_id_one_poll_later():
    """The watch never synchronises: the poll after the one that queued the copy raises."""
    from b200attn import ops

    ops.read_error_word()
    watch = ops.ErrorWordWatch()
    watch.poll()
    kc = torch.zeros(4, 1, 32, 64, dtype=torch.bfloat16, device="cuda")
    new = torch.ones(1, 1, 64, dtype=torch.bfloat16, device="cuda")
    ops.kv_scatter_slots(kc, kc.clone(), new, new, torch.tensor([4 * 32 + 1], device="cuda"))
    watch.poll()                      # queues the copy that sees word 2
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="outside the KV cache"):
        watch.poll()
    assert ops.read_error_word() == 0 and float(kc.abs().sum()) == 0
    watch.poll()


def test_layer_wrapper_rotary_writes_the_cache_in_the_same_launch(clean_error_word):
    """A layer built with rotary_dim gets positions: q and k are rotated in place and, because the
    step's metadata carries a slot mapping, the rotated k and v land in the cache in that one
    launch; the Impl then only attends.  Checked against the rotary restatement followed by the
    oracle's forward (rotation arithmetic as the plugin's rotary layer does it: within 2 bf16 ulps
    of the CPU statement, so the comparison of the attention uses the usual budget and the cache
    is compared with the rotated k the launch returned)."""
    from b200attn import B200Attention, B200AttentionMetadataBuilder, sharding

    g = torch.Generator().manual_seed(23)
    nq, nkv, hd, bs, n, width = 8, 2, 128, 64, 4, 6
    bt = (torch.randperm(n * width, generator=g) + 1).reshape(n, width).int()
    computed = torch.randint(1, width * bs - 2, (n,), generator=g).int()
    sched = torch.ones(n, dtype=torch.int32)
    nb = n * width + 1
    layer = B200Attention(nq, hd, hd ** -0.5, num_kv_heads=nkv, rotary_dim=hd, rope_theta=500000.0)
    caches = sharding.allocate_kv_caches(["attn"], nb, nkv, bs, hd, device="cuda")
    sharding.bind_kv_caches({"attn": layer}, caches)
    kc0, vc0 = randn_bf16((nb, nkv, bs, hd), g), randn_bf16((nb, nkv, bs, hd), g)
    caches["attn"][0].copy_(kc0)
    caches["attn"][1].copy_(vc0)
    state = B200AttentionMetadataBuilder(device=torch.device("cuda")).device_step_state(
        n, width, bs, tokens_per_row=1)
    meta = state.build(computed.cuda(), sched.cuda(), bt.cuda())
    q, k, v = (randn_bf16((n, h * hd), g) for h in (nq, nkv, nkv))
    positions = computed.long()                      # the new token's position
    dq, dk = q.cuda(), k.cuda()
    out = layer(dq, dk, v.cuda(), attn_metadata=meta, positions=positions.cuda())
    assert layer.impl.kv_written_upstream is False    # consumed by the forward

    want_q, want_k = restate.rotary_embedding(positions, q, k, layer.inv_freq.cpu(), hd, hd)
    for got, want in ((dq.cpu(), want_q), (dk.cpu(), want_k)):    # rotated in place
        assert (got.float() - want.float()).abs().max() <= 2 * 2.0 ** -7 * want.float().abs().max()
    rot_q, rot_k = dq.cpu(), dk.cpu()
    want_out, want_kc, want_vc = restate.impl_forward(
        rot_q, rot_k, v, kc0, vc0, num_heads=nq, num_kv_heads=nkv, head_size=hd, scale=hd ** -0.5,
        num_users=n, cache_position=computed, page_table=bt, compute_dtype=torch.float32)
    assert torch.equal(caches["attn"][0].cpu(), want_kc) and torch.equal(caches["attn"][1].cpu(), want_vc)
    assert_attention_close(out, want_out, "rotary + cache write + decode")
