"""vLLM varlen form through forward(): decode rows and prefill / chunk rows in one batch (the
shape of benchmark config 3, scaled to sizes the oracle finishes in seconds).  The reference never
mixes the two in one pass (its scheduler runs prefill first, ascend_scheduler.py:486-489), so the
expected result is the concatenation of its two passes: the decode op over the decode rows and
the chunked op over the chunk rows.  Cache writes bit-exact, outputs within the bf16 budget."""
import pytest
import torch

from oracle import restate
from oracle.inputs import randn_bf16
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def build_mixed(nq, nkv, hd, bs, dec_ctx, chunk_prefix, chunk_len, seed):
    """dec_ctx: context lengths (incl. the new token) of the decode rows; then len(chunk_prefix)
    chunk rows of chunk_len tokens on prefixes chunk_prefix."""
    g = torch.Generator().manual_seed(seed)
    seq_lens = list(dec_ctx) + [p + chunk_len for p in chunk_prefix]
    q_lens = [1] * len(dec_ctx) + [chunk_len] * len(chunk_prefix)
    nblks = [(L + bs - 1) // bs for L in seq_lens]
    width = max(nblks)
    nb = sum(nblks) + 1
    perm = torch.randperm(nb - 1, generator=g) + 1
    bt = torch.zeros(len(seq_lens), width, dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblks):
        bt[i, :n] = perm[o:o + n].int()
        o += n
    k_cache = randn_bf16((nb, nkv, bs, hd), g)
    v_cache = randn_bf16((nb, nkv, bs, hd), g)
    total = sum(q_lens)
    q = randn_bf16((total, nq * hd), g)
    k = randn_bf16((total, nkv * hd), g)
    v = randn_bf16((total, nkv * hd), g)
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    slots = []
    for i, (L, ql) in enumerate(zip(seq_lens, q_lens)):
        for pos in range(L - ql, L):
            slots.append(int(bt[i, pos // bs]) * bs + pos % bs)
    return dict(seq_lens=torch.tensor(seq_lens, dtype=torch.int32), q_lens=q_lens, bt=bt,
                k_cache=k_cache, v_cache=v_cache, q=q, k=k, v=v, qsl=qsl,
                slots=torch.tensor(slots, dtype=torch.int64), nblks=nblks)


def oracle_mixed(m, nq, nkv, hd, bs, n_dec, scale):
    """Reference semantics: write every new token, then pass A (decode op) + pass B (chunked op
    per chunk row)."""
    kc, vc = m["k_cache"].clone(), m["v_cache"].clone()
    for t, slot in enumerate(m["slots"].tolist()):
        kc[slot // bs, :, slot % bs] = m["k"][t].view(nkv, hd)
        vc[slot // bs, :, slot % bs] = m["v"][t].view(nkv, hd)
    outs = []
    if n_dec:
        pos = (m["seq_lens"][:n_dec] - 1).int()
        o = restate.paged_sdpa_decode(m["q"][:n_dec].view(1, n_dec, nq, hd).float(), kc.float(),
                                      vc.float(), m["bt"][:n_dec], pos, scale)[0]
        outs.append(o.reshape(n_dec, nq * hd))
    for i in range(n_dec, len(m["q_lens"])):
        a, b = int(m["qsl"][i]), int(m["qsl"][i + 1])
        start = int(m["seq_lens"][i]) - (b - a)
        qi = m["q"][a:b].view(b - a, nq, hd).transpose(0, 1)[None].float()
        o = restate.chunked_sdpa(qi, kc.float(), vc.float(), m["bt"][i:i + 1, :m["nblks"][i]],
                                 start, scale)[0].transpose(0, 1)
        outs.append(o.reshape(b - a, nq * hd))
    return torch.cat(outs), kc, vc


@pytest.mark.parametrize("fused_cache", [False, True])
def test_mixed_decode_and_chunk_rows(fused_cache, clean_error_word):
    from b200attn import B200AttentionBackendImpl
    from b200attn.backend import build_varlen_metadata

    nq, nkv, hd, bs = 32, 8, 128, 64
    g = torch.Generator().manual_seed(3)
    dec_ctx = torch.randint(100, 900, (12,), generator=g).tolist()
    m = build_mixed(nq, nkv, hd, bs, dec_ctx, chunk_prefix=[512, 512], chunk_len=192, seed=33)
    scale = hd ** -0.5
    want, want_k, want_v = oracle_mixed(m, nq, nkv, hd, bs, len(dec_ctx), scale)

    impl = B200AttentionBackendImpl(nq, hd, scale, nkv, None, None, "auto")
    md = build_varlen_metadata(m["qsl"].cuda(), m["qsl"], m["seq_lens"].cuda(), m["bt"].cuda(),
                               m["slots"].cuda(), max_seq_len=int(m["seq_lens"].max()))
    assert md.num_decodes == 12
    if fused_cache:   # vLLM's single tensor per layer
        kv = torch.stack([m["k_cache"], m["v_cache"]]).cuda()
    else:
        kv = [m["k_cache"].cuda(), m["v_cache"].cuda()]
    out = torch.empty(m["q"].shape[0], nq * hd, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, m["q"].cuda(), m["k"].cuda(), m["v"].cuda(), kv, md, output=out)
    assert torch.equal(kv[0].cpu(), want_k) and torch.equal(kv[1].cpu(), want_v)
    assert_attention_close(out, want, "mixed batch")


def test_pure_decode_and_pure_prefill_varlen(clean_error_word):
    from b200attn import B200AttentionBackendImpl
    from b200attn.backend import build_varlen_metadata

    nq, nkv, hd, bs = 8, 2, 64, 32
    scale = hd ** -0.5
    impl = B200AttentionBackendImpl(nq, hd, scale, nkv, None, None, "auto")
    for dec_ctx, prefixes, clen in (([5, 64, 65, 300], [], 0), ([], [0, 32, 96], 70)):
        m = build_mixed(nq, nkv, hd, bs, dec_ctx, prefixes, clen, seed=len(dec_ctx) + 5)
        want, want_k, want_v = oracle_mixed(m, nq, nkv, hd, bs, len(dec_ctx), scale)
        md = build_varlen_metadata(m["qsl"].cuda(), m["qsl"], m["seq_lens"].cuda(),
                                   m["bt"].cuda(), m["slots"].cuda())
        kv = [m["k_cache"].cuda(), m["v_cache"].cuda()]
        out = torch.empty(m["q"].shape[0], nq * hd, dtype=torch.bfloat16, device="cuda")
        impl.forward(None, m["q"].cuda(), m["k"].cuda(), m["v"].cuda(), kv, md, output=out)
        assert torch.equal(kv[0].cpu(), want_k) and torch.equal(kv[1].cpu(), want_v)
        assert_attention_close(out, want, f"varlen dec={len(dec_ctx)} pre={len(prefixes)}")


def test_many_sequences_use_plain_item_order(clean_error_word):
    """More than 64 sequences switch the prefill kernel's item order to the plain one; results
    must not depend on the order."""
    from b200attn import ops

    g = torch.Generator().manual_seed(9)
    nq, nkv, hd, S = 4, 2, 64, 70
    lens = torch.randint(1, 300, (S,), generator=g).tolist()
    total = sum(lens)
    q = randn_bf16((total, nq, hd), g)
    k = randn_bf16((total, nkv, hd), g)
    v = randn_bf16((total, nkv, hd), g)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    out = ops.prefill(q.cuda(), k.cuda(), v.cuda(), cu, scale=hd ** -0.5).cpu()
    for i in (0, 1, 17, 42, 69):
        a, b = int(cu[i]), int(cu[i + 1])
        want = restate.sdpa(q[a:b].transpose(0, 1)[None].float(), k[a:b].transpose(0, 1)[None].float(),
                            v[a:b].transpose(0, 1)[None].float(), True, hd ** -0.5)[0].transpose(0, 1)
        assert_attention_close(out[a:b], want, f"seq {i}")


def test_more_sequences_than_the_shared_memory_cache_holds(clean_error_word):
    """Above 1024 sequences the prefill kernel reads the sequence offsets from global memory
    instead of its shared-memory copy, and a CTA has more rounds than its item table holds."""
    from b200attn import ops

    g = torch.Generator().manual_seed(19)
    nq, nkv, hd, S = 32, 2, 64, 1100      # 35200 items: 238 rounds per CTA, table holds 128
    lens = torch.randint(1, 40, (S,), generator=g).tolist()
    total = sum(lens)
    q = randn_bf16((total, nq, hd), g)
    k = randn_bf16((total, nkv, hd), g)
    v = randn_bf16((total, nkv, hd), g)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    out = ops.prefill(q.cuda(), k.cuda(), v.cuda(), cu, scale=hd ** -0.5).cpu()
    for i in (0, 1, 511, 1023, 1024, 1099):
        a, b = int(cu[i]), int(cu[i + 1])
        want = restate.sdpa(q[a:b].transpose(0, 1)[None].float(), k[a:b].transpose(0, 1)[None].float(),
                            v[a:b].transpose(0, 1)[None].float(), True, hd ** -0.5)[0].transpose(0, 1)
        assert_attention_close(out[a:b], want, f"seq {i}")


def test_a_list_too_long_to_tabulate_is_searched(clean_error_word):
    """More 128-row blocks than the kernel tabulates (1024): the drawing thread finds each item
    by a scan of cu_q instead.  Three sequences, 1040 blocks in all; rows at the start, around
    a sequence boundary and at the very end are compared with fp32 attention computed by torch
    over the same bf16 inputs."""
    from b200attn import ops

    nq, nkv, hd = 2, 1, 64
    lens = [70000, 128 * 3 + 5, 62000]
    assert sum((n + 127) // 128 for n in lens) > 1024
    cu_q = torch.tensor([0, lens[0], lens[0] + lens[1], sum(lens)], dtype=torch.int32)
    total = int(cu_q[-1])
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(total, nq, hd, generator=g, device="cuda").bfloat16()
    k = torch.randn(total, nkv, hd, generator=g, device="cuda").bfloat16()
    v = torch.randn(total, nkv, hd, generator=g, device="cuda").bfloat16()
    out = ops.prefill(q, k, v, cu_q, scale=hd ** -0.5)
    assert ops.read_error_word() == 0
    for s, (lo, n) in enumerate(zip(cu_q[:-1].tolist(), lens)):
        rows = sorted({0, 1, 127, 128, n // 2, n - 2, n - 1})
        for h in range(nq):
            qs = q[lo:lo + n, h].float()[rows]                      # [r, hd]
            ks, vs = k[lo:lo + n, 0].float(), v[lo:lo + n, 0].float()
            sc = (qs @ ks.t()) * hd ** -0.5
            pos = torch.tensor(rows, device="cuda")[:, None]
            sc = sc.masked_fill(torch.arange(n, device="cuda")[None, :] > pos, float("-inf"))
            want = torch.softmax(sc, -1) @ vs
            assert_attention_close(out[lo:lo + n, h][rows], want, f"sequence {s} head {h}")
