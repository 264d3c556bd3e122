"""Seeded random geometry sweep of the three kernels against the oracle: head counts, group
sizes 1..16, both head sizes and block sizes, ragged lengths, page tables wider than needed,
strided inputs.  Scatter bit-exact, attention within the bf16 budget."""
import pytest
import torch

from oracle import restate
from oracle.inputs import randn_bf16
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def _rand_geometry(g):
    hd = [64, 128][int(torch.randint(0, 2, (1,), generator=g))]
    bs = [32, 64][int(torch.randint(0, 2, (1,), generator=g))]
    nkv = int(torch.randint(1, 5, (1,), generator=g))
    group = [1, 2, 3, 4, 5, 7, 8, 16][int(torch.randint(0, 8, (1,), generator=g))]
    return hd, bs, nkv, nkv * group


@pytest.mark.parametrize("seed", range(12))
def test_random_decode(seed, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(1000 + seed)
    hd, bs, nkv, nq = _rand_geometry(g)
    users = int(torch.randint(1, 40, (1,), generator=g))
    max_ctx = int(torch.randint(1, 1500, (1,), generator=g))
    ctx = torch.randint(1, max_ctx + 1, (users,), generator=g)
    width = (max_ctx + bs - 1) // bs + int(torch.randint(0, 5, (1,), generator=g))   # slack columns
    nb = users * width + 2
    pt = torch.randperm(nb, generator=g)[: users * width].reshape(users, width).int()
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    # query rows with a stride larger than nq*hd (a view into a wider buffer)
    qbuf = randn_bf16((users, nq * hd + 64), g)
    q = qbuf[:, : nq * hd].reshape(users, nq, hd)
    pos = (ctx - 1).int()
    want = restate.paged_sdpa_decode(q[None].float(), kc.float(), vc.float(), pt, pos, hd ** -0.5)[0]
    for splits in (0, 1, int(torch.randint(2, 9, (1,), generator=g))):
        out = ops.paged_decode(qbuf.cuda()[:, : nq * hd].reshape(users, nq, hd), kc.cuda(), vc.cuda(),
                               pt.cuda(), pos.cuda(), scale=hd ** -0.5, num_splits=splits)
        assert_attention_close(out, want, f"seed {seed} hd{hd} bs{bs} nq{nq}/nkv{nkv} splits {splits}")


@pytest.mark.parametrize("seed", range(10))
def test_random_prefill(seed, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(2000 + seed)
    hd, bs, nkv, nq = _rand_geometry(g)
    nseq = int(torch.randint(1, 6, (1,), generator=g))
    q_lens = torch.randint(1, 400, (nseq,), generator=g).tolist()
    starts = [int(torch.randint(0, 6, (1,), generator=g)) * bs for _ in range(nseq)]
    if seed % 3 == 0:
        starts = [s + int(torch.randint(0, bs, (1,), generator=g)) for s in starts]   # unaligned prefix
    nblks = [(s + t + bs - 1) // bs for s, t in zip(starts, q_lens)]
    width = max(nblks) + 1
    nb = sum(nblks) + 1
    perm = torch.randperm(nb - 1, generator=g) + 1
    pt = torch.zeros(nseq, width, dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblks):
        pt[i, :n] = perm[o:o + n].int()
        o += n
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    total = sum(q_lens)
    q = randn_bf16((total, nq, hd), g)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    out = ops.prefill(q.cuda(), kc.cuda(), vc.cuda(), cu, scale=hd ** -0.5, page_table=pt.cuda(),
                      q_start=torch.tensor(starts, dtype=torch.int32).cuda()).cpu()
    for i, (t, s) in enumerate(zip(q_lens, starts)):
        a, b = int(cu[i]), int(cu[i + 1])
        qi = q[a:b].transpose(0, 1)[None].float()
        want = restate.chunked_sdpa(qi, kc.float(), vc.float(), pt[i:i + 1, :nblks[i]], s,
                                    hd ** -0.5)[0].transpose(0, 1)
        assert_attention_close(out[a:b], want, f"seed {seed} seq {i} hd{hd} bs{bs} nq{nq}/nkv{nkv}")


@pytest.mark.parametrize("seed", range(6))
def test_random_scatter_slots(seed, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(3000 + seed)
    hd, bs, nkv, _ = _rand_geometry(g)
    nb = int(torch.randint(4, 64, (1,), generator=g))
    n = int(torch.randint(1, nb * bs, (1,), generator=g))
    slots = torch.randperm(nb * bs, generator=g)[:n].long()
    slots[torch.rand(n, generator=g) < 0.1] = -1
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    kbuf = randn_bf16((n, nkv * hd + 8), g)       # strided rows
    vbuf = randn_bf16((n, nkv * hd + 8), g)
    want_k, want_v = kc.clone(), vc.clone()
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            want_k[s // bs, :, s % bs] = kbuf[t, : nkv * hd].view(nkv, hd)
            want_v[s // bs, :, s % bs] = vbuf[t, : nkv * hd].view(nkv, hd)
    kcd, vcd = kc.cuda(), vc.cuda()
    ops.kv_scatter_slots(kcd, vcd, kbuf.cuda()[:, : nkv * hd].reshape(n, nkv, hd),
                         vbuf.cuda()[:, : nkv * hd].reshape(n, nkv, hd), slots.cuda())
    assert torch.equal(kcd.cpu(), want_k) and torch.equal(vcd.cpu(), want_v)
