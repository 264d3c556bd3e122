"""KV-cache write kernels against the oracle and the reference golden vectors: bit-exact."""
import pytest
import torch

from oracle import restate
from oracle.inputs import randn_bf16
from tests.golden.golden_io import load_case

pytestmark = pytest.mark.gpu


def dev(t):
    return t.cuda() if isinstance(t, torch.Tensor) else t


def test_update_cache_golden(clean_error_word):
    from b200attn import ops

    c = load_case("update_cache")
    kc, vc = dev(c["k_cache"]), dev(c["v_cache"])
    ops.paged_update_cache(kc, vc, dev(c["k"]), dev(c["v"]), dev(c["update_indices"]),
                           dev(c["page_table"]))
    assert torch.equal(kc.cpu(), c["out_k"]) and torch.equal(vc.cpu(), c["out_v"])


@pytest.mark.parametrize("T", [10, 32, 50, 70])
def test_fill_cache_golden(T, clean_error_word):
    from b200attn import ops

    c = load_case(f"fill_cache_T{T}")
    kc = dev(c["cache"])
    vc = dev(c["cache"]).clone()
    ops.paged_fill_cache(kc, vc, dev(c["fill"]), dev(c["fill"]), dev(c["page_table"]),
                         dev(c["batch_idx"]))
    assert torch.equal(kc.cpu(), c["out"]) and torch.equal(vc.cpu(), c["out"])


# parametrisation of the reference's device test (tests/torch/ops/test_custom_ops.py:139-168),
# thinned to the supported head sizes / block sizes
@pytest.mark.parametrize("users", [8, 32])
@pytest.mark.parametrize("nblk", [16])
@pytest.mark.parametrize("nkv", [1, 8])
@pytest.mark.parametrize("bs", [32, 64])
@pytest.mark.parametrize("hd", [64, 128])
def test_update_cache_vs_oracle(users, nblk, nkv, bs, hd, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(users * 1000 + nkv * 10 + bs + hd)
    nb = users * nblk
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    pt = torch.randperm(nb, generator=g).reshape(users, nblk).int()
    pos = torch.randint(0, nblk * bs, (users,), generator=g).int()
    k = randn_bf16((1, users, nkv, hd), g)
    v = randn_bf16((1, users, nkv, hd), g)
    want_k = restate.paged_update_cache(kc, k, pos, pt)
    want_v = restate.paged_update_cache(vc, v, pos, pt)
    kcd, vcd = kc.cuda(), vc.cuda()
    ops.paged_update_cache(kcd, vcd, k.cuda(), v.cuda(), pos.cuda(), pt.cuda())
    assert torch.equal(kcd.cpu(), want_k) and torch.equal(vcd.cpu(), want_v)


@pytest.mark.parametrize("T", [1, 31, 64, 100, 512])
@pytest.mark.parametrize("users", [1, 3])
@pytest.mark.parametrize("bs,hd", [(32, 64), (64, 128)])
def test_fill_cache_vs_oracle(T, users, bs, hd, clean_error_word):
    from b200attn import ops

    g = torch.Generator().manual_seed(T * 7 + users)
    nkv = 4
    nblk = (T + bs - 1) // bs
    nb = users * nblk + 3
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    pt = torch.randperm(nb, generator=g)[: users * nblk].reshape(users, nblk).int()
    k = randn_bf16((users, T, nkv, hd), g)
    v = randn_bf16((users, T, nkv, hd), g)
    bidx = torch.arange(users, dtype=torch.int32).flip(0).contiguous()
    want_k = restate.paged_fill_cache(kc, k.transpose(1, 2), pt, bidx)
    want_v = restate.paged_fill_cache(vc, v.transpose(1, 2), pt, bidx)
    kcd, vcd = kc.cuda(), vc.cuda()
    ops.paged_fill_cache(kcd, vcd, k.cuda(), v.cuda(), pt.cuda(), bidx.cuda())
    assert torch.equal(kcd.cpu(), want_k) and torch.equal(vcd.cpu(), want_v)


def test_slot_mapping_equals_reference_addressing(clean_error_word):
    """slot = page_table[u, pos // bs] * bs + pos % bs addresses the same element as the
    (cache_position, page_table) form; negative slots are skipped."""
    from b200attn import ops

    g = torch.Generator().manual_seed(5)
    users, nblk, nkv, bs, hd = 16, 8, 8, 32, 64
    nb = users * nblk
    kc = randn_bf16((nb, nkv, bs, hd), g)
    vc = randn_bf16((nb, nkv, bs, hd), g)
    pt = torch.randperm(nb, generator=g).reshape(users, nblk).int()
    pos = torch.randint(0, nblk * bs, (users,), generator=g).int()
    k = randn_bf16((users, nkv, hd), g)
    v = randn_bf16((users, nkv, hd), g)
    slots = pt[torch.arange(users), (pos // bs).long()].long() * bs + (pos % bs).long()
    slots[3] = -1
    want_k = restate.paged_update_cache(kc, k[None], pos, pt)
    want_v = restate.paged_update_cache(vc, v[None], pos, pt)
    blk3 = int(pt[3, int(pos[3]) // bs])
    want_k[blk3, :, int(pos[3]) % bs] = kc[blk3, :, int(pos[3]) % bs]
    want_v[blk3, :, int(pos[3]) % bs] = vc[blk3, :, int(pos[3]) % bs]
    kcd, vcd = kc.cuda(), vc.cuda()
    ops.kv_scatter_slots(kcd, vcd, k.cuda(), v.cuda(), slots.cuda())
    assert torch.equal(kcd.cpu(), want_k) and torch.equal(vcd.cpu(), want_v)


def test_bad_page_id_is_reported_not_written():
    from b200attn import ops

    ops.read_error_word()
    kc = torch.zeros(4, 2, 32, 64, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    k = torch.ones(1, 2, 64, dtype=torch.bfloat16, device="cuda")
    pt = torch.tensor([[99]], dtype=torch.int32, device="cuda")
    ops.paged_update_cache(kc, vc, k, k, torch.zeros(1, dtype=torch.int32, device="cuda"), pt)
    assert ops.read_error_word() == 2
    assert kc.abs().sum().item() == 0
    assert ops.read_error_word() == 0


def test_full_size_prefill_scatter_roundtrip(clean_error_word):
    """Config-2 size (4 x 2048 tokens, nkv 8, hd 128, bs 64): scatter then gather back through
    the page table returns the inputs bit for bit; untouched blocks stay zero."""
    from b200attn import ops

    users, T, nkv, hd, bs = 4, 2048, 8, 128, 64
    nblk = T // bs
    nb = users * nblk + 1
    g = torch.Generator(device="cuda").manual_seed(0)
    k = torch.randn(users, T, nkv, hd, generator=g, device="cuda").bfloat16()
    v = torch.randn(users, T, nkv, hd, generator=g, device="cuda").bfloat16()
    pt = (torch.randperm(nb - 1)[: users * nblk] + 1).reshape(users, nblk).int().cuda()
    kc = torch.zeros(nb, nkv, bs, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.paged_fill_cache(kc, vc, k, v, pt, torch.arange(users, dtype=torch.int32, device="cuda"))
    back_k = kc[pt.long()].permute(0, 1, 3, 2, 4).reshape(users, T, nkv, hd)
    back_v = vc[pt.long()].permute(0, 1, 3, 2, 4).reshape(users, T, nkv, hd)
    assert torch.equal(back_k, k) and torch.equal(back_v, v)
    assert kc[0].abs().sum().item() == 0
