"""The decode step in one launch (`b200attn_paged_decode_step`): the cache write of
tt.paged_update_cache (custom_ops.py:962-1013) done by the decode kernel itself must leave the
caches bit-identical to the separate write and give bit-identical attention output."""
import pytest
import torch

from oracle import restate
from oracle.inputs import make_decode_case
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _run(case, fused, splits, window=0, fp8=False, wrap=True):
    from b200attn import ops

    u = case.users
    kc = (restate.quantize_kv_fp8(case.k_cache) if fp8 else case.k_cache).cuda()
    vc = (restate.quantize_kv_fp8(case.v_cache) if fp8 else case.v_cache).cuda()
    q = case.q.reshape(u, case.nq, case.hd).cuda()
    k = case.k.reshape(u, case.nkv, case.hd).cuda()
    v = case.v.reshape(u, case.nkv, case.hd).cuda()
    pt, pos = case.page_table.cuda(), case.cache_position.cuda()
    kw = dict(scale=case.scale, num_splits=splits, sliding_window=window)
    if fused:
        out = ops.paged_decode(q, kc, vc, pt, pos, new_key=k, new_value=v,
                               wrap_negative_positions=wrap, **kw)
    else:
        ops.paged_update_cache(kc, vc, k, v, pos, pt)
        out = ops.paged_decode(q, kc, vc, pt, pos, **kw)
    torch.cuda.synchronize()
    return out.cpu(), kc.cpu().view(torch.uint8 if fp8 else torch.int16), \
        vc.cpu().view(torch.uint8 if fp8 else torch.int16)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("bs", [32, 64])
def test_fused_step_equals_write_then_decode(fp8, splits, bs, clean_error_word):
    case = make_decode_case(nq=16, nkv=4, hd=128, bs=bs, users=9, ctx_lo=1, ctx_hi=700,
                            seed=bs + splits)
    # positions on tile and page edges: the new token opens a tile, closes one, is the first ever
    case.ctx_lens[:6] = torch.tensor([1, 64, 65, 128, 129, 640])
    # make the new token matter: without its row the output would change visibly
    case.k = case.k * 4
    a = _run(case, False, splits, fp8=fp8)
    b = _run(case, True, splits, fp8=fp8)
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]), "caches differ"
    assert torch.equal(a[0], b[0]), "attention output differs"
    if not fp8:
        ref, _, _ = restate.impl_forward(
            case.q, case.k, case.v, case.k_cache, case.v_cache, num_heads=case.nq,
            num_kv_heads=case.nkv, head_size=case.hd, scale=case.scale, num_users=case.users,
            cache_position=case.cache_position, page_table=case.page_table,
            compute_dtype=torch.float32)
        assert_attention_close(b[0].reshape(case.users, -1), ref, "fused step vs oracle")


def test_fused_step_head_size_64_and_window(clean_error_word):
    case = make_decode_case(nq=8, nkv=2, hd=64, bs=32, users=7, ctx_lo=1, ctx_hi=500, seed=5)
    for window in (0, 70):
        a = _run(case, False, 2, window)
        b = _run(case, True, 2, window)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])


def test_negative_positions_wrap_or_skip(clean_error_word):
    """Position -1 (a padded row): the reference's CPU indexing writes the row through the LAST
    page-table column at the block's last offset (custom_ops.py:985-998); the slot convention
    skips it.  Both are available; attention output of such rows is zeros either way."""
    case = make_decode_case(nq=8, nkv=2, hd=128, bs=64, users=4, ctx_lo=40, ctx_hi=300, seed=9)
    case.ctx_lens[2] = 0
    sep = _run(case, False, 1)
    wrap = _run(case, True, 1, wrap=True)
    assert torch.equal(sep[1], wrap[1]) and torch.equal(sep[2], wrap[2])
    assert torch.equal(sep[0], wrap[0]) and wrap[0][2].abs().sum() == 0
    skip = _run(case, True, 1, wrap=False)
    want_k, want_v = sep[1].clone(), sep[2].clone()
    blk = int(case.page_table[2, -1])
    want_k[blk, :, -1] = case.k_cache.view(torch.int16)[blk, :, -1]
    want_v[blk, :, -1] = case.v_cache.view(torch.int16)[blk, :, -1]
    assert torch.equal(skip[1], want_k) and torch.equal(skip[2], want_v)
    assert torch.equal(skip[0], sep[0])
