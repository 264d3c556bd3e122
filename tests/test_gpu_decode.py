"""Paged GQA decode kernel against the oracle / reference golden vectors (bf16 tolerance:
max abs <= 2e-2, mean abs <= 2e-3 against fp32 arithmetic)."""
import pytest
import torch

from oracle import restate
from oracle.inputs import config1, make_decode_case
from tests.conftest import assert_attention_close
from tests.golden.golden_io import load_case

pytestmark = pytest.mark.gpu


def run_decode(case, num_splits=0):
    from b200attn import ops

    users = case.users
    out = ops.paged_decode(
        case.q.reshape(users, case.nq, case.hd).cuda(), case.k_cache.cuda(), case.v_cache.cuda(),
        case.page_table.cuda(), case.cache_position.cuda(), scale=case.scale,
        num_splits=num_splits,
    )
    return out.cpu()


def oracle_decode(case):
    users = case.users
    return restate.paged_sdpa_decode(
        case.q.reshape(1, users, case.nq, case.hd).float(), case.k_cache.float(),
        case.v_cache.float(), case.page_table, case.cache_position, case.scale,
    )[0]


@pytest.mark.parametrize("name", ["decode_mha", "decode_gqa4_hd64", "decode_gqa8_hd128"])
def test_decode_golden(name, clean_error_word):
    from b200attn import ops

    c = load_case(name)
    out = ops.paged_decode(c["q"].cuda(), c["k_cache"].cuda(), c["v_cache"].cuda(),
                           c["page_table"].cuda(), c["cur_pos"].cuda(), scale=float(c["scale"]))
    assert out.shape == c["q"].shape
    assert_attention_close(out, c["out_fp32"], name)


@pytest.mark.parametrize("splits", [0, 1, 2, 3, 7])
def test_config1_all_split_counts(splits, clean_error_word):
    """benchmark config 1: nq 32 / nkv 8 / hd 64 / bs 32, 8 users, contexts U[128,1024]."""
    case = config1()
    assert_attention_close(run_decode(case, splits), oracle_decode(case), f"splits={splits}")


@pytest.mark.parametrize("nq,nkv,hd,bs", [(8, 8, 64, 32), (32, 8, 128, 64), (64, 8, 128, 64),
                                          (16, 1, 128, 32), (4, 2, 64, 64)])
def test_decode_geometries(nq, nkv, hd, bs, clean_error_word):
    case = make_decode_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=5, ctx_lo=1, ctx_hi=700,
                            seed=nq + hd + bs)
    assert_attention_close(run_decode(case), oracle_decode(case), f"{nq}/{nkv}/{hd}/{bs}")


@pytest.mark.parametrize("bs,hd", [(32, 64), (64, 128)])
def test_every_context_length_in_three_tiles(bs, hd, clean_error_word):
    """Every context length 1..192 (three 64-token tiles): catches tail masking and page
    boundary mistakes."""
    users = 192
    case = make_decode_case(nq=8, nkv=2, hd=hd, bs=bs, users=users, ctx_lo=192, ctx_hi=192, seed=3)
    case.ctx_lens = torch.arange(1, users + 1)
    for splits in (1, 2):
        assert_attention_close(run_decode(case, splits), oracle_decode(case), f"splits={splits}")


def test_padded_rows_yield_zeros_and_do_not_disturb_others(clean_error_word):
    case = make_decode_case(nq=8, nkv=2, hd=64, bs=32, users=4, ctx_lo=40, ctx_hi=200, seed=9)
    ref = oracle_decode(case)
    case.ctx_lens[2] = 0          # cache_position = -1: padding row
    out = run_decode(case, 2)
    assert out[2].abs().sum().item() == 0
    keep = [0, 1, 3]
    assert_attention_close(out[keep], ref[keep], "padded batch")


def test_stale_non_finite_cache_tail_is_ignored(clean_error_word):
    """Slots past the context hold garbage in a live cache; NaN / Inf there must not leak."""
    case = make_decode_case(nq=8, nkv=2, hd=128, bs=64, users=3, ctx_lo=70, ctx_hi=100, seed=4)
    ref = oracle_decode(case)
    for u in range(case.users):
        L = int(case.ctx_lens[u])
        blk = int(case.page_table[u, L // case.bs])
        case.k_cache[blk, :, L % case.bs:] = float("nan")
        case.v_cache[blk, :, L % case.bs:] = float("inf")
    assert_attention_close(run_decode(case, 1), ref, "nan tail")


def test_decode_is_deterministic(clean_error_word):
    case = config1(seed=12)
    a = run_decode(case, 4)
    b = run_decode(case, 4)
    assert torch.equal(a, b)


def test_long_context_property(clean_error_word):
    """Config-4 shape (nq 64, nkv 8, hd 128, bs 64) at 32768 context: V rows all equal to one
    vector => the output equals that vector whatever the scores (softmax weights sum to 1).  A
    property of the normalisation only; the comparison with the oracle at this size is in
    test_gpu_baseline_sizes.py."""
    from b200attn import ops

    users, nq, nkv, hd, bs, ctx = 2, 64, 8, 128, 64, 32768
    nblk = ctx // bs
    nb = users * nblk
    g = torch.Generator(device="cuda").manual_seed(0)
    kc = torch.randn(nb, nkv, bs, hd, generator=g, device="cuda").bfloat16()
    vec = torch.randn(nkv, 1, hd, generator=g, device="cuda").bfloat16()
    vc = vec.expand(nkv, bs, hd).unsqueeze(0).expand(nb, nkv, bs, hd).contiguous()
    q = torch.randn(users, nq, hd, generator=g, device="cuda").bfloat16()
    pt = torch.randperm(nb).reshape(users, nblk).int().cuda()
    pos = torch.full((users,), ctx - 1, dtype=torch.int32, device="cuda")
    out = ops.paged_decode(q, kc, vc, pt, pos, scale=hd ** -0.5)
    want = vec[:, 0].repeat_interleave(nq // nkv, 0).float()       # [nq, hd]
    assert (out.float() - want[None]).abs().max().item() <= 2e-2


def test_split_merge_inside_the_launch_leaves_the_workspace_reusable(clean_error_word):
    """The last split to arrive merges the partials and resets its arrival counter: the same
    workspace serves calls of different shapes back to back, results bit-identical to a fresh
    zeroed workspace."""
    from b200attn import ops

    ws = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    for seed, (users, nq, nkv, hd, bs, splits) in enumerate(
            [(5, 32, 8, 128, 64, 4), (9, 8, 2, 64, 32, 3), (5, 32, 8, 128, 64, 7), (2, 16, 1, 128, 32, 16)]):
        case = make_decode_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=users, ctx_lo=1, ctx_hi=900,
                                seed=seed)
        args = (case.q.reshape(users, nq, hd).cuda(), case.k_cache.cuda(), case.v_cache.cuda(),
                case.page_table.cuda(), case.cache_position.cuda())
        shared = ops.paged_decode(*args, scale=case.scale, num_splits=splits, workspace=ws)
        fresh = ops.paged_decode(*args, scale=case.scale, num_splits=splits,
                                 workspace=torch.zeros_like(ws))
        assert torch.equal(shared, fresh)
        assert_attention_close(shared.cpu(), oracle_decode(case), f"case {seed}")
        assert int(ws[:65536].view(torch.int32).abs().sum()) == 0     # counters back at zero


def test_batches_beyond_the_ticket_region_use_the_separate_merge(clean_error_word):
    """More (user, KV head) pairs than arrival counters: the partials are merged by the second
    launch, same results."""
    users, nq, nkv, hd, bs = 4100, 4, 4, 64, 32
    case = make_decode_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=users, ctx_lo=1, ctx_hi=96, seed=21)
    assert users * nkv * 4 > 65536
    out = run_decode(case, 2)
    pick = torch.arange(0, users, 37)
    sub = make_decode_case(nq=nq, nkv=nkv, hd=hd, bs=bs, users=users, ctx_lo=1, ctx_hi=96, seed=21)
    want = restate.paged_sdpa_decode(
        case.q.reshape(1, users, nq, hd)[:, pick].float(), sub.k_cache.float(), sub.v_cache.float(),
        case.page_table[pick], case.cache_position[pick], case.scale)[0]
    assert_attention_close(out[pick], want, "beyond the ticket region")
    assert_attention_close(run_decode(case, 1)[pick], want, "single split, same batch")
