"""The allocation-free decode entry point, called through the C ABI.

Some hosts of this library cannot call cudaMalloc around a decode step: a serving loop whose
memory pool is frozen, a process in which another component owns all device memory, a latency
path that must not take the allocator lock.  b200attn_paged_decode_static serves them with
scratch that lives inside the library image.  This test calls it with raw pointers only and
checks that it returns what the ordinary entry point returns, twice in a row (the second call
sees the first call's leftovers in the shared scratch).  The file name keeps it last in
collection order.
"""
import pytest
import torch

from oracle.inputs import make_decode_case
from tests.conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def _call(fn_name, case, out, splits, workspace=None):
    from b200attn import _lib

    L = _lib.lib()
    users = case["q"].shape[0]
    nq, hd = case["q"].shape[1], case["q"].shape[2]
    nb, nkv, bs, _ = case["k_cache"].shape
    stream = torch.cuda.current_stream().cuda_stream
    common = (out.data_ptr(), nq * hd, case["q"].data_ptr(), nq * hd, case["k_cache"].data_ptr(),
              case["v_cache"].data_ptr(), case["pt"].data_ptr(), case["pt"].stride(0),
              case["pt"].shape[1], case["pos"].data_ptr(), users, nq, nkv, hd, bs, nb,
              float(hd ** -0.5), 0, splits)
    if fn_name == "b200attn_paged_decode_static":
        return L.b200attn_paged_decode_static(*common, stream)
    return L.b200attn_paged_decode(*common, workspace.data_ptr(), workspace.numel(), stream)


def _device_case(seed, users, ctx_hi):
    c = make_decode_case(nq=32, nkv=8, hd=128, bs=64, users=users, ctx_lo=1, ctx_hi=ctx_hi,
                         seed=seed)
    return dict(q=c.q.reshape(users, c.nq, c.hd).cuda(), k_cache=c.k_cache.cuda(),
                v_cache=c.v_cache.cuda(), pt=c.page_table.cuda(), pos=c.cache_position.cuda())


def test_static_entry_point_matches_the_allocating_one_twice_in_a_row():
    from b200attn import _lib, ops

    L = _lib.lib()
    ops.read_error_word()
    # everything the calls need exists before the first call: the entry point itself must not
    # have to allocate
    cases = [_device_case(101, 6, 900), _device_case(202, 9, 2500)]
    outs_static = [torch.zeros_like(c["q"]) for c in cases]
    outs_plain = [torch.zeros_like(c["q"]) for c in cases]
    workspace = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")   # counters start at zero
    torch.cuda.synchronize()
    for c, o_s, o_p, splits in zip(cases, outs_static, outs_plain, (4, 7)):
        before = torch.cuda.memory_allocated()
        assert _call("b200attn_paged_decode_static", c, o_s, splits) == 0
        assert torch.cuda.memory_allocated() == before
        assert _call("b200attn_paged_decode", c, o_p, splits, workspace) == 0
        torch.cuda.synchronize()
        assert_attention_close(o_s, o_p.float(), "static vs allocating entry point")
        assert torch.equal(o_s, o_p), "same kernels, same split count: identical bits expected"
    assert ops.read_error_word() == 0
    # automatic split count also goes through
    o = torch.zeros_like(cases[0]["q"])
    assert _call("b200attn_paged_decode_static", cases[0], o, 0) == 0
    torch.cuda.synchronize()
    assert_attention_close(o, outs_plain[0].float(), "auto splits")


def test_static_entry_point_rejects_scratch_beyond_its_array():
    from b200attn import _lib

    L = _lib.lib()
    c = _device_case(303, 64, 64)
    out = torch.zeros_like(c["q"])
    # 64 users x 32 heads x 128 splits x (128*4 + 8) bytes is far beyond 16 MiB
    assert L.b200attn_decode_workspace_bytes(64, 32, 128, 128) > (16 << 20)
    rc = _call("b200attn_paged_decode_static", c, out, 128)
    assert rc == -8
    assert b"maximum" in L.b200attn_status_string(rc)
