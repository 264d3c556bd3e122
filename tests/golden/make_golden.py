"""Generates the golden vectors under tests/golden/ by running the UNMODIFIED reference ops'
CPU branches (python_package/tt_torch/custom_ops.py) and the reference attention backend
(vllm_tt/attention_impls/attention.py) on small seeded inputs.

Run where the reference tree is mounted:   python tests/golden/make_golden.py
The vectors pin the oracle restatement (oracle/restate.py) and, through it and directly, the
CUDA kernels.  Shapes follow the parametrisations of the reference's own op tests
(tests/torch/ops/test_custom_ops.py:139-231, tests/torch/ops/test_chunked_sdpa_op_cpu.py),
scaled down so each file stays small.
"""
from __future__ import annotations

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import reference_loader as ref  # noqa: E402
from oracle.inputs import randn_bf16  # noqa: E402
from tests.golden.golden_io import save_case  # noqa: E402


def gen(seed):
    return torch.Generator().manual_seed(seed)


def case_update_cache():
    g = gen(11)
    nb, nkv, bs, hd, users, nblk = 9, 2, 32, 64, 4, 2
    cache_k = randn_bf16((nb, nkv, bs, hd), g)
    cache_v = randn_bf16((nb, nkv, bs, hd), g)
    page_table = torch.randperm(nb, generator=g)[: users * nblk].reshape(users, nblk).int()
    # one row per interesting position: block start, block end, mid, and a padded row (-1),
    # which the reference's indexing sends to the LAST page-table column at offset bs-1
    pos = torch.tensor([0, bs - 1, bs + 5, -1], dtype=torch.int32)  # columns 0, 0, 1, -1
    k = randn_bf16((1, users, nkv, hd), g)
    v = randn_bf16((1, users, nkv, hd), g)
    out_k = ref.ref_paged_update_cache(cache_k, k, pos, page_table)
    out_v = ref.ref_paged_update_cache(cache_v, v, pos, page_table)
    save_case("update_cache", dict(k_cache=cache_k, v_cache=cache_v, page_table=page_table,
                                   update_indices=pos, k=k, v=v, out_k=out_k, out_v=out_v))


def case_fill_cache():
    for T in (10, 32, 50, 70):
        g = gen(20 + T)
        nb, nkv, bs, hd, users = 10, 2, 32, 64, 2
        nblk = (T + bs - 1) // bs
        cache = randn_bf16((nb, nkv, bs, hd), g)
        page_table = torch.randperm(nb, generator=g)[: users * nblk].reshape(users, nblk).int()
        fill = randn_bf16((users, T, nkv, hd), g)            # token-major, as the plugin holds it
        batch_idx = torch.tensor([1, 0], dtype=torch.int32)  # non-identity on purpose
        out = ref.ref_paged_fill_cache(cache, fill.transpose(1, 2), page_table, batch_idx)
        save_case(f"fill_cache_T{T}", dict(cache=cache, page_table=page_table, fill=fill,
                                           batch_idx=batch_idx, out=out))


def _decode_inputs(seed, nq, nkv, hd, bs, users, nblk):
    g = gen(seed)
    nb = users * nblk + 2
    k_cache = randn_bf16((nb, nkv, bs, hd), g)
    v_cache = randn_bf16((nb, nkv, bs, hd), g)
    page_table = torch.randperm(nb, generator=g)[: users * nblk].reshape(users, nblk).int()
    pos = torch.randint(0, nblk * bs, (users,), generator=g).int()
    pos[0] = 0
    pos[-1] = nblk * bs - 1
    q = randn_bf16((1, users, nq, hd), g)
    return k_cache, v_cache, page_table, pos, q


def case_decode():
    # MHA: the reference op called directly (what tests/torch/ops/test_custom_ops.py:206-231 pins)
    k_cache, v_cache, pt, pos, q = _decode_inputs(31, 2, 2, 64, 32, 3, 3)
    scale = 64 ** -0.5
    o32 = ref.load_ops().paged_scaled_dot_product_attention_decode(
        q.float(), k_cache.float(), v_cache.float(), pt, is_causal=True, cur_pos_tensor=pos,
        scale=scale)
    o16 = ref.load_ops().paged_scaled_dot_product_attention_decode(
        q, k_cache, v_cache, pt, is_causal=True, cur_pos_tensor=pos, scale=scale)
    save_case("decode_mha", dict(k_cache=k_cache, v_cache=v_cache, page_table=pt, cur_pos=pos,
                                 q=q, scale=scale, out_fp32=o32, out_bf16=o16))
    # GQA (G=4) and hd128/bs64 (G=8): the reference op looped per KV-head group, cross-checked
    # against the MLA decode CPU branch, which does GQA natively
    for name, (seed, nq, nkv, hd, bs, users, nblk) in {
        "decode_gqa4_hd64": (32, 8, 2, 64, 32, 3, 4),
        "decode_gqa8_hd128": (33, 8, 1, 128, 64, 2, 3),
    }.items():
        k_cache, v_cache, pt, pos, q = _decode_inputs(seed, nq, nkv, hd, bs, users, nblk)
        scale = hd ** -0.5
        o32 = ref.ref_paged_decode(q.float(), k_cache.float(), v_cache.float(), pt, pos, scale)
        o16 = ref.ref_paged_decode(q, k_cache, v_cache, pt, pos, scale)
        om = ref.ref_paged_decode_mla_branch(q.float(), k_cache.float(), v_cache.float(), pt, pos, scale)
        assert (om - o32).abs().max() < 1e-5, "group loop and MLA branch disagree"
        save_case(name, dict(k_cache=k_cache, v_cache=v_cache, page_table=pt, cur_pos=pos, q=q,
                             scale=scale, out_fp32=o32, out_bf16=o16))


def case_sdpa():
    g = gen(41)
    B, nq, nkv, T, hd = 2, 4, 2, 64, 64
    q = randn_bf16((B, nq, T, hd), g)
    k = randn_bf16((B, nkv, T, hd), g)
    v = randn_bf16((B, nkv, T, hd), g)
    scale = hd ** -0.5
    o32 = ref.ref_sdpa(q.float(), k.float(), v.float(), scale)
    o16 = ref.ref_sdpa(q, k, v, scale)
    save_case("sdpa_gqa", dict(q=q, k=k, v=v, scale=scale, out_fp32=o32, out_bf16=o16))


def case_chunked():
    for start in (0, 64, 96):
        g = gen(50 + start)
        users, nq, nkv, hd, bs, T = 1, 8, 2, 64, 32, 64
        nblk = (start + T) // bs
        nb = users * nblk + 1
        k_cache = randn_bf16((nb, nkv, bs, hd), g)
        v_cache = randn_bf16((nb, nkv, bs, hd), g)
        pt = (torch.randperm(nb - 1, generator=g)[: users * nblk] + 1).reshape(users, nblk).int()
        q = randn_bf16((users, nq, T, hd), g)
        scale = hd ** -0.5
        o32 = ref.ref_chunked_sdpa(q.float(), k_cache.float(), v_cache.float(), pt, start, scale)
        o16 = ref.ref_chunked_sdpa(q, k_cache, v_cache, pt, start, scale)
        save_case(f"chunked_start{start}", dict(q=q, k_cache=k_cache, v_cache=v_cache,
                                                page_table=pt, chunk_start=start, scale=scale,
                                                out_fp32=o32, out_bf16=o16))


def case_impl_forward():
    """The reference TTAttentionBackendImpl.forward on CPU (its CPU branches end to end)."""
    att = ref.load_attention()
    # decode, MHA (the reference CPU decode branch is MHA-only), bf16 as the plugin runs it
    g = gen(61)
    nq = nkv = 2
    hd, bs, users, nblk = 64, 32, 4, 3
    nb = users * nblk + 1
    impl = att.TTAttentionBackendImpl(nq, hd, hd ** -0.5, nkv, None, None, "auto")
    k_cache = randn_bf16((nb, nkv, bs, hd), g)
    v_cache = randn_bf16((nb, nkv, bs, hd), g)
    pt = (torch.randperm(nb - 1, generator=g)[: users * nblk] + 1).reshape(users, nblk).int()
    pos = torch.tensor([0, 31, 32, 95], dtype=torch.int32)
    q = randn_bf16((users, nq * hd), g)
    k = randn_bf16((users, nkv * hd), g)
    v = randn_bf16((users, nkv * hd), g)
    md = att.TTMetadata(cache_position=pos, attn_mask=None, page_table=pt, is_causal=True,
                        batch_idx=torch.arange(users, dtype=torch.int32), num_users=users)
    kv = [k_cache.clone(), v_cache.clone()]
    out = torch.empty(users, nq * hd, dtype=torch.bfloat16)
    impl.forward(None, q, k, v, kv, md, output=out)
    save_case("impl_decode_mha", dict(k_cache=k_cache, v_cache=v_cache, page_table=pt,
                                      cache_position=pos, q=q, k=k, v=v, out_bf16=out,
                                      out_k=kv[0], out_v=kv[1], nq=nq, nkv=nkv))
    # prefill, GQA, one user (the reference CPU fill branch serves one user), first chunk
    g = gen(62)
    nq, nkv, T, users = 8, 2, 64, 1
    nblk = T // bs
    nb = nblk + 2
    impl = att.TTAttentionBackendImpl(nq, hd, hd ** -0.5, nkv, None, None, "auto")
    k_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
    v_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
    pt = (torch.randperm(nb - 1, generator=g)[:nblk] + 1).reshape(1, nblk).int()
    q = randn_bf16((T, nq * hd), g)
    k = randn_bf16((T, nkv * hd), g)
    v = randn_bf16((T, nkv * hd), g)
    md = att.TTMetadata(cache_position=torch.tensor([T - 1], dtype=torch.int32), attn_mask=None,
                        page_table=pt, is_causal=True, fill_page_table=pt,
                        batch_idx=torch.zeros(1, dtype=torch.int32), num_users=1)
    kv = [k_cache.clone(), v_cache.clone()]
    out = torch.empty(T, nq * hd, dtype=torch.bfloat16)
    impl.forward(None, q, k, v, kv, md, output=out)
    save_case("impl_prefill_gqa", dict(page_table=pt, q=q, k=k, v=v, out_bf16=out, out_k=kv[0],
                                       out_v=kv[1], nq=nq, nkv=nkv, nb=nb, bs=bs))
    # continuation chunk over a cached prefix of 64 tokens (chunk_start_idx set)
    g = gen(63)
    start = 64
    nblk = (start + T) // bs
    nb = nblk + 2
    k_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
    v_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
    pt = (torch.randperm(nb - 1, generator=g)[:nblk] + 1).reshape(1, nblk).int()
    pre = pt[0, : start // bs].long()
    k_cache[pre] = randn_bf16((pre.numel(), nkv, bs, hd), g)
    v_cache[pre] = randn_bf16((pre.numel(), nkv, bs, hd), g)
    q = randn_bf16((T, nq * hd), g)
    k = randn_bf16((T, nkv * hd), g)
    v = randn_bf16((T, nkv * hd), g)
    fpt = torch.roll(pt, -(start // bs), dims=1).contiguous()
    md = att.TTMetadata(cache_position=torch.tensor([start + T - 1], dtype=torch.int32),
                        attn_mask=None, page_table=pt, is_causal=True, fill_page_table=fpt,
                        chunk_start_idx=torch.tensor([start], dtype=torch.int32),
                        batch_idx=torch.zeros(1, dtype=torch.int32), num_users=1)
    kv = [k_cache.clone(), v_cache.clone()]
    out = torch.empty(T, nq * hd, dtype=torch.bfloat16)
    impl.forward(None, q, k, v, kv, md, output=out)
    save_case("impl_chunk_gqa", dict(k_cache=k_cache, v_cache=v_cache, page_table=pt,
                                     fill_page_table=fpt, chunk_start=start, q=q, k=k, v=v,
                                     out_bf16=out, out_k=kv[0], out_v=kv[1], nq=nq, nkv=nkv))


def case_rotary():
    for name, (hd, rot) in {"rotary_hd64": (64, 64), "rotary_hd128": (128, 128),
                            "rotary_hd64_partial32": (64, 32)}.items():
        g = gen(70 + hd + rot)
        tokens, nq, nkv = 6, 4, 2
        pos = torch.tensor([0, 1, 17, 1023, 4096, 8191], dtype=torch.int64)
        q = randn_bf16((tokens, nq * hd), g)
        k = randn_bf16((tokens, nkv * hd), g)
        qo, ko, inv_freq = ref.ref_rotary(pos, q, k, hd, rot)
        save_case(name, dict(positions=pos, q=q, k=k, inv_freq=inv_freq, head_size=hd,
                             rotary_dim=rot, out_q=qo, out_k=ko))


if __name__ == "__main__":
    if not ref.available():
        sys.exit("reference tree not mounted; nothing generated")
    case_update_cache()
    case_fill_cache()
    case_decode()
    case_sdpa()
    case_chunked()
    case_impl_forward()
    case_rotary()
    total = sum(os.path.getsize(os.path.join(os.path.dirname(__file__), f))
                for f in os.listdir(os.path.dirname(__file__)) if f.endswith(".npz"))
    print(f"golden vectors written, {total / 1024:.0f} KiB")
