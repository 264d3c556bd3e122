"""KV-head sharding: host logic, and a world_size-2 gloo run where each rank attends over its own
heads and the gathered result equals the unsharded one (the oracle stands in for the kernels on
CPU; on GPUs the same partition feeds the CUDA ops)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from b200attn import sharding
from b200attn.sharding import ParallelismMode, kv_cache_shard_factor
from oracle import restate
from oracle.inputs import make_decode_case


# reference unit test parametrisation:
# tests/integrations/vllm_plugin/unit_tests/test_kv_cache_shard_factor.py
@pytest.mark.parametrize("mode,shape,expected", [
    (ParallelismMode.DISABLED, (1, 1), 1),
    (ParallelismMode.DATA_PARALLEL_ONLY, (2, 1), 1),
    (ParallelismMode.TENSOR_PARALLEL_ONLY_1D, (1, 2), 2),
    (ParallelismMode.TENSOR_PARALLEL_ONLY_1D, (1, 4), 4),
    (ParallelismMode.TENSOR_PARALLEL_ONLY_2D, (2, 4), 4),
    (ParallelismMode.DATA_TENSOR_PARALLEL, (4, 8), 8),
])
def test_kv_cache_shard_factor(mode, shape, expected):
    mesh = dict(zip(("batch", "model"), shape))
    assert kv_cache_shard_factor(mode, mesh) == expected
    assert kv_cache_shard_factor(mode, mesh, is_mla=True) == 1


def test_head_shard_ranges():
    parts = [sharding.head_shard(r, 4, 64, 8) for r in range(4)]
    assert [(p.kv_begin, p.kv_end) for p in parts] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert [(p.q_begin, p.q_end) for p in parts] == [(0, 16), (16, 32), (32, 48), (48, 64)]
    assert all(p.num_q_heads == 16 and p.num_kv_heads == 2 for p in parts)
    with pytest.raises(ValueError, match="divisible by TP size"):
        sharding.head_shard(0, 3, 32, 8)


def test_shard_and_gather_roundtrip():
    x = torch.arange(5 * 8 * 4, dtype=torch.float32).reshape(5, 32)
    parts = []
    for r in range(2):
        s = sharding.head_shard(r, 2, 8, 4)
        parts.append(sharding.shard_heads(x, s.q_begin, s.q_end, 8))
    assert torch.equal(sharding.gather_heads(parts, 4), x)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = make_decode_case(nq=8, nkv=4, hd=64, bs=32, users=3, ctx_lo=10, ctx_hi=150, seed=5)
        s = sharding.head_shard(rank, world, case.nq, case.nkv)
        kc = sharding.shard_cache(case.k_cache, s)
        vc = sharding.shard_cache(case.v_cache, s)
        q = sharding.shard_heads(case.q, s.q_begin, s.q_end, case.nq)
        k = sharding.shard_heads(case.k, s.kv_begin, s.kv_end, case.nkv)
        v = sharding.shard_heads(case.v, s.kv_begin, s.kv_end, case.nkv)
        out, kc2, vc2 = restate.impl_forward(
            q, k, v, kc, vc, num_heads=s.num_q_heads, num_kv_heads=s.num_kv_heads,
            head_size=case.hd, scale=case.scale, num_users=case.users,
            cache_position=case.cache_position, page_table=case.page_table,
            compute_dtype=torch.float32)
        outs = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(outs, out.contiguous())
        caches = [torch.empty_like(kc2.float()) for _ in range(world)]
        dist.all_gather(caches, kc2.float().contiguous())
        if rank == 0:
            full_out, full_k, _ = restate.impl_forward(
                case.q, case.k, case.v, case.k_cache, case.v_cache, num_heads=case.nq,
                num_kv_heads=case.nkv, head_size=case.hd, scale=case.scale, num_users=case.users,
                cache_position=case.cache_position, page_table=case.page_table,
                compute_dtype=torch.float32)
            got = sharding.gather_heads(outs, case.hd)
            ok_out = torch.allclose(got, full_out, atol=1e-5, rtol=1e-5)
            ok_cache = torch.equal(torch.cat(caches, dim=1), full_k.float())
            with open(os.path.join(out_dir, "result"), "w") as f:
                f.write(f"{int(ok_out)}{int(ok_cache)}")
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharded_forward_equals_unsharded(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "result").read_text() == "11"
