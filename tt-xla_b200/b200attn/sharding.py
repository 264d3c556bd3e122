"""KV-head partitioning of the attention path across tensor-parallel ranks.

The reference shards the KV cache on its "model" mesh axis, heads only
(`safe_mark_sharding(cache, mesh, (None, "model", None, None))`, model_runner.py:4632-4656, after
asserting `num_kv_heads % tp == 0`, :4590-4599), column-splits q/k/v projections per head group
and row-splits o_proj (vllm_distributed_utils.py:228-363).  Here that becomes explicit per-rank
tensors: rank r holds KV heads [r*nkv/g, (r+1)*nkv/g) of every block as a DENSE cache, the
matching query heads, and a replica of the int32 metadata.  Attention needs no exchange.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import torch


class ParallelismMode(Enum):
    """vllm_distributed_utils.py:98-103."""

    DISABLED = "disabled"
    DATA_PARALLEL_ONLY = "data_parallel_only"
    TENSOR_PARALLEL_ONLY_1D = "tensor_parallel_only_1D"
    TENSOR_PARALLEL_ONLY_2D = "tensor_parallel_only_2d"
    DATA_TENSOR_PARALLEL = "data_tensor_parallel"


def kv_cache_shard_factor(parallel_mode: ParallelismMode, mesh_shape: dict, is_mla: bool = False) -> int:
    """How many ways the KV cache is sharded (vllm_distributed_utils.py:106-134): the size of the
    "model" axis under any tensor-parallel mode, 1 otherwise and for MLA's replicated latent
    cache.  `mesh_shape` maps axis name -> size."""
    if parallel_mode in (ParallelismMode.DISABLED, ParallelismMode.DATA_PARALLEL_ONLY):
        return 1
    if is_mla:
        return 1
    return int(mesh_shape["model"])


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    q_begin: int
    q_end: int
    kv_begin: int
    kv_end: int

    @property
    def num_q_heads(self) -> int:
        return self.q_end - self.q_begin

    @property
    def num_kv_heads(self) -> int:
        return self.kv_end - self.kv_begin


def head_shard(rank: int, world: int, num_q_heads: int, num_kv_heads: int) -> HeadShard:
    """Rank r's contiguous head ranges.  KV heads must divide evenly (the reference asserts the
    same, model_runner.py:4594-4599); query heads follow their KV head."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if num_kv_heads % world != 0:
        raise ValueError(
            f"Number of KV heads ({num_kv_heads}) must be divisible by TP size ({world})"
        )
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be a multiple of num_kv_heads")
    kv_per = num_kv_heads // world
    group = num_q_heads // num_kv_heads
    return HeadShard(rank, world, rank * kv_per * group, (rank + 1) * kv_per * group,
                     rank * kv_per, (rank + 1) * kv_per)


def shard_cache(cache: torch.Tensor, shard: HeadShard) -> torch.Tensor:
    """[nb, nkv, bs, hd] -> this rank's dense [nb, nkv/g, bs, hd]."""
    return cache[:, shard.kv_begin:shard.kv_end].contiguous()


def shard_heads(x: torch.Tensor, begin: int, end: int, num_heads: int) -> torch.Tensor:
    """[tokens, num_heads*hd] (or [tokens, num_heads, hd]) -> the columns of heads [begin, end)."""
    tokens = x.shape[0]
    x3 = x.reshape(tokens, num_heads, -1)
    return x3[:, begin:end].reshape(tokens, -1).contiguous()


def gather_heads(parts: list[torch.Tensor], head_size: int) -> torch.Tensor:
    """Concatenates per-rank outputs [tokens, nq/g*hd] back into [tokens, nq*hd] (rank order)."""
    tokens = parts[0].shape[0]
    return torch.cat([p.reshape(tokens, -1, head_size) for p in parts], dim=1).reshape(tokens, -1)
