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


def allocate_kv_caches(
    layer_names,
    num_blocks: int,
    num_kv_heads: int,
    block_size: int,
    head_size: int,
    *,
    dtype: torch.dtype = torch.bfloat16,
    device=None,
    tp_size: int = 1,
    shared_kv_layers=None,
) -> dict:
    """Per-layer paged caches the way the plugin's runner creates them
    (`initialize_kv_cache`, model_runner.py:4560-4630): for every attention layer a zeroed
    `[k_cache, v_cache]` pair of `B200AttentionBackend.get_kv_cache_shape`, separate tensors so a
    decode step never slices or concatenates.  Under tensor parallelism each rank allocates only
    its own KV heads — a dense `[num_blocks, num_kv_heads / tp_size, block_size, head_size]`
    tensor, the per-device shard of the reference's `(None, "model", None, None)` sharding
    (:4632-4656) — after the same divisibility check (:4590-4599).

    `layer_names`: names, or a layer count (names become "layers.<i>.attn").
    `shared_kv_layers`: {layer: target layer} for cross-layer KV sharing; such a layer gets the
    target's pair itself, not a copy (`maybe_setup_cross_layer_kv_sharing`).
    Returns {layer name: [k_cache, v_cache]} in layer order."""
    from .backend import B200AttentionBackend

    if isinstance(layer_names, int):
        layer_names = [f"layers.{i}.attn" for i in range(layer_names)]
    if tp_size > 1:
        assert num_kv_heads % tp_size == 0, (
            f"num_kv_heads {num_kv_heads} must be divisible by tp_size {tp_size} "
            "for correct KV-head sharding"
        )
    if not B200AttentionBackend.supports_head_size(head_size):
        raise ValueError(f"head_size {head_size} is not supported (64 or 128)")
    if not B200AttentionBackend.supports_block_size(block_size):
        raise ValueError(f"block_size {block_size} is not supported (32 or 64)")
    if dtype not in (torch.bfloat16, torch.float8_e4m3fn):
        raise ValueError("KV caches are bfloat16 or float8_e4m3fn")
    shared_kv_layers = dict(shared_kv_layers or {})
    shape = B200AttentionBackend.get_kv_cache_shape(
        num_blocks, block_size, num_kv_heads // max(tp_size, 1), head_size)
    caches: dict = {}
    for name in layer_names:
        if name in shared_kv_layers:
            continue
        caches[name] = [torch.zeros(shape, dtype=dtype, device=device),
                        torch.zeros(shape, dtype=dtype, device=device)]
    for name, target in shared_kv_layers.items():
        if target not in caches:
            raise ValueError(f"layer {name} shares the KV cache of unknown layer {target}")
        caches[name] = caches[target]
    return {name: caches[name] for name in layer_names}


def bind_kv_caches(layers: dict, caches: dict) -> None:
    """Hands every attention layer its cache pair (`bind_kv_cache`, model_runner.py:4626-4630):
    sets `layer.kv_cache` for each name present in both mappings."""
    for name, layer in layers.items():
        if name in caches:
            layer.kv_cache = caches[name]
