"""Seeded synthetic inputs for the benchmark configurations and the parity tests.
TEST / BENCHMARK INFRASTRUCTURE — no dataset stands behind these; every tensor is drawn from a
seeded CPU generator as fp32 and then cast to bf16 (a native bf16 `randn` on CPU has a coarser
grid and a visible share of exact zeros).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


def randn_bf16(shape, gen: torch.Generator) -> torch.Tensor:
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(torch.bfloat16)


@dataclass
class DecodeCase:
    """One paged decode step in the plugin's form."""

    nq: int
    nkv: int
    hd: int
    bs: int
    nb: int
    ctx_lens: torch.Tensor          # [users] context length INCLUDING the new token
    page_table: torch.Tensor        # [users, nblk] i32
    k_cache: torch.Tensor           # [nb, nkv, bs, hd] bf16 (before the write)
    v_cache: torch.Tensor
    q: torch.Tensor                 # [users, nq*hd]
    k: torch.Tensor                 # [users, nkv*hd]
    v: torch.Tensor
    scale: float
    extra: dict = field(default_factory=dict)

    @property
    def users(self) -> int:
        return self.ctx_lens.numel()

    @property
    def cache_position(self) -> torch.Tensor:
        return (self.ctx_lens - 1).to(torch.int32)

    def kv_bytes(self) -> int:
        """Algorithmic bytes of the decode attention: K and V rows of every context read once,
        q read and o written, page-table entries and positions read."""
        s = 2
        kv = int(self.ctx_lens.sum()) * 2 * self.nkv * self.hd * s
        qo = 2 * self.users * self.nq * self.hd * s
        meta = int(((self.ctx_lens + self.bs - 1) // self.bs).sum()) * 4 + 4 * self.users
        return kv + qo + meta


def make_decode_case(
    *, nq: int, nkv: int, hd: int, bs: int, users: int, ctx_lo: int, ctx_hi: int,
    nb: Optional[int] = None, seed: int = 0, fill_cache: bool = True,
) -> DecodeCase:
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(ctx_lo, ctx_hi + 1, (users,), generator=g)
    nblk = (ctx_hi + bs - 1) // bs
    need = users * nblk
    nb = nb if nb is not None else need + 1
    assert nb >= need, "pool too small for the page table"
    page_table = torch.randperm(nb, generator=g)[:need].reshape(users, nblk).to(torch.int32)
    if fill_cache:
        k_cache = randn_bf16((nb, nkv, bs, hd), g)
        v_cache = randn_bf16((nb, nkv, bs, hd), g)
    else:
        k_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
        v_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
    return DecodeCase(
        nq=nq, nkv=nkv, hd=hd, bs=bs, nb=nb, ctx_lens=ctx, page_table=page_table,
        k_cache=k_cache, v_cache=v_cache,
        q=randn_bf16((users, nq * hd), g), k=randn_bf16((users, nkv * hd), g),
        v=randn_bf16((users, nkv * hd), g), scale=hd ** -0.5,
    )


def config1(seed: int = 1) -> DecodeCase:
    """Llama-3.2-1B GQA decode: nq 32, nkv 8, hd 64, batch 8, contexts U[128,1024], block 32,
    pool of 512 blocks, page table = a seeded permutation of the pool."""
    return make_decode_case(nq=32, nkv=8, hd=64, bs=32, users=8, ctx_lo=128, ctx_hi=1024,
                            nb=512, seed=seed)


@dataclass
class PrefillCase:
    """Prefill / chunked prefill in the plugin's [users x T] form."""

    nq: int
    nkv: int
    hd: int
    bs: int
    nb: int
    users: int
    T: int
    chunk_start: int                # tokens already in the cache (0 = first chunk)
    page_table: torch.Tensor        # [users, nblk] i32 covering prefix + chunk
    fill_page_table: torch.Tensor   # page_table rolled left by chunk_start // bs
    k_cache: torch.Tensor           # holds the prefix
    v_cache: torch.Tensor
    q: torch.Tensor                 # [users*T, nq*hd]
    k: torch.Tensor                 # [users*T, nkv*hd]
    v: torch.Tensor
    scale: float

    def flops(self) -> int:
        """4*hd*nq per attended (query, key) pair; masked pairs are not counted."""
        pairs = self.users * (self.T * self.chunk_start + self.T * (self.T + 1) // 2)
        return 4 * self.hd * self.nq * pairs


def make_prefill_case(
    *, nq: int, nkv: int, hd: int, bs: int, users: int, T: int, chunk_start: int = 0,
    seed: int = 0,
) -> PrefillCase:
    assert chunk_start % bs == 0, "chunks start on a block boundary (scheduler invariant)"
    g = torch.Generator().manual_seed(seed)
    nblk = (chunk_start + T + bs - 1) // bs
    nb = users * nblk + 1
    # block 0 stays unused, like the null block of the runner
    page_table = (torch.randperm(nb - 1, generator=g)[: users * nblk] + 1).reshape(users, nblk)
    page_table = page_table.to(torch.int32)
    k_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
    v_cache = torch.zeros((nb, nkv, bs, hd), dtype=torch.bfloat16)
    pre_blocks = chunk_start // bs
    if pre_blocks:
        ids = page_table[:, :pre_blocks].reshape(-1).long()
        k_cache[ids] = randn_bf16((ids.numel(), nkv, bs, hd), g)
        v_cache[ids] = randn_bf16((ids.numel(), nkv, bs, hd), g)
    fill_page_table = torch.roll(page_table, -pre_blocks, dims=1).contiguous()
    return PrefillCase(
        nq=nq, nkv=nkv, hd=hd, bs=bs, nb=nb, users=users, T=T, chunk_start=chunk_start,
        page_table=page_table, fill_page_table=fill_page_table, k_cache=k_cache, v_cache=v_cache,
        q=randn_bf16((users * T, nq * hd), g), k=randn_bf16((users * T, nkv * hd), g),
        v=randn_bf16((users * T, nkv * hd), g), scale=hd ** -0.5,
    )


def config2(seed: int = 2) -> PrefillCase:
    """Llama-3.1-8B causal prefill: nq 32, nkv 8, hd 128, 4 x 2048 tokens, block 64."""
    return make_prefill_case(nq=32, nkv=8, hd=128, bs=64, users=4, T=2048, seed=seed)
