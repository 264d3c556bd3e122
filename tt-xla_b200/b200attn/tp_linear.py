"""Row-parallel linear layers with the tensor-parallel all-reduce fused into the GEMM epilogue.

The reference shards o_proj / down_proj along the input dimension and lets the compiler insert
the all-reduce of the partial sums (vllm_tt/vllm_distributed_utils.py:356-363,
`partition_row_parallel_linear`); vLLM's own RowParallelLinear runs a GEMM and then
`tensor_model_parallel_all_reduce`.  Here `partition_row_parallel_linear(layer, comm)` points the
layer's forward at one CUDA launch per rank that does both for decode-sized batches
(<= 128 token rows); larger batches keep the layer's original forward.

`RowLinearComm` owns the per-rank communicator buffer (staging for the peers' fp32 partials, one
flag per source rank and tile, an epoch word) and the mappings of the peers' buffers; the handles
travel over a `torch.distributed` group once, at construction.  There is no CPU path.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _lib
from ._lib import check as _check
from .ops import _need_cuda, _stream

MAX_TOKENS = 128          # token rows one launch can take
STAGE_OFFSET = 32768      # staging areas [parity][source rank] start here; epoch / ticket words at 0
TILE_N = 128              # output columns per cluster


def comm_bytes(world: int, max_tokens: int, max_n: int) -> int:
    n = _lib.lib().b200attn_comm_bytes(world, max_tokens, max_n)
    if n == 0:
        raise ValueError(
            f"unsupported communicator geometry world={world} max_tokens={max_tokens} max_n={max_n}"
        )
    return n


def plan(num_tokens: int, n: int, k_local: int) -> tuple[int, int]:
    """(token rows of the MMA, K splits) the launch uses on the current device."""
    rows, splits = ctypes.c_int(0), ctypes.c_int(0)
    _check("b200attn_rowlinear_plan",
           _lib.lib().b200attn_rowlinear_plan(num_tokens, n, k_local, ctypes.byref(rows),
                                              ctypes.byref(splits)))
    return rows.value, splits.value


def area_bytes(max_tokens: int, max_n: int) -> int:
    """Bytes of one staging area (per parity: one area per source rank, then one for two-shot
    results): 8-byte units {bf16 pair, epoch} laid out
    [tile * splits + share][pair of the share][column of the tile]."""
    rows = 32 if max_tokens <= 32 else (64 if max_tokens <= 64 else 128)
    return ((max_n + TILE_N - 1) // TILE_N) * rows * (TILE_N * 8 // 2)


class RowLinearComm:
    """Communicator of one tensor-parallel group for `rowlinear_allreduce`.

    `group` is a torch.distributed process group whose ranks each drive one GPU of one node
    (any backend: it only carries 64 handle bytes per rank, once).  `max_n` bounds the output
    width, `max_tokens` the token rows.  Collective: every rank of the group constructs it at the
    same point.  With `buffers` (one device uint8 tensor per rank, all in this process) no handles
    are exchanged; that form exists for single-process tests."""

    def __init__(self, group=None, *, max_n: int, max_tokens: int = MAX_TOKENS,
                 device: Optional[torch.device] = None, rank: Optional[int] = None,
                 buffers: Optional[List[torch.Tensor]] = None):
        L = _lib.lib()
        self.max_n, self.max_tokens = int(max_n), int(max_tokens)
        self._own_ptr = None
        self._imported: List[int] = []
        self._keepalive = buffers
        if buffers is not None:
            self.world = len(buffers)
            self.rank = int(rank)
            self.nbytes = comm_bytes(self.world, self.max_tokens, self.max_n)
            for b in buffers:
                _need_cuda(b)
                if b.dtype != torch.uint8 or b.numel() < self.nbytes:
                    raise ValueError("communicator buffers must be uint8 tensors of comm_bytes()")
            ptrs = [b.data_ptr() for b in buffers]
        else:
            import torch.distributed as dist

            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
            self.nbytes = comm_bytes(self.world, self.max_tokens, self.max_n)
            dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
            with torch.cuda.device(dev):
                own = ctypes.c_void_p()
                _check("b200attn_comm_alloc", L.b200attn_comm_alloc(self.nbytes, ctypes.byref(own)))
                self._own_ptr = own.value
                handle = (ctypes.c_ubyte * 64)()
                _check("b200attn_comm_export", L.b200attn_comm_export(own, handle))
                handles: List[Optional[bytes]] = [None] * self.world
                dist.all_gather_object(handles, bytes(handle), group=group)
                ptrs = []
                for r, h in enumerate(handles):
                    if r == self.rank:
                        ptrs.append(self._own_ptr)
                        continue
                    peer = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    _check("b200attn_comm_import", L.b200attn_comm_import(buf, ctypes.byref(peer)))
                    self._imported.append(peer.value)
                    ptrs.append(peer.value)
                # nobody may push before every rank has mapped every buffer
                dist.barrier(group=group)
        self._ptr_array = (ctypes.c_void_p * self.world)(*ptrs)

    def close(self) -> None:
        """Unmaps the peers' buffers and frees the own one (collective in spirit: no rank may
        still be inside a call)."""
        L = _lib.lib()
        for p in self._imported:
            L.b200attn_comm_close(ctypes.c_void_p(p))
        self._imported = []
        if self._own_ptr is not None:
            L.b200attn_comm_free(ctypes.c_void_p(self._own_ptr))
            self._own_ptr = None


def rowlinear_allreduce(
    x: torch.Tensor,
    weight: torch.Tensor,
    comm: Optional[RowLinearComm],
    out: Optional[torch.Tensor] = None,
    peer_timeout_s: float = 0.0,
    reduce_mode: int = 0,
) -> torch.Tensor:
    """out[t, n] = sum over ranks of bf16(x_r[t, :] @ weight_r[n, :]), x_r [tokens <= 128, K/world]
    bf16, weight_r [N, K/world] bf16 (this rank's slices); every rank of `comm` calls it with its
    own slices and gets the same bf16 [tokens, N] (fp32 accumulation inside each product and
    across ranks).  `comm=None` is the single-rank GEMM.  `reduce_mode`: 0 automatic, 1 one
    shot, 2 two shots (see include/b200attn.h)."""
    _need_cuda(x, weight)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise ValueError(f"x [tokens, K] and weight [N, K] expected, got {tuple(x.shape)} and "
                         f"{tuple(weight.shape)}")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise ValueError("only bfloat16 is supported")
    if x.stride(1) != 1 or weight.stride(1) != 1:
        raise ValueError("x and weight must be dense along K")
    tokens, k = x.shape
    n = weight.shape[0]
    if out is None:
        out = torch.empty(tokens, n, dtype=torch.bfloat16, device=x.device)
    elif out.shape != (tokens, n) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("out must be a bf16 [tokens, N] tensor dense along N")
    L = _lib.lib()
    world = comm.world if comm is not None else 1
    _check(
        "b200attn_rowlinear_allreduce",
        L.b200attn_rowlinear_allreduce(
            out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), weight.data_ptr(),
            weight.stride(0), tokens, n, k, comm.rank if comm is not None else 0, world,
            comm._ptr_array if comm is not None else None,
            comm.max_tokens if comm is not None else 0, comm.max_n if comm is not None else 0,
            int(reduce_mode), int(peer_timeout_s * 1e9), _stream(x),
        ),
    )
    return out


def partition_row_parallel_linear(layer: torch.nn.Module, comm: RowLinearComm) -> torch.nn.Module:
    """Mirror of vllm_distributed_utils.py:356-363 for a vLLM RowParallelLinear whose weight is
    already this rank's [N, K/world] slice: batches of up to `comm.max_tokens` rows take the fused
    launch, anything else (larger batches, bias, quantised weights, no reduction wanted) the
    layer's own forward.  Returns the layer."""
    original = layer.forward

    def forward(input_):
        w = getattr(layer, "weight", None)
        fused = (
            w is not None and w.dtype == torch.bfloat16 and input_.dtype == torch.bfloat16
            and getattr(layer, "reduce_results", True) and getattr(layer, "input_is_parallel", True)
            and getattr(layer, "bias", None) is None
            and input_.dim() == 2 and 0 < input_.shape[0] <= comm.max_tokens
            and w.shape[0] <= comm.max_n and input_.stride(1) == 1
        )
        if not fused:
            return original(input_)
        out = rowlinear_allreduce(input_, w, comm)
        if not getattr(layer, "return_bias", True):
            return out
        return out, None

    layer.forward = forward
    return layer
