"""vLLM registration of the B200 attention backend.

The reference plugin registers its backend as `AttentionBackendEnum.CUSTOM` at import
(integrations/vllm_plugin/vllm_tt/__init__.py:10-17) and is discovered through the
`vllm.platform_plugins` / `vllm.general_plugins` entry points of its setup.py (:58-61).  Here
`register()` is the `vllm.general_plugins` entry point (see the `b200attn-*.dist-info` directory
next to this package): vLLM calls it in every process it starts, so engine core and
tensor-parallel workers all know the backend.  Select it with `attention_backend="CUSTOM"` and a
KV block size of 32 or 64.

The classes below only adapt `b200attn.backend` to vLLM's abstract base classes; the attention
math, the cache layout and the metadata derivation live there.
"""
from __future__ import annotations

import logging
import os

import torch

from vllm.v1.attention.backend import (AttentionBackend, AttentionCGSupport, AttentionImpl,
                                       AttentionMetadataBuilder, AttentionType)

from . import backend as _b

logger = logging.getLogger("b200attn")


class B200VllmMetadataBuilder(AttentionMetadataBuilder[_b.B200Metadata]):
    """CommonAttentionMetadata -> B200Metadata, once per step; decode rows are ordered first."""

    reorder_batch_threshold = 1
    # A pure decode step launches the same three kernels on persistent buffers (slot_mapping,
    # block table, positions), so it can be captured and replayed as one CUDA graph.
    _cudagraph_support = AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    def __init__(self, kv_cache_spec, layer_names, vllm_config, device):
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        self._init_reorder_batch_threshold(1)
        self._impl = _b.B200AttentionMetadataBuilder(kv_cache_spec, layer_names, vllm_config,
                                                     device)

    def build(self, common_prefix_len, common_attn_metadata, fast_build: bool = False):
        return self._impl.build(common_prefix_len, common_attn_metadata, fast_build)


class B200VllmAttentionImpl(_b.B200AttentionBackendImpl, AttentionImpl[_b.B200Metadata]):
    def __init__(self, num_heads, head_size, scale, num_kv_heads=None, alibi_slopes=None,
                 sliding_window=None, kv_cache_dtype="auto", logits_soft_cap=None,
                 attn_type=AttentionType.DECODER, kv_sharing_target_layer_name=None, **extra):
        _b.B200AttentionBackendImpl.__init__(
            self, num_heads, head_size, scale,
            num_kv_heads if num_kv_heads is not None else num_heads, alibi_slopes,
            sliding_window, kv_cache_dtype, logits_soft_cap, attn_type,
            kv_sharing_target_layer_name, extra.get("sinks"))
        self.kv_cache_dtype = kv_cache_dtype

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                output_scale=None, output_block_scale=None):
        if attn_metadata is None:          # memory-profiling run: no metadata, nothing to attend
            return output.fill_(0) if output is not None else query.new_zeros(query.shape)
        return _b.B200AttentionBackendImpl.forward(
            self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale,
            output_block_scale)


class B200VllmAttentionBackend(AttentionBackend):
    accept_output_buffer = True
    forward_includes_kv_cache_update = True
    supported_dtypes = [torch.bfloat16]
    # fp8 = unscaled e4m3, as the plugin stores it (attention.py:42-51, 692-700); head_size 128
    supported_kv_cache_dtypes = ["auto", "bfloat16", "fp8", "fp8_e4m3"]

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return B200VllmAttentionImpl

    @staticmethod
    def get_builder_cls():
        return B200VllmMetadataBuilder

    @staticmethod
    def get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size,
                           cache_dtype_str: str = "auto"):
        # vLLM's CUDA runner holds one tensor per layer: index 0 / 1 are the K and V tensors of
        # the plugin layout (attention.py:103-112).
        return _b.B200AttentionBackend.get_fused_kv_cache_shape(num_blocks, block_size,
                                                                num_kv_heads, head_size)

    @staticmethod
    def get_supported_kernel_block_sizes():
        return list(_b.B200AttentionBackend.supported_block_sizes)

    @classmethod
    def get_supported_head_sizes(cls):
        return list(_b.B200AttentionBackend.supported_head_sizes)

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return getattr(capability, "major", 10) == 10


def register() -> None:
    """`vllm.general_plugins` entry point."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend

    register_backend(AttentionBackendEnum.CUSTOM,
                     "b200attn.vllm_plugin.B200VllmAttentionBackend")
    # o_proj / down_proj through the fused GEMM + all-reduce launch is opt-in:
    # B200ATTN_FUSED_ROW_PARALLEL=1 (every tensor-parallel size) or =4 / =8 (from that many ranks
    # up).  Unset or 0: vLLM's own GEMM + all-reduce.
    mode = os.environ.get("B200ATTN_FUSED_ROW_PARALLEL", "0")
    if mode.isdigit() and int(mode) >= 1:
        enable_fused_row_parallel(min_world=max(2, int(mode)))


def config_allows_fused_row_parallel(vllm_config) -> tuple[bool, str]:
    """The fused launch is a raw C-ABI call: it is used only where vLLM runs the layer eagerly
    or inside its own CUDA graphs (compilation mode 0), and only in an engine that selected this
    repository's attention backend."""
    if vllm_config is None:
        return False, "no vLLM config at layer construction"
    backend = getattr(getattr(vllm_config, "attention_config", None), "backend", None)
    if getattr(backend, "name", str(backend)) != "CUSTOM":
        return False, f"attention backend is {backend}, not CUSTOM"
    mode = getattr(getattr(vllm_config, "compilation_config", None), "mode", None)
    if int(getattr(mode, "value", mode if mode is not None else -1)) != 0:
        return False, f"compilation mode {mode}: the launch is not traceable by torch.compile"
    return True, "ok"


def ranks_allow_fused_row_parallel(infos: list, can_access_peer) -> tuple[bool, str]:
    """`infos`: one dict per tensor-parallel rank (`host`, `device` index, compute capability
    `major`).  The kernel is sm_100a code, and `cudaIpcOpenMemHandle` plus peer stores need every
    rank on one node with peer access between every pair of GPUs.  `can_access_peer(i, j)`
    answers for device indices of this node."""
    if len(infos) < 2:
        return False, "a single rank has nothing to reduce"
    if any(i["major"] != 10 for i in infos):
        return False, "not every rank runs on compute capability 10.x"
    if len({i["host"] for i in infos}) != 1:
        return False, "the tensor-parallel group spans more than one node"
    devs = [i["device"] for i in infos]
    if len(set(devs)) != len(devs):
        return False, "two ranks share one GPU"
    for a in devs:
        for b in devs:
            if a != b and not can_access_peer(a, b):
                return False, f"GPU {a} cannot access GPU {b} as a peer"
    return True, "ok"


def _agree(group, ok: bool) -> bool:
    """True only if every rank of `group` says ok (carried as Python objects, any backend)."""
    import torch.distributed as dist

    votes = [None] * dist.get_world_size(group)
    dist.all_gather_object(votes, bool(ok), group=group)
    return all(votes)


def create_group_communicator(group, device, max_n: int, max_tokens: int):
    """Collective over `group`: checks the ranks, creates the communicator, and returns it only
    if every rank succeeded; otherwise every rank returns None (and keeps vLLM's forward)."""
    import socket

    import torch.distributed as dist

    from . import tp_linear

    mine = {"host": socket.gethostname(), "device": torch.device(device).index or 0,
            "major": torch.cuda.get_device_capability(device)[0]}
    infos = [None] * dist.get_world_size(group)
    dist.all_gather_object(infos, mine, group=group)
    ok, why = ranks_allow_fused_row_parallel(infos, torch.cuda.can_device_access_peer)
    comm = None
    if _agree(group, ok):
        try:
            comm = tp_linear.RowLinearComm(group, max_n=max_n, max_tokens=max_tokens,
                                           device=device)
        except Exception as exc:
            why = f"communicator creation failed: {exc}"
            comm = None
        if not _agree(group, comm is not None):
            if comm is not None:
                comm.close()
            comm = None
    elif ok:
        why = "another rank refused"
    if dist.get_rank(group) == 0:
        if comm is not None:
            logger.warning("b200attn: fused row-parallel linear ON for %d ranks", len(infos))
        else:
            logger.warning("b200attn: fused row-parallel linear stays off: %s", why)
    return comm


def enable_fused_row_parallel(max_tokens: int = 128, max_n: int = 8192, min_world: int = 2) -> None:
    """Points vLLM's RowParallelLinear (o_proj, down_proj: the layers the reference row-shards,
    vllm_tt/vllm_distributed_utils.py:356-363) at the fused GEMM + all-reduce launch for bf16
    batches of up to `max_tokens` rows; every other case keeps vLLM's GEMM + all-reduce.

    A layer takes part only if it was built in an engine that selected the CUSTOM attention
    backend with compilation mode 0 (`config_allows_fused_row_parallel`).  The communicator of the
    tensor-parallel group is created at the first forward of any such layer, which all ranks
    reach together during vLLM's eager profiling pass, well before decode steps are captured
    into CUDA graphs; the ranks first agree that all of them sit on one node with peer access
    and compute capability 10 (`create_group_communicator`), and fall back together otherwise.
    When the per-step watch on the diagnostics word reports a problem, the hook switches itself
    off for the rest of the process.  Layers of groups smaller than `min_world` are left alone."""
    from vllm.config import get_current_vllm_config_or_none
    from vllm.distributed import get_tp_group
    from vllm.model_executor.layers.linear import RowParallelLinear, UnquantizedLinearMethod

    from . import ops, tp_linear

    if getattr(RowParallelLinear, "_b200attn_fused", False):
        return
    original = RowParallelLinear.forward
    original_init = RowParallelLinear.__init__
    state = {"comm": None, "tried": False, "off": False}

    def switch_off(_word=None):
        state["off"] = True

    ops.ErrorWordWatch.on_error.append(switch_off)

    def __init__(self, *args, **kwargs):
        original_init(self, *args, **kwargs)
        self._b200attn_fusable = config_allows_fused_row_parallel(
            get_current_vllm_config_or_none())[0]

    def forward(self, input_):
        eligible = (
            not state["off"] and getattr(self, "_b200attn_fusable", False)
            and self.tp_size >= min_world and self.reduce_results and self.input_is_parallel
            and self.bias is None and isinstance(self.quant_method, UnquantizedLinearMethod)
            and input_.dim() == 2 and input_.dtype == torch.bfloat16 and input_.is_cuda
            and self.weight.dtype == torch.bfloat16 and self.weight.shape[0] <= max_n
        )
        if not eligible:
            return original(self, input_)
        if not state["tried"]:
            state["tried"] = True
            state["comm"] = create_group_communicator(get_tp_group().cpu_group, input_.device,
                                                      max_n, max_tokens)
        if (state["comm"] is None or input_.shape[0] == 0 or input_.shape[0] > max_tokens
                or input_.stride(1) != 1):
            return original(self, input_)
        out = tp_linear.rowlinear_allreduce(input_, self.weight, state["comm"])
        return out if not self.return_bias else (out, None)

    RowParallelLinear.__init__ = __init__
    RowParallelLinear.forward = forward
    RowParallelLinear._b200attn_fused = True
    RowParallelLinear._b200attn_state = state
