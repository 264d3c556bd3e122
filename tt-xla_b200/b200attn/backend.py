"""Attention backend classes with the surface of tt-xla's vLLM plugin backend
(integrations/vllm_plugin/vllm_tt/attention_impls/attention.py), running on b200attn's CUDA
kernels instead of `torch.ops.tt.*` custom calls lowered through PJRT.

    TTAttentionBackend         (attention.py:89-160)  -> B200AttentionBackend
    TTAttentionMetadataBuilder (attention.py:56-86)   -> B200AttentionMetadataBuilder
    TTMetadata                 (attention.py:177-218) -> B200Metadata
    TTAttentionBackendImpl     (attention.py:221-668) -> B200AttentionBackendImpl

Two metadata forms reach `forward`:
  * the plugin's own: `[users x padded tokens]` rows with `cache_position`, `page_table`,
    `fill_page_table`, `batch_idx`, `chunk_start_idx`, `num_users` (what TTModelRunner
    builds, model_runner.py:1894-2016);
  * vLLM's flattened varlen form (`query_start_loc`, `seq_lens`, `block_table`,
    `slot_mapping`), which B200AttentionMetadataBuilder.build derives from
    CommonAttentionMetadata; decode rows go to the split-KV kernel and prefill / chunk rows
    to the tcgen05 kernel in the same forward.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import ops

# B200ATTN_NVTX=1 wraps every layer's forward in an NVTX range (timeline tools group the
# launches of a layer under it); off, the path takes one global read more.
_NVTX = os.environ.get("B200ATTN_NVTX", "0") not in ("", "0")

# head_size must be a multiple of 32 on the reference device; page accounting keeps that
# padding rule (attention.py:37-38, 721-771).
HEAD_SIZE_ALIGNMENT = 32

STR_DTYPE_TO_TORCH_DTYPE = {
    "half": torch.half,
    "bfloat16": torch.bfloat16,
    "float": torch.float,
    "fp8": torch.float8_e4m3fn,
    "fp8_e4m3": torch.float8_e4m3fn,
    "fp8_e5m2": torch.float8_e5m2,
    "int8": torch.int8,
    "uint8": torch.uint8,
}

DECODER, ENCODER, ENCODER_ONLY = "decoder", "encoder", "encoder_only"


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class B200Metadata:
    """Per-step attention metadata; the first nine fields are TTMetadata's (attention.py:177-218),
    the rest carry vLLM's varlen form."""

    cache_position: Optional[torch.Tensor] = None   # [users] i32 = seq_len-1; -1 on padded rows
    attn_mask: Optional[torch.Tensor] = None        # always None on the generative path
    page_table: Optional[torch.Tensor] = None       # [users, nblk] i32, logical block order
    is_causal: bool = True
    fill_page_table: Optional[torch.Tensor] = None  # page_table rolled left by computed blocks
    dp_size: int = 1
    chunk_start_idx: Optional[torch.Tensor] = None  # [1] i32 shared prefix length, or None
    batch_idx: Optional[torch.Tensor] = None        # [users] i32
    num_users: Optional[int] = None
    # ---- vLLM varlen form
    slot_mapping: Optional[torch.Tensor] = None     # [tokens] i64
    query_start_loc: Optional[torch.Tensor] = None  # [seqs+1] i32, device
    query_start_loc_cpu: Optional[torch.Tensor] = None
    seq_lens: Optional[torch.Tensor] = None         # [seqs] i32, device
    block_table: Optional[torch.Tensor] = None      # [seqs, nblk] i32
    num_decodes: int = 0                            # leading rows with one query token
    max_seq_len: int = 0
    # derived once per step by the builder (shared by all layers)
    decode_cur_pos: Optional[torch.Tensor] = None
    prefill_cu_q: Optional[torch.Tensor] = None
    prefill_cu_q_cpu: Optional[torch.Tensor] = None
    prefill_q_start: Optional[torch.Tensor] = None
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        # attention.py:210-212: fill_page_table defaults to page_table.
        if self.fill_page_table is None:
            self.fill_page_table = self.page_table

    @property
    def is_varlen(self) -> bool:
        return self.query_start_loc is not None


class B200AttentionMetadataBuilder:
    """Turns vLLM's CommonAttentionMetadata into B200Metadata.  The reference's builder is a stub
    (attention.py:56-86) because its runner fills TTMetadata itself; on CUDA, vLLM's runner
    calls `build` once per step and hands the result to every layer."""

    reorder_batch_threshold = 1  # decode rows (one query token) are ordered first by vLLM

    def __init__(self, kv_cache_spec=None, layer_names=None, vllm_config=None, device=None):
        self.kv_cache_spec = kv_cache_spec
        self.layer_names = layer_names
        self.vllm_config = vllm_config
        self.device = device
        self.decode_cur_pos_buffer = None
        self.error_watch = None
        max_seqs = getattr(getattr(vllm_config, "scheduler_config", None), "max_num_seqs", None)
        if max_seqs and device is not None:
            # -1 = padding row: the decode launch neither streams nor writes anything for it
            self.decode_cur_pos_buffer = torch.full((int(max_seqs),), -1, dtype=torch.int32,
                                                    device=device)
        if device is not None and torch.device(device).type == "cuda":
            self.error_watch = ops.ErrorWordWatch(torch.device(device))

    def device_step_state(self, rows: int, page_table_width: int, block_size: int,
                          tokens_per_row: int = 1) -> "DeviceStepState":
        """For runners that hold their scheduler state on the GPU: the one-launch metadata build
        (see DeviceStepState)."""
        return DeviceStepState(rows, page_table_width, block_size, tokens_per_row, self.device)

    def build(self, common_prefix_len: int, common_attn_metadata, fast_build: bool = False):
        m = common_attn_metadata
        if self.error_watch is not None:
            self.error_watch.poll()      # raises when an earlier step's kernels reported a problem
        qsl = getattr(m, "query_start_loc", None)
        if qsl is None:
            # Same minimal object the reference builder returns.
            return B200Metadata(is_causal=getattr(m, "causal", True))
        qsl_cpu = getattr(m, "query_start_loc_cpu", None)
        if qsl_cpu is None:
            qsl_cpu = qsl.cpu()
        return build_varlen_metadata(
            query_start_loc=qsl,
            query_start_loc_cpu=qsl_cpu,
            seq_lens=m.seq_lens,
            block_table=m.block_table_tensor,
            slot_mapping=m.slot_mapping,
            max_seq_len=int(getattr(m, "max_seq_len", 0) or 0),
            is_causal=getattr(m, "causal", True),
            decode_cur_pos_buffer=self.decode_cur_pos_buffer,
        )


class DeviceStepState:
    """Persistent device buffers of the plugin-form metadata for a runner that keeps its
    scheduler state (`num_computed`, `num_scheduled`, `block_table`) on the GPU.  `build()` fills
    them with ONE launch (`b200attn_build_step_metadata`) and returns the B200Metadata every layer
    of the step receives: what `TTModelRunner._prepare_inputs` computes on the host and copies
    over tensor by tensor (model_runner.py:1722-1741, 1945-1993).  The buffers keep their
    addresses, so a step captured into a CUDA graph replays against the next step's values."""

    def __init__(self, rows: int, page_table_width: int, block_size: int, tokens_per_row: int,
                 device):
        from . import metadata as _md

        self.rows, self.block_size, self.tokens_per_row = rows, block_size, tokens_per_row
        fill_width = _md.fill_page_table_width(tokens_per_row, block_size, page_table_width)
        i32 = dict(dtype=torch.int32, device=device)
        self.buffers = _md.StepMetadata(
            cache_position=torch.full((rows,), -1, **i32),
            page_table=torch.zeros((rows, page_table_width), **i32),
            fill_page_table=torch.zeros((rows, fill_width), **i32),
            slot_mapping=torch.full((rows * tokens_per_row,), -1, dtype=torch.int64,
                                    device=device),
            chunk_start_idx=None)
        self.batch_idx = torch.arange(rows, **i32)

    def build(self, num_computed: torch.Tensor, num_scheduled: torch.Tensor,
              block_table: torch.Tensor, chunk_start_idx: Optional[torch.Tensor] = None,
              max_seq_len: int = 0) -> "B200Metadata":
        from . import metadata as _md

        _md.build_step_metadata(num_computed, num_scheduled, block_table, self.block_size,
                                self.buffers, self.tokens_per_row)
        b = self.buffers
        return B200Metadata(cache_position=b.cache_position, page_table=b.page_table,
                            fill_page_table=b.fill_page_table, batch_idx=self.batch_idx,
                            chunk_start_idx=chunk_start_idx, num_users=self.rows,
                            slot_mapping=b.slot_mapping, max_seq_len=max_seq_len)


def build_varlen_metadata(
    query_start_loc: torch.Tensor,
    query_start_loc_cpu: torch.Tensor,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    slot_mapping: torch.Tensor,
    max_seq_len: int = 0,
    is_causal: bool = True,
    decode_cur_pos_buffer: Optional[torch.Tensor] = None,
) -> B200Metadata:
    """Derives the per-kernel index tensors from vLLM's varlen fields.  Rows whose query length
    is 1 must come first (vLLM's decode-first batch order).  `decode_cur_pos_buffer`, when
    given, is a persistent int32 buffer the decode positions are written into, so that a CUDA
    graph captured over a decode step keeps reading the right memory on replay."""
    qsl_cpu = query_start_loc_cpu.to(torch.int32)
    q_lens = qsl_cpu[1:] - qsl_cpu[:-1]
    num_seqs = q_lens.numel()
    num_decodes = 0
    while num_decodes < num_seqs and int(q_lens[num_decodes]) == 1:
        num_decodes += 1
    # A one-token row after a longer one is served as a prefill row of length 1.
    seq_lens = seq_lens.to(torch.int32)
    qsl = query_start_loc.to(torch.int32)
    md = B200Metadata(
        is_causal=is_causal,
        slot_mapping=slot_mapping,
        query_start_loc=qsl,
        query_start_loc_cpu=qsl_cpu,
        seq_lens=seq_lens,
        block_table=block_table,
        num_decodes=num_decodes,
        max_seq_len=max_seq_len,
        num_users=num_seqs,
    )
    if num_decodes > 0:
        if decode_cur_pos_buffer is not None and decode_cur_pos_buffer.numel() >= num_decodes:
            md.decode_cur_pos = decode_cur_pos_buffer[:num_decodes]
            torch.sub(seq_lens[:num_decodes], 1, out=md.decode_cur_pos)
            # A CUDA graph captured at a larger (padded) batch reads further into the buffer:
            # rows past this step's decodes must read as padding, not as an earlier step's
            # positions.
            decode_cur_pos_buffer[num_decodes:].fill_(-1)
        else:
            md.decode_cur_pos = (seq_lens[:num_decodes] - 1).contiguous()
    if num_decodes < num_seqs:
        base = int(qsl_cpu[num_decodes])
        md.prefill_cu_q_cpu = (qsl_cpu[num_decodes:] - base).contiguous()
        md.prefill_cu_q = (qsl[num_decodes:] - base).contiguous()
        # first query row of sequence s sits at position seq_len - q_len
        md.prefill_q_start = (
            seq_lens[num_decodes:] - (qsl[num_decodes + 1:] - qsl[num_decodes:-1])
        ).contiguous()
    return md


class B200AttentionBackend:
    """Static descriptors of the backend (attention.py:89-160)."""

    accept_output_buffer = True
    forward_includes_kv_cache_update = True
    supported_dtypes = [torch.bfloat16]
    supported_kv_cache_dtypes = ["auto", "bfloat16", "fp8", "fp8_e4m3"]   # fp8: head_size 128
    supported_head_sizes = [64, 128]
    supported_block_sizes = [32, 64]

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls():
        return B200AttentionBackendImpl

    @staticmethod
    def get_builder_cls():
        return B200AttentionMetadataBuilder

    @staticmethod
    def get_metadata_cls():
        return B200Metadata

    @staticmethod
    def get_kv_cache_shape(
        num_blocks: int,
        block_size: int,
        num_kv_heads: int,
        head_size: int,
        cache_dtype_str: str = "auto",
    ) -> tuple[int, ...]:
        # One of the two separate K / V tensors per layer (attention.py:103-112).
        return (num_blocks, num_kv_heads, block_size, head_size)

    @staticmethod
    def get_fused_kv_cache_shape(
        num_blocks: int, block_size: int, num_kv_heads: int, head_size: int
    ) -> tuple[int, ...]:
        # vLLM's CUDA runner allocates one tensor per layer; index 0 / 1 of this shape are the
        # K and V tensors above, bit-identical in layout.
        return (2, num_blocks, num_kv_heads, block_size, head_size)

    @staticmethod
    def swap_blocks(src_kv_cache, dst_kv_cache, src_to_dst) -> None:
        raise RuntimeError("swap_blocks is not used for the B200 backend.")

    # The plugin keeps one request's page-table row under a fixed budget of int32 entries:
    # 128 Ki entries (half a MiB) shared by all resident requests (attention.py:126-140).
    PAGE_TABLE_ENTRY_BUDGET = (1 << 20) // 2 // 4

    @classmethod
    def get_min_page_size(cls, max_model_len: int, max_num_seqs: int) -> int:
        """Smallest power-of-two page size whose page-table rows fit the entry budget."""
        entries_per_request = cls.PAGE_TABLE_ENTRY_BUDGET // max_num_seqs
        return 1 << (cdiv(max_model_len, entries_per_request) - 1).bit_length()

    @classmethod
    def get_max_num_seqs(cls, model_len: int, page_size: int) -> int:
        """How many requests of `model_len` tokens fit the entry budget at `page_size`."""
        return cls.PAGE_TABLE_ENTRY_BUDGET // cdiv(model_len, page_size)

    @staticmethod
    def get_page_size(vllm_config=None) -> int:
        # attention.py:146-152: the reference pins 32.
        return 32

    @classmethod
    def supports_head_size(cls, head_size: int) -> bool:
        return head_size in cls.supported_head_sizes

    @classmethod
    def supports_block_size(cls, block_size: int) -> bool:
        return block_size in cls.supported_block_sizes


def dtype_bits(dtype: torch.dtype) -> int:
    """Storage bits of one element (attention.py:721-737); bool counts as a byte."""
    if dtype == torch.bool:
        return 8
    info = torch.finfo(dtype) if dtype.is_floating_point else torch.iinfo(dtype)
    return info.bits


def get_dtype_packing(dtype: torch.dtype) -> int:
    """Elements per 32-bit word (attention.py:740-747)."""
    bits = dtype_bits(dtype)
    per_word, rest = divmod(32, bits)
    if rest:
        raise ValueError(f"The bit width must be divisible by 32, but got bits={bits}")
    return per_word


def get_page_size_bytes(
    block_size: int, num_kv_heads: int, head_size: int, kv_cache_dtype: torch.dtype
) -> int:
    """Bytes of one page holding K and V (attention.py:750-771): head_size rounded up to the
    device's 32-element granule, the 2 * num_kv_heads rows rounded up to whole 32-bit words."""
    packing = get_dtype_packing(kv_cache_dtype)
    rows = cdiv(2 * num_kv_heads, packing) * packing
    width = cdiv(head_size, HEAD_SIZE_ALIGNMENT) * HEAD_SIZE_ALIGNMENT
    return block_size * rows * width * dtype_bits(kv_cache_dtype) // 8


def rows_by_user(tensor: torch.Tensor, name: str, heads: int, head_size: int,
                 users: int) -> torch.Tensor:
    """View of a plugin-form activation as [users, tokens, heads, head_size].  Accepted inputs
    and the error texts are those of attention.py:338-379: token rows flattened to
    `heads * head_size` columns, or already split into (heads, head_size)."""
    hidden = heads * head_size
    if tensor.ndim < 2:
        raise ValueError(f"{name} must have rank >= 2, got shape={tuple(tensor.shape)}")
    flat = tensor.ndim == 2 and tensor.shape[1] == hidden
    split = tensor.ndim == 3 and tuple(tensor.shape[1:]) == (heads, head_size)
    if not (flat or split):
        raise ValueError(
            f"{name} must be either a flattened-token tensor with "
            f"shape[-1] == {hidden} or a head-shaped tensor with "
            f"shape[-2:] == ({heads}, {head_size}); "
            f"got shape={tuple(tensor.shape)}"
        )
    rows = tensor.shape[0]
    if rows % users:
        raise ValueError(
            f"{name} total tokens ({rows}) must be divisible "
            f"by num_users ({users})"
        )
    return tensor.reshape(users, rows // users, heads, head_size)


@dataclass
class PluginBatch:
    """One pass in the plugin's [users x tokens] form.  The whole batch is in one mode: a pass
    with more than one query token per user is a prefill pass (attention.py:429)."""

    query: torch.Tensor      # [users, tokens, nq, hd]
    key: torch.Tensor        # [users, tokens, nkv, hd]
    value: torch.Tensor
    users: int
    query_num_tokens: int
    kv_num_tokens: int

    @property
    def is_prefill(self) -> bool:
        return self.query_num_tokens > 1


class B200AttentionBackendImpl:
    """Per-layer attention implementation (attention.py:221-668)."""

    def __init__(
        self,
        num_heads: int,
        head_size: int,
        scale: float,
        num_kv_heads: int,
        alibi_slopes: Optional[list] = None,
        sliding_window: Optional[int] = None,
        kv_cache_dtype: str = "auto",
        logits_soft_cap: Optional[float] = None,
        attn_type: str = DECODER,
        kv_sharing_target_layer_name: Optional[str] = None,
        sinks: Optional[torch.Tensor] = None,
    ) -> None:
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = float(scale)
        self.num_kv_heads = num_kv_heads
        self.sliding_window = sliding_window
        self.logits_soft_cap = logits_soft_cap
        self.kv_sharing_target_layer_name = kv_sharing_target_layer_name
        self.num_queries_per_kv = self.num_heads // self.num_kv_heads
        if alibi_slopes is not None:
            raise NotImplementedError("Alibi slopes is not supported.")
        if str(getattr(attn_type, "value", attn_type)) not in (DECODER, ENCODER, ENCODER_ONLY):
            raise NotImplementedError(
                f"B200 attention only supports encoder or decoder attention, but got {attn_type}."
            )
        self.attn_type = attn_type
        # The reference maps the engine's names to torch dtypes (attention.py:42-51, 259-263).
        # The CUDA kernels store bf16 or unscaled e4m3 and refuse the rest instead of silently
        # converting.
        self.kv_cache_quantized_dtype = None
        if kv_cache_dtype in ("fp8", "fp8_e4m3"):
            self.kv_cache_quantized_dtype = torch.float8_e4m3fn
        elif kv_cache_dtype not in ("auto", "bfloat16"):
            raise NotImplementedError(
                f"kv_cache_dtype {kv_cache_dtype!r} is not supported (bfloat16 or fp8_e4m3 caches)"
            )
        if sliding_window is not None and int(sliding_window) <= 0:
            raise ValueError(f"sliding_window must be positive, got {sliding_window}")
        self._window = 0 if sliding_window is None else int(sliding_window)
        if logits_soft_cap is not None:
            raise NotImplementedError("logits_soft_cap is not supported")
        self.sinks = sinks
        self._sinks_f32 = None   # ((device, data_ptr, version), fp32 copy)
        # Set by a caller that has already written this step's K / V rows into the cache (the
        # fused rotary + cache write of B200Attention); consumed by the next forward.
        self.kv_written_upstream = False
        if self.sinks is not None:
            assert self.sinks.shape[0] == num_heads, (
                "Sinks must have the same number of heads as the number of "
                f"heads in the layer. Sinks shape: {sinks.shape}, num_heads: {num_heads}."
            )   # attention.py:265-270

    def _sinks_for(self, device) -> Optional[torch.Tensor]:
        """fp32 copy of the per-head sink logits on `device` (made once; the decode kernel reads
        fp32).  attention.py:650 hands the op the parameter as it is."""
        if self.sinks is None:
            return None
        key = (str(device), self.sinks.data_ptr(), self.sinks._version)
        if self._sinks_f32 is None or self._sinks_f32[0] != key:
            copy = self.sinks.detach().to(device=device, dtype=torch.float32).contiguous()
            self._sinks_f32 = (key, copy)
        return self._sinks_f32[1]

    # ------------------------------------------------------------------ forward
    def forward(
        self,
        layer,
        query: torch.Tensor,
        key: torch.Tensor,
        value: torch.Tensor,
        kv_cache,
        attn_metadata: B200Metadata,
        output: Optional[torch.Tensor] = None,
        output_scale: Optional[torch.Tensor] = None,
        output_block_scale: Optional[torch.Tensor] = None,
    ) -> Optional[torch.Tensor]:
        """query [tokens, nq*hd], key/value [tokens, nkv*hd], kv_cache = [k_cache, v_cache]
        (or one tensor [2, nb, nkv, bs, hd]); writes `output` in place (attention.py:273-336)."""
        assert attn_metadata is not None, "B200 attention requires metadata."
        assert output is not None, "B200 attention requires an output buffer."
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantisation is not supported")
        if _NVTX:
            with torch.cuda.nvtx.range(f"b200attn.forward[{getattr(layer, 'layer_name', '')}]"):
                return self._forward(query, key, value, kv_cache, attn_metadata, output)
        return self._forward(query, key, value, kv_cache, attn_metadata, output)

    def _forward(self, query, key, value, kv_cache, attn_metadata, output):
        kv_pair = self._split_kv_cache(kv_cache)
        written, self.kv_written_upstream = self.kv_written_upstream, False
        if attn_metadata.is_varlen:
            self._forward_varlen(query, key, value, kv_pair, attn_metadata, output,
                                 writes_cache=not written)
            return output

        inputs = self._prepare_inputs(query, key, value, attn_metadata)
        has_cache = kv_pair is not None
        writes_cache = has_cache and self.kv_sharing_target_layer_name is None and not written
        if inputs.is_prefill:
            if writes_cache:
                self._handle_paged_attention(inputs, kv_pair, attn_metadata)
            self._compute_full_attention(inputs, kv_pair, attn_metadata, output)
        else:
            if not has_cache:
                raise ValueError("decode attention needs the paged KV cache")
            # the decode step's cache write (attention.py:468-484) rides in the decode launch
            self._compute_decode_attention(inputs, kv_pair, attn_metadata, output,
                                           write_new_token=writes_cache)
        return output

    def _split_kv_cache(self, kv_cache):
        """[k_cache, v_cache] (the reference's form, model_runner.py:4603-4609), or vLLM's single
        [2, nb, nkv, bs, hd] tensor; None while profiling with a placeholder.  An engine that
        stores an fp8 cache as raw bytes (vLLM allocates uint8) gets the e4m3 view the kernels
        and the plugin's dtype map (attention.py:42-51) mean."""
        pair = None
        if isinstance(kv_cache, (list, tuple)):
            if len(kv_cache) >= 2 and kv_cache[0].numel() > 0:
                pair = (kv_cache[0], kv_cache[1])
        elif isinstance(kv_cache, torch.Tensor) and kv_cache.dim() == 5 and kv_cache.shape[0] == 2:
            pair = (kv_cache[0], kv_cache[1])
        if pair is not None and self.kv_cache_quantized_dtype is not None \
                and pair[0].dtype == torch.uint8:
            pair = (pair[0].view(self.kv_cache_quantized_dtype),
                    pair[1].view(self.kv_cache_quantized_dtype))
        return pair

    def _prepare_inputs(self, query, key, value, attn_metadata: B200Metadata) -> PluginBatch:
        """Shapes the three activations by user (what attention.py:381-459 hands its ops)."""
        users = attn_metadata.num_users
        assert users is not None, "num_users must be provided in attn_metadata."
        q = rows_by_user(query, "query", self.num_heads, self.head_size, users)
        k = rows_by_user(key, "key", self.num_kv_heads, self.head_size, users)
        v = rows_by_user(value, "value", self.num_kv_heads, self.head_size, users)
        if k.shape != v.shape:
            raise ValueError(
                f"key and value must match after normalization, got "
                f"key={tuple(k.shape)} value={tuple(v.shape)}"
            )
        return PluginBatch(q, k, v, users, q.shape[1], k.shape[1])

    def _handle_paged_attention(self, inputs, kv_pair, attn_metadata: B200Metadata) -> None:
        """KV-cache write (attention.py:461-515): one launch covers K and V."""
        k_cache, v_cache = kv_pair
        if not inputs.is_prefill:
            ops.paged_update_cache(
                k_cache, v_cache, inputs.key[:, 0], inputs.value[:, 0],
                attn_metadata.cache_position, attn_metadata.page_table,
            )
            return
        batch_idxs = attn_metadata.batch_idx
        assert batch_idxs is not None, "batch_idx must be provided for prefill."
        if attn_metadata.dp_size > 1:
            local_batch = inputs.key.shape[0] // attn_metadata.dp_size
            batch_idxs = batch_idxs % local_batch
        ops.paged_fill_cache(
            k_cache, v_cache, inputs.key, inputs.value, attn_metadata.fill_page_table, batch_idxs
        )

    def _uniform_cu_q(self, users: int, tokens: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        key = (users, tokens, str(device))
        cache = self.__dict__.setdefault("_cu_q_cache", {})
        if key not in cache:
            host = torch.arange(users + 1, dtype=torch.int32) * tokens
            cache[key] = (host, host.to(device))
        return cache[key]

    def _compute_full_attention(self, inputs, kv_pair, attn_metadata: B200Metadata, output) -> None:
        """Prefill (attention.py:517-598): chunk over the paged prefix when chunk_start_idx is
        set, dense causal attention on the fresh K/V otherwise."""
        if attn_metadata.attn_mask is not None or not attn_metadata.is_causal:
            raise NotImplementedError(
                "only causal attention without an explicit mask is supported (the generative "
                "path; model_runner.py:2004-2016)"
            )
        assert self.sinks is None, "Attention sink is unsupported in SDPA prefill"  # :321
        users, tokens = inputs.users, inputs.query_num_tokens
        q = inputs.query.reshape(users * tokens, self.num_heads, self.head_size)
        out = output.reshape(users * tokens, self.num_heads, self.head_size)
        cu_host, cu_dev = self._uniform_cu_q(users, tokens, q.device)
        has_cache = kv_pair is not None
        shared_kv_mode = self.kv_sharing_target_layer_name is not None and has_cache
        if attn_metadata.chunk_start_idx is not None and has_cache and not shared_kv_mode:
            q_start = attn_metadata.chunk_start_idx.reshape(-1)[:1].to(torch.int32).expand(users)
            ops.prefill(
                q, kv_pair[0], kv_pair[1], cu_host, scale=self.scale,
                page_table=attn_metadata.page_table, q_start=q_start.contiguous(), out=out,
                cu_q=cu_dev, sliding_window=self._window,
            )
        elif shared_kv_mode:
            # Shared-KV layers read the target layer's cache (attention.py:562-574); the kernel
            # reads pages directly, so no dense gather is needed.
            ops.prefill(
                q, kv_pair[0], kv_pair[1], cu_host, scale=self.scale,
                page_table=attn_metadata.page_table, q_start=None, out=out, cu_q=cu_dev,
                sliding_window=self._window,
            )
        else:
            k = inputs.key.reshape(users * tokens, self.num_kv_heads, self.head_size)
            v = inputs.value.reshape(users * tokens, self.num_kv_heads, self.head_size)
            ops.prefill(q, k, v, cu_host, scale=self.scale, out=out, cu_q=cu_dev,
                        sliding_window=self._window)

    def _compute_decode_attention(self, inputs, kv_pair, attn_metadata: B200Metadata, output,
                                  write_new_token: bool = False) -> None:
        """attention.py:634-668; with `write_new_token` also the K / V write of attention.py:468-484
        (same positions, same page table) inside the same launch."""
        if attn_metadata.attn_mask is not None or not attn_metadata.is_causal:
            raise NotImplementedError("decode supports the causal cur_pos form only")
        users = inputs.users
        fused = {}
        if write_new_token:
            fused = dict(new_key=inputs.key[:, 0], new_value=inputs.value[:, 0])
        ops.paged_decode(
            inputs.query.reshape(users, self.num_heads, self.head_size),
            kv_pair[0], kv_pair[1], attn_metadata.page_table, attn_metadata.cache_position,
            scale=self.scale,
            out=output.reshape(users, self.num_heads, self.head_size),
            max_context_len=attn_metadata.max_seq_len,
            sliding_window=self._window, sinks=self._sinks_for(output.device), **fused,
        )

    # ------------------------------------------------------------------ vLLM varlen form
    def _forward_varlen(self, query, key, value, kv_pair, md: B200Metadata, output,
                        writes_cache: bool = True) -> None:
        if kv_pair is None:
            # Memory-profiling run before the cache exists: nothing to attend to.
            output.zero_()
            return
        nq, nkv, hd = self.num_heads, self.num_kv_heads, self.head_size
        n_tok = int(md.query_start_loc_cpu[-1])
        q = query[:n_tok].reshape(n_tok, nq, hd)
        out = output[:n_tok].reshape(n_tok, nq, hd)
        nd = md.num_decodes
        writes_cache = writes_cache and self.kv_sharing_target_layer_name is None
        # A pure decode batch writes its new rows inside the decode launch (a row's slot is
        # block_table[pos // bs] * bs + pos % bs, which is what that launch computes; padding
        # rows carry position -1 and are skipped like slot -1); mixed batches scatter by slot.
        fused = {}
        if writes_cache and nd == n_tok and md.prefill_cu_q_cpu is None:
            fused = dict(new_key=key[:n_tok].reshape(n_tok, nkv, hd),
                         new_value=value[:n_tok].reshape(n_tok, nkv, hd),
                         wrap_negative_positions=False)
        elif writes_cache:
            ops.kv_scatter_slots(
                kv_pair[0], kv_pair[1], key[:n_tok].reshape(n_tok, nkv, hd),
                value[:n_tok].reshape(n_tok, nkv, hd), md.slot_mapping[:n_tok],
            )
        if nd > 0:
            ops.paged_decode(
                q[:nd], kv_pair[0], kv_pair[1], md.block_table[:nd], md.decode_cur_pos,
                scale=self.scale, out=out[:nd], max_context_len=md.max_seq_len,
                sliding_window=self._window, sinks=self._sinks_for(output.device), **fused,
            )
        if md.prefill_cu_q_cpu is not None:
            assert self.sinks is None, "Attention sink is unsupported in SDPA prefill"
            ops.prefill(
                q[nd:], kv_pair[0], kv_pair[1], md.prefill_cu_q_cpu, scale=self.scale,
                page_table=md.block_table[nd:], q_start=md.prefill_q_start, out=out[nd:],
                cu_q=md.prefill_cu_q, sliding_window=self._window,
            )


def flatten_heads(tensor: Optional[torch.Tensor], name: str, heads: int,
                  head_size: int) -> Optional[torch.Tensor]:
    """Any-rank activation -> [rows, heads * head_size] (the layer wrapper's input rule,
    attention.py:798-825): the last dim is already the hidden width, or the last two are
    (heads, head_size)."""
    if tensor is None:
        return None
    if tensor.ndim < 2:
        raise ValueError(f"{name} must have rank >= 2, got shape={tuple(tensor.shape)}")
    hidden = heads * head_size
    if tensor.shape[-1] != hidden and tuple(tensor.shape[-2:]) != (heads, head_size):
        raise ValueError(
            f"{name} must satisfy one of: "
            f"shape[-1] == {hidden} or "
            f"shape[-2:] == ({heads}, {head_size}); "
            f"got shape={tuple(tensor.shape)}"
        )
    return tensor.reshape(-1, hidden)


class B200Attention(torch.nn.Module):
    """Attention layer around the backend Impl for callers outside vLLM, with the input handling
    of the plugin's `TTAttention` wrapper (attention.py:774-856): query / key / value of any rank
    are flattened to 2-D token rows, the Impl runs, and the result comes back in the query's
    shape.  The layer owns what vLLM's `Attention` would hold for it: the Impl, the bound
    `kv_cache` pair (see `sharding.allocate_kv_caches` / `bind_kv_caches`) and the step's
    metadata (`set_metadata`, or the `attn_metadata` argument)."""

    def __init__(self, num_heads: int, head_size: int, scale: float,
                 num_kv_heads: Optional[int] = None, *, rotary_dim: Optional[int] = None,
                 rope_theta: float = 10000.0, **impl_kwargs) -> None:
        super().__init__()
        # NeoX-style rotary embedding applied by the layer itself when `forward` is given
        # positions (the plugin's rotary layer, layers/rotary_embedding.py:51-66): one launch
        # rotates q and k in place and, when the step's metadata carries a slot mapping, also
        # writes the rotated k and v into the cache, so the Impl skips its own cache write.
        self.rotary_dim = rotary_dim
        self.inv_freq = None
        if rotary_dim is not None:
            self.inv_freq = 1.0 / (rope_theta ** (
                torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
        self.num_heads = num_heads
        self.head_size = self.head_size_v = head_size
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        self.impl = B200AttentionBackendImpl(
            num_heads, head_size, scale, self.num_kv_heads,
            impl_kwargs.pop("alibi_slopes", None), impl_kwargs.pop("sliding_window", None),
            impl_kwargs.pop("kv_cache_dtype", "auto"), impl_kwargs.pop("logits_soft_cap", None),
            impl_kwargs.pop("attn_type", DECODER),
            impl_kwargs.pop("kv_sharing_target_layer_name", None), impl_kwargs.pop("sinks", None))
        if impl_kwargs:
            raise TypeError(f"unexpected arguments: {sorted(impl_kwargs)}")
        self.kv_cache = None
        self.attn_metadata: Optional[B200Metadata] = None

    def set_metadata(self, attn_metadata: B200Metadata) -> None:
        self.attn_metadata = attn_metadata

    def _rotate_and_write(self, q2, k2, v2, positions, md) -> None:
        """q2 / k2 rotated in place; with a slot mapping in the metadata and a cache of its own
        the same launch writes k and v, and the Impl is told so."""
        if self.inv_freq.device != q2.device:
            self.inv_freq = self.inv_freq.to(q2.device)
        kv_pair = self.impl._split_kv_cache(self.kv_cache)
        slots = getattr(md, "slot_mapping", None)
        fused_write = (kv_pair is not None and slots is not None
                       and self.impl.kv_sharing_target_layer_name is None
                       and kv_pair[0].dtype == torch.bfloat16)
        ops.rope_kv_scatter_slots(
            q2, k2, v2 if fused_write else None, positions.reshape(-1).to(torch.int64),
            self.inv_freq, self.rotary_dim, self.head_size,
            kv_pair[0] if fused_write else None, kv_pair[1] if fused_write else None,
            slots[: q2.shape[0]] if fused_write else None)
        self.impl.kv_written_upstream = fused_write

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                output_shape: Optional[torch.Size] = None,
                attn_metadata: Optional[B200Metadata] = None,
                positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        q2 = flatten_heads(query, "query", self.num_heads, self.head_size)
        k2 = flatten_heads(key, "key", self.num_kv_heads, self.head_size)
        v2 = flatten_heads(value, "value", self.num_kv_heads, self.head_size_v)
        out = torch.empty(output_shape if output_shape is not None else q2.shape,
                          dtype=q2.dtype, device=q2.device)
        md = attn_metadata if attn_metadata is not None else self.attn_metadata
        if positions is not None:
            if self.inv_freq is None:
                raise ValueError("positions given to a layer built without rotary_dim")
            self._rotate_and_write(q2, k2, v2, positions, md)
        self.impl.forward(self, q2, k2, v2, self.kv_cache, md, output=out.view(q2.shape[0], -1))
        if out.numel() != query.numel():
            raise ValueError(
                "Cannot reshape attention output back to query shape: "
                f"output_shape={tuple(out.shape)}, "
                f"query_shape={tuple(query.shape)}"
            )
        return out.reshape(query.shape)


def write_to_kv_cache(key, value, kv_cache, slot_mapping, *unused, **unused_kw) -> None:
    """Slot-mapping cache write (attention.py:671-716) on the live [k_cache, v_cache] layout."""
    k_cache, v_cache = kv_cache[0], kv_cache[1]
    nkv, hd = k_cache.shape[1], k_cache.shape[3]
    ops.kv_scatter_slots(
        k_cache, v_cache, key.reshape(-1, nkv, hd), value.reshape(-1, nkv, hd), slot_mapping
    )
