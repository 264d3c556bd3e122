"""Host-side logic of the backend mirror (no GPU): descriptors, page accounting, argument checks,
varlen metadata derivation."""
import pytest
import torch

from b200attn import (B200AttentionBackend, B200AttentionBackendImpl,
                      B200AttentionMetadataBuilder, B200Metadata, backend, ops)


def test_backend_descriptors_match_reference_contract():
    B = B200AttentionBackend
    assert B.get_name() == "CUSTOM"
    assert B.get_impl_cls() is B200AttentionBackendImpl
    assert B.get_builder_cls() is B200AttentionMetadataBuilder
    # one of the two separate K / V tensors per layer (attention.py:103-112)
    assert B.get_kv_cache_shape(512, 32, 8, 64) == (512, 8, 32, 64)
    assert B.get_fused_kv_cache_shape(512, 32, 8, 64) == (2, 512, 8, 32, 64)
    assert B.get_page_size() == 32
    with pytest.raises(RuntimeError, match="swap_blocks"):
        B.swap_blocks(None, None, None)
    # attention.py:137-140
    assert B.get_max_num_seqs(32768, 32) == 1024 * 1024 // 2 // 1024 // 4
    assert B.get_min_page_size(32768, 64) == 16


def test_page_size_bytes():
    # attention.py:750-771 arithmetic: 32 tokens x 16 combined heads x 64 x 2 bytes
    assert backend.get_page_size_bytes(32, 8, 64, torch.bfloat16) == 32 * 16 * 64 * 2
    # head_size padded to a multiple of 32
    assert backend.get_page_size_bytes(32, 8, 80, torch.bfloat16) == 32 * 16 * 96 * 2
    assert backend.get_dtype_packing(torch.bfloat16) == 2
    assert backend.dtype_bits(torch.int8) == 8


def test_metadata_defaults_and_positional_order():
    pt = torch.zeros(2, 4, dtype=torch.int32)
    md = B200Metadata(torch.tensor([3, 4], dtype=torch.int32), None, pt, True)
    assert md.fill_page_table is pt            # attention.py:210-212
    assert md.dp_size == 1 and md.chunk_start_idx is None and not md.is_varlen


def test_impl_constructor_errors():
    with pytest.raises(NotImplementedError, match="Alibi"):
        B200AttentionBackendImpl(8, 64, 0.125, 8, [1.0], None, "auto")
    with pytest.raises(NotImplementedError, match="encoder or decoder"):
        B200AttentionBackendImpl(8, 64, 0.125, 8, None, None, "auto", attn_type="encoder_decoder")
    for kw in (dict(kv_cache_dtype="fp8_e5m2"), dict(kv_cache_dtype="int8"),
               dict(logits_soft_cap=30.0)):
        args = dict(num_heads=8, head_size=64, scale=0.125, num_kv_heads=8, alibi_slopes=None,
                    sliding_window=None, kv_cache_dtype="auto")
        args.update(kw)
        with pytest.raises(NotImplementedError):
            B200AttentionBackendImpl(**args)
    with pytest.raises(ValueError, match="sliding_window"):
        B200AttentionBackendImpl(8, 64, 0.125, 8, None, 0, "auto")
    with pytest.raises(AssertionError, match="Sinks must have the same number of heads"):
        B200AttentionBackendImpl(8, 64, 0.125, 8, None, None, "auto", sinks=torch.zeros(4))
    impl = B200AttentionBackendImpl(8, 64, 0.125, 8, None, 128, "auto", sinks=torch.zeros(8))
    assert impl.sliding_window == 128 and impl.sinks is not None
    assert impl.kv_cache_quantized_dtype is None
    # attention.py:42-51: "fp8" and "fp8_e4m3" both mean float8_e4m3fn
    for name in ("fp8", "fp8_e4m3"):
        assert B200AttentionBackendImpl(8, 128, 0.1, 8, None, None, name).kv_cache_quantized_dtype \
            is torch.float8_e4m3fn


def test_normalize_shapes_and_messages():
    impl = B200AttentionBackendImpl(8, 64, 0.125, 2, None, None, "auto")
    x = torch.zeros(6, 8 * 64)
    assert backend.rows_by_user(x, "query", 8, 64, 3).shape == (3, 2, 8, 64)
    assert backend.rows_by_user(x.view(6, 8, 64), "query", 8, 64, 2).shape == (2, 3, 8, 64)
    with pytest.raises(ValueError, match="rank >= 2"):
        backend.rows_by_user(torch.zeros(5), "query", 8, 64, 1)
    with pytest.raises(ValueError, match="flattened-token tensor"):
        backend.rows_by_user(torch.zeros(6, 100), "key", 2, 64, 3)
    with pytest.raises(ValueError, match="divisible"):
        backend.rows_by_user(x, "query", 8, 64, 4)
    md = B200Metadata(num_users=3)
    ins = impl._prepare_inputs(x, torch.zeros(6, 2 * 64), torch.zeros(6, 2 * 64), md)
    assert ins.is_prefill and ins.query_num_tokens == 2 and ins.users == 3
    with pytest.raises(ValueError, match="key and value must match"):
        impl._prepare_inputs(x, torch.zeros(6, 2 * 64), torch.zeros(3, 2 * 64), md)


def test_forward_requires_metadata_and_output():
    impl = B200AttentionBackendImpl(8, 64, 0.125, 2, None, None, "auto")
    x = torch.zeros(2, 512)
    with pytest.raises(AssertionError, match="requires metadata"):
        impl.forward(None, x, x, x, None, None, output=x)
    with pytest.raises(AssertionError, match="output buffer"):
        impl.forward(None, x, x, x, None, B200Metadata(num_users=2), output=None)


def test_ops_refuse_cpu_tensors():
    kc = torch.zeros(4, 2, 32, 64, dtype=torch.bfloat16)
    q = torch.zeros(1, 8, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.paged_decode(q, kc, kc, torch.zeros(1, 4, dtype=torch.int32),
                         torch.zeros(1, dtype=torch.int32))


def test_varlen_metadata_from_vllm_fields():
    # 3 decode rows first (vLLM's order), then a 5-token chunk on a 64-token prefix and a fresh
    # 7-token prompt
    qsl = torch.tensor([0, 1, 2, 3, 8, 15], dtype=torch.int32)
    seq_lens = torch.tensor([10, 20, 30, 69, 7], dtype=torch.int32)
    md = backend.build_varlen_metadata(qsl, qsl.clone(), seq_lens,
                                       torch.zeros(5, 4, dtype=torch.int32),
                                       torch.arange(15, dtype=torch.int64), max_seq_len=69)
    assert md.is_varlen and md.num_decodes == 3 and md.num_users == 5
    assert md.decode_cur_pos.tolist() == [9, 19, 29]
    assert md.prefill_cu_q_cpu.tolist() == [0, 5, 12]
    assert md.prefill_q_start.tolist() == [64, 0]


def test_builder_returns_stub_without_varlen_fields():
    class Common:
        causal = True
    md = B200AttentionMetadataBuilder().build(0, Common())
    assert isinstance(md, B200Metadata) and md.cache_position is None and md.is_causal


def test_padding_rows_of_the_decode_position_buffer_read_minus_one():
    """A CUDA graph captured at a padded batch reads past this step's decode rows: a shrinking
    batch must leave -1 there, not an earlier step's positions."""
    buf = torch.full((8,), -1, dtype=torch.int32)
    bt = torch.zeros(8, 4, dtype=torch.int32)

    def step(seq_lens):
        n = len(seq_lens)
        qsl = torch.arange(n + 1, dtype=torch.int32)
        return backend.build_varlen_metadata(qsl, qsl.clone(), torch.tensor(seq_lens, dtype=torch.int32),
                                             bt[:n], torch.zeros(n, dtype=torch.int64),
                                             decode_cur_pos_buffer=buf)

    md = step([10, 20, 30, 40, 50])
    assert md.decode_cur_pos.tolist() == [9, 19, 29, 39, 49] and buf.tolist()[5:] == [-1, -1, -1]
    md = step([11, 21])
    assert md.decode_cur_pos.tolist() == [10, 20]
    assert buf.tolist() == [10, 20, -1, -1, -1, -1, -1, -1]


def test_allocate_kv_caches_per_rank_and_shared_layers():
    from b200attn import sharding

    caches = sharding.allocate_kv_caches(3, 16, 8, 64, 128, tp_size=4,
                                         shared_kv_layers={"layers.2.attn": "layers.0.attn"})
    assert list(caches) == ["layers.0.attn", "layers.1.attn", "layers.2.attn"]
    k, v = caches["layers.1.attn"]
    assert k.shape == v.shape == (16, 2, 64, 128) and k.dtype == torch.bfloat16
    assert k.data_ptr() != v.data_ptr() and float(k.abs().sum()) == 0
    assert caches["layers.2.attn"] is caches["layers.0.attn"]
    with pytest.raises(AssertionError, match="must be divisible by tp_size 3"):
        sharding.allocate_kv_caches(1, 16, 8, 64, 128, tp_size=3)
    with pytest.raises(ValueError, match="unknown layer"):
        sharding.allocate_kv_caches(["a"], 4, 8, 64, 128, shared_kv_layers={"b": "c"})
    f8 = sharding.allocate_kv_caches(["a"], 4, 8, 32, 128, dtype=torch.float8_e4m3fn)
    assert f8["a"][0].dtype == torch.float8_e4m3fn

    class Layer:
        kv_cache = None
    layers = {"layers.0.attn": Layer(), "other": Layer()}
    sharding.bind_kv_caches(layers, caches)
    assert layers["layers.0.attn"].kv_cache is caches["layers.0.attn"]
    assert layers["other"].kv_cache is None


def test_layer_wrapper_input_rules():
    """attention.py:798-825: rank >= 2, hidden-width or (heads, head_size) trailing dims."""
    assert backend.flatten_heads(torch.zeros(2, 3, 8, 64), "query", 8, 64).shape == (6, 512)
    assert backend.flatten_heads(torch.zeros(2, 3, 512), "query", 8, 64).shape == (6, 512)
    assert backend.flatten_heads(None, "key", 8, 64) is None
    with pytest.raises(ValueError, match="rank >= 2"):
        backend.flatten_heads(torch.zeros(512), "query", 8, 64)
    with pytest.raises(ValueError, match="must satisfy one of"):
        backend.flatten_heads(torch.zeros(4, 100), "value", 2, 64)
    layer = backend.B200Attention(8, 64, 0.125, num_kv_heads=2, sliding_window=128)
    assert layer.impl.num_kv_heads == 2 and layer.impl.sliding_window == 128
    with pytest.raises(TypeError, match="unexpected arguments"):
        backend.B200Attention(8, 64, 0.125, bogus=1)


def test_split_count_env_override(monkeypatch):
    """`B200ATTN_NUM_SPLITS` pins the split count of calls that leave it to the library."""
    from b200attn import ops

    monkeypatch.delenv("B200ATTN_NUM_SPLITS", raising=False)
    assert ops._env_num_splits() == 0
    monkeypatch.setenv("B200ATTN_NUM_SPLITS", "6")
    assert ops._env_num_splits() == 6
    monkeypatch.setenv("B200ATTN_NUM_SPLITS", "1000")
    with pytest.raises(ValueError):
        ops._env_num_splits()
