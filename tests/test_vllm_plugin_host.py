"""The vLLM adapter on a machine without a GPU: registration under the enum member the reference
uses (vllm_tt/__init__.py:10-17), the static backend contract, and the opt-in row-parallel hook
leaving single-rank layers alone."""
import pytest
import torch

vllm = pytest.importorskip("vllm")


def test_register_points_custom_at_this_backend(monkeypatch):
    from vllm.v1.attention.backends.registry import AttentionBackendEnum

    from b200attn import vllm_plugin

    monkeypatch.setenv("B200ATTN_FUSED_ROW_PARALLEL", "0")     # keep vLLM's linear layers as they are
    vllm_plugin.register()
    assert AttentionBackendEnum.CUSTOM.get_path() == "b200attn.vllm_plugin.B200VllmAttentionBackend"
    B = vllm_plugin.B200VllmAttentionBackend
    assert B.get_name() == "CUSTOM"
    assert B.get_impl_cls() is vllm_plugin.B200VllmAttentionImpl
    assert B.get_builder_cls() is vllm_plugin.B200VllmMetadataBuilder
    # one tensor per layer, halves = the plugin's separate K and V caches (attention.py:103-112)
    assert B.get_kv_cache_shape(100, 64, 8, 128) == (2, 100, 8, 64, 128)
    assert sorted(B.get_supported_kernel_block_sizes()) == [32, 64]
    assert sorted(B.get_supported_head_sizes()) == [64, 128]
    assert B.accept_output_buffer and B.forward_includes_kv_cache_update
    assert B.supported_kv_cache_dtypes == ["auto", "bfloat16"]


def test_impl_accepts_vllm_constructor_arguments():
    from b200attn import vllm_plugin

    impl = vllm_plugin.B200VllmAttentionImpl(32, 128, 0.088, num_kv_heads=8, sliding_window=1024,
                                             sinks=torch.zeros(32))
    assert impl.num_kv_heads == 8 and impl.sliding_window == 1024 and impl.sinks is not None
    # no metadata = vLLM's memory-profiling pass: zeros, no kernel
    out = torch.ones(4, 32 * 128)
    assert impl.forward(None, out, out, out, None, None, output=out).abs().sum() == 0
    with pytest.raises(NotImplementedError):
        vllm_plugin.B200VllmAttentionImpl(32, 128, 0.088, num_kv_heads=8, kv_cache_dtype="fp8_e5m2")


def test_fused_row_parallel_hook_is_idempotent_and_skips_single_rank_layers(monkeypatch):
    from vllm.model_executor.layers.linear import RowParallelLinear

    from b200attn import vllm_plugin

    original = RowParallelLinear.forward
    monkeypatch.setattr(RowParallelLinear, "forward", original)      # restored after the test
    monkeypatch.setattr(RowParallelLinear, "_b200attn_fused", False, raising=False)
    vllm_plugin.enable_fused_row_parallel()
    hooked = RowParallelLinear.forward
    assert hooked is not original and RowParallelLinear._b200attn_fused
    vllm_plugin.enable_fused_row_parallel()
    assert RowParallelLinear.forward is hooked

    # a single-rank layer must fall through to vLLM's own forward; the stand-in has nothing but
    # tp_size, so reaching vLLM's forward shows as the AttributeError it raises there
    import types

    with pytest.raises(AttributeError):
        hooked(types.SimpleNamespace(tp_size=1), torch.zeros(2, 8))


def test_register_enables_the_row_parallel_hook_by_mode(monkeypatch):
    """"auto" (the default) hooks groups of four ranks and more, "1" every tensor-parallel group,
    "0" none."""
    from b200attn import vllm_plugin

    seen = []
    monkeypatch.setattr(vllm_plugin, "enable_fused_row_parallel", lambda **kw: seen.append(kw))
    for mode, want in (("0", []), ("1", [dict(min_world=2)]), ("auto", [dict(min_world=4)]),
                       (None, [dict(min_world=4)])):
        seen.clear()
        if mode is None:
            monkeypatch.delenv("B200ATTN_FUSED_ROW_PARALLEL", raising=False)
        else:
            monkeypatch.setenv("B200ATTN_FUSED_ROW_PARALLEL", mode)
        vllm_plugin.register()
        assert seen == want, mode
