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
    assert B.supported_kv_cache_dtypes == ["auto", "bfloat16", "fp8", "fp8_e4m3"]


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


def _unhook(monkeypatch):
    from vllm.model_executor.layers.linear import RowParallelLinear

    from b200attn import ops

    monkeypatch.setattr(RowParallelLinear, "forward", RowParallelLinear.forward)
    monkeypatch.setattr(RowParallelLinear, "__init__", RowParallelLinear.__init__)
    monkeypatch.setattr(RowParallelLinear, "_b200attn_fused", False, raising=False)
    monkeypatch.setattr(ops.ErrorWordWatch, "on_error", [])
    return RowParallelLinear


def test_fused_row_parallel_hook_is_idempotent_and_skips_ineligible_layers(monkeypatch):
    import types

    from b200attn import vllm_plugin

    RowParallelLinear = _unhook(monkeypatch)
    original = RowParallelLinear.forward
    vllm_plugin.enable_fused_row_parallel()
    hooked = RowParallelLinear.forward
    assert hooked is not original and RowParallelLinear._b200attn_fused
    vllm_plugin.enable_fused_row_parallel()
    assert RowParallelLinear.forward is hooked

    # A single-rank layer, and a layer built outside an engine that selected this backend, must
    # fall through to vLLM's own forward; the stand-ins have nothing but the fields the hook
    # reads first, so reaching vLLM's forward shows as the AttributeError it raises there.
    with pytest.raises(AttributeError):
        hooked(types.SimpleNamespace(tp_size=1, _b200attn_fusable=True), torch.zeros(2, 8))
    with pytest.raises(AttributeError):
        hooked(types.SimpleNamespace(tp_size=8), torch.zeros(2, 8))


def test_hook_switches_itself_off_when_the_diagnostics_watch_reports(monkeypatch):
    """A wait that ran out (word 1) must not pass silently: the per-step watch raises, and the
    fused path is off from then on."""
    from b200attn import ops, vllm_plugin

    RowParallelLinear = _unhook(monkeypatch)
    vllm_plugin.enable_fused_row_parallel()
    state = RowParallelLinear._b200attn_state
    assert state["off"] is False
    watch = ops.ErrorWordWatch(torch.device("cpu"))       # host-side stand-in: no device copy
    watch._host[0] = 1                                    # what an earlier step's copy found
    with pytest.raises(RuntimeError, match="bounded wait"):
        watch.poll()
    assert state["off"] is True and watch.value() == 0
    watch._host[0] = 2
    with pytest.raises(RuntimeError, match="outside the KV cache"):
        watch.poll()


def test_config_guard():
    import types

    from b200attn.vllm_plugin import config_allows_fused_row_parallel as allows

    def cfg(backend, mode):
        return types.SimpleNamespace(
            attention_config=types.SimpleNamespace(backend=types.SimpleNamespace(name=backend)),
            compilation_config=types.SimpleNamespace(mode=mode))

    assert allows(cfg("CUSTOM", 0)) == (True, "ok")
    assert not allows(None)[0]
    assert not allows(cfg("FLASHINFER", 0))[0]
    ok, why = allows(cfg("CUSTOM", 3))
    assert not ok and "torch.compile" in why


def test_rank_guard():
    from b200attn.vllm_plugin import ranks_allow_fused_row_parallel as allows

    def ranks(n, host="a", major=10):
        return [dict(host=host, device=i, major=major) for i in range(n)]

    yes = lambda a, b: True
    assert allows(ranks(4), yes) == (True, "ok")
    assert not allows(ranks(1), yes)[0]
    assert not allows(ranks(2, major=9), yes)[0]
    two_nodes = ranks(2) + ranks(2, host="b")
    assert "more than one node" in allows(two_nodes, yes)[1]
    assert "share one GPU" in allows([dict(host="a", device=0, major=10)] * 2, yes)[1]
    assert "cannot access" in allows(ranks(4), lambda a, b: (a, b) != (1, 3))[1]


def test_register_enables_the_row_parallel_hook_only_on_request(monkeypatch):
    """Off unless asked for: "1" hooks every tensor-parallel group, a larger number groups of at
    least that many ranks."""
    from b200attn import vllm_plugin

    seen = []
    monkeypatch.setattr(vllm_plugin, "enable_fused_row_parallel", lambda **kw: seen.append(kw))
    for mode, want in ((None, []), ("0", []), ("auto", []), ("1", [dict(min_world=2)]),
                       ("4", [dict(min_world=4)])):
        seen.clear()
        if mode is None:
            monkeypatch.delenv("B200ATTN_FUSED_ROW_PARALLEL", raising=False)
        else:
            monkeypatch.setenv("B200ATTN_FUSED_ROW_PARALLEL", mode)
        vllm_plugin.register()
        assert seen == want, mode
