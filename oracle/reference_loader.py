"""Imports the UNMODIFIED reference ops (python_package/tt_torch/custom_ops.py) and the
reference attention backend (vllm_tt/attention_impls/attention.py) on a machine where the
reference tree is mounted.  TEST INFRASTRUCTURE ONLY — see the package docstring.

The reference imports torch_xla at module level but only its `xla` branches call it; stub
modules stand in so that the `cpu` branches (the reference's own golden path,
tests/infra/testers/single_chip/op/op_tester.py:62-78) run.  Wrappers below loop the reference
op where its CPU branch is narrower than its device op:
  - GQA decode: per KV-head group (custom_ops.py:1259,1297 reshape `query` with the KV head
    count, so the CPU branch is MHA-only);
  - multi-user fill: per user (custom_ops.py:1044 reads `batch_idx.item()`).
The reference tree does not travel to the GPU machine; tests that need it skip there and rely
on the committed golden vectors.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import torch

REFERENCE_ROOT = os.environ.get("TT_XLA_REFERENCE_ROOT", os.path.join(os.sep, "root", "reference"))
_CUSTOM_OPS = os.path.join("python_package", "tt_torch", "custom_ops.py")
_ATTENTION = os.path.join(
    "integrations", "vllm_plugin", "vllm_tt", "attention_impls", "attention.py"
)

_state: dict = {}


def available() -> bool:
    return os.path.exists(os.path.join(REFERENCE_ROOT, _CUSTOM_OPS))


def _stub(name: str, **attrs) -> types.ModuleType:
    m = types.ModuleType(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    return m


def _no_xla(*a, **k):
    raise RuntimeError("the xla branch of a reference op is not available here")


def _load(name: str, path: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_ops():
    """Registers torch.ops.tt.* from the reference file; returns torch.ops.tt."""
    if "ops" in _state:
        return _state["ops"]
    if not available():
        raise RuntimeError(f"reference tree not found under {REFERENCE_ROOT}")
    if "torch_xla" not in sys.modules:
        tx = _stub("torch_xla")
        core = _stub("torch_xla.core")
        xb = _stub("torch_xla.core.xla_builder")
        ex = _stub("torch_xla.experimental")
        sc = _stub("torch_xla.experimental.stablehlo_custom_call", stablehlo_custom_call=_no_xla)
        lib = torch.library.Library("xla", "DEF")
        lib.define(
            "mark_tensor(Tensor x, str name, int pos, str id, bool is_input, Any? attr=None) "
            "-> Tensor"
        )
        ck = _stub("torch_xla.experimental.custom_kernel", XLA_LIB=lib)
        tx.core, core.xla_builder = core, xb
        tx.experimental, ex.stablehlo_custom_call, ex.custom_kernel = ex, sc, ck
        _state["xla_lib"] = lib
    pkg = _stub("tt_torch")
    pkg.__path__ = []
    mod = _load("tt_torch.custom_ops", os.path.join(REFERENCE_ROOT, _CUSTOM_OPS))
    pkg.custom_ops = mod
    _state["ops"] = torch.ops.tt
    return _state["ops"]


def load_attention():
    """Imports the reference attention.py (needs vllm importable); returns the module."""
    if "attention" in _state:
        return _state["attention"]
    load_ops()
    os.environ.setdefault("VLLM_TARGET_DEVICE", "empty")
    root = os.path.join(REFERENCE_ROOT, "integrations", "vllm_plugin", "vllm_tt")
    pkg = _stub("vllm_tt")
    pkg.__path__ = [root]
    sub = _stub("vllm_tt.attention_impls")
    sub.__path__ = [os.path.join(root, "attention_impls")]
    _load("vllm_tt.logger", os.path.join(root, "logger.py"))
    _state["attention"] = _load(
        "vllm_tt.attention_impls.attention", os.path.join(REFERENCE_ROOT, _ATTENTION)
    )
    return _state["attention"]


# ------------------------------------------------------------------ wrappers over the live ops
def ref_paged_update_cache(cache, fill_value, update_indices, page_table):
    return load_ops().paged_update_cache(cache, fill_value, update_indices, page_table)


def ref_paged_fill_cache(cache, fill_value, page_table, batch_idx=None):
    """fill_value [users,nkv,T,hd]; loops the single-user reference op over the users."""
    ops = load_ops()
    users = fill_value.shape[0]
    if batch_idx is None:
        batch_idx = torch.arange(users, dtype=torch.int32)
    for u in range(users):
        cache = ops.paged_fill_cache(
            cache, fill_value[u:u + 1], page_table, batch_idx=batch_idx[u:u + 1]
        )
    return cache


def ref_paged_decode(query, k_cache, v_cache, page_table, cur_pos, scale):
    """query [1,users,nq,hd]; loops the MHA-only reference op over the KV-head groups."""
    ops = load_ops()
    nq, nkv = query.shape[2], k_cache.shape[1]
    G = nq // nkv
    outs = []
    for h in range(nkv):
        qg = query[:, :, h * G:(h + 1) * G, :].contiguous()
        kg = k_cache[:, h:h + 1].expand(-1, G, -1, -1).contiguous()
        vg = v_cache[:, h:h + 1].expand(-1, G, -1, -1).contiguous()
        outs.append(
            ops.paged_scaled_dot_product_attention_decode(
                qg, kg, vg, page_table, is_causal=True, cur_pos_tensor=cur_pos, scale=scale
            )
        )
    return torch.cat(outs, dim=2)


def ref_paged_decode_mla_branch(query, k_cache, v_cache, page_table, cur_pos, scale):
    """Cross-check through `tt.paged_flash_mla_decode`'s CPU branch, which handles GQA natively
    (custom_ops.py:551-610)."""
    ops = load_ops()
    return ops.paged_flash_mla_decode(
        query, k_cache, query.shape[-1], page_table, value=v_cache, is_causal=True,
        cur_pos_tensor=cur_pos, scale=scale,
    )


def ref_sdpa(query, key, value, scale):
    return load_ops().scaled_dot_product_attention(query, key, value, is_causal=True, scale=scale)


def ref_chunked_sdpa(query, k_cache, v_cache, page_table, chunk_start, scale):
    return load_ops().chunked_scaled_dot_product_attention(
        query, k_cache, v_cache, page_table,
        torch.tensor([chunk_start], dtype=torch.int32), scale=scale,
    )


def ref_rotary(positions, query, key, head_size, rotary_dim, base=500000.0, max_position=8192):
    """The reference rotary layer (vllm_tt/layers/rotary_embedding.py) wrapped around vLLM's
    RotaryEmbedding, on CPU.  Returns (rotated query, rotated key, inv_freq)."""
    from vllm.config import DeviceConfig, VllmConfig, set_current_vllm_config
    from vllm.model_executor.layers.rotary_embedding.base import RotaryEmbedding

    path = os.path.join(REFERENCE_ROOT, "integrations", "vllm_plugin", "vllm_tt", "layers",
                        "rotary_embedding.py")
    mod = _state.get("rotary") or _load("vllm_tt_layers_rotary_embedding", path)
    _state["rotary"] = mod
    with set_current_vllm_config(VllmConfig(device_config=DeviceConfig(device="cpu"))):
        layer = RotaryEmbedding(head_size=head_size, rotary_dim=rotary_dim,
                                max_position_embeddings=max_position, base=base,
                                is_neox_style=True, dtype=query.dtype)
    tt = mod.TTRotaryEmbedding(layer)
    q, k = tt(positions, query, key)
    return q, k, tt.inv_freq.clone()


def load_swa_utils():
    """The reference's sliding-window ring helpers (vllm_tt/swa_cache_utils.py: pure ints/numpy)."""
    if "swa" not in _state:
        if not available():
            raise RuntimeError(f"reference tree not found under {REFERENCE_ROOT}")
        path = os.path.join(REFERENCE_ROOT, "integrations", "vllm_plugin", "vllm_tt",
                            "swa_cache_utils.py")
        _state["swa"] = _load("vllm_tt_swa_cache_utils", path)
    return _state["swa"]
