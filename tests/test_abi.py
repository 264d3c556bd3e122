"""The C-ABI library builds, loads without a GPU and exports every symbol the header declares.
No compute runs here."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200attn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("b200attn_paged_update_cache", "b200attn_paged_fill_cache",
                 "b200attn_kv_scatter_slots", "b200attn_paged_decode", "b200attn_prefill"):
        assert must in names


def test_library_exports_every_declared_symbol(built_library):
    handle = ctypes.CDLL(built_library)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in b200attn.h but not exported"


def test_binding_covers_every_declared_symbol(built_library):
    from b200attn import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()
    L = _lib.lib()
    assert L.b200attn_version() == 100
    assert L.b200attn_status_string(0) == b"ok"
    assert b"CPU" in L.b200attn_status_string(-6)


def test_argument_errors_are_detected_on_the_host(built_library):
    from b200attn import _lib

    L = _lib.lib()
    # unsupported head size: rejected before any device work
    rc = L.b200attn_kv_scatter_slots(16, 16, 16, 16, 96 * 2, 16, 1, 2, 96, 32, 4, None)
    assert rc == -2
    rc = L.b200attn_paged_decode(None, 0, None, 0, None, None, None, 0, 1, None, 1, 8, 8, 64, 32,
                                 4, 1.0, 0, 0, None, 0, None)
    assert rc == -1
    assert L.b200attn_decode_workspace_bytes(8, 32, 64, 1) == 0
    assert L.b200attn_decode_workspace_bytes(8, 32, 64, 4) >= 8 * 32 * 4 * (64 * 4 + 8)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_compute_entry_points_fail_loudly_without_a_device(built_library):
    from b200attn import _lib, ops

    L = _lib.lib()
    rc = L.b200attn_kv_scatter_slots(16, 16, 16, 16, 128, 16, 1, 2, 64, 32, 4, None)
    assert rc == -6  # B200ATTN_ERR_NO_DEVICE: no silent fallback
    kc = torch.zeros(4, 2, 32, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.kv_scatter_slots(kc, kc.clone(), torch.zeros(1, 2, 64, dtype=torch.bfloat16),
                             torch.zeros(1, 2, 64, dtype=torch.bfloat16),
                             torch.zeros(1, dtype=torch.int64))
