"""npz (de)serialisation of the golden vectors: bf16 tensors are stored as their int16 bit
patterns under `<name>__bf16`, everything else as plain numpy arrays."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.dirname(os.path.abspath(__file__))


def save_case(name: str, tensors: dict) -> str:
    arrays = {}
    for k, v in tensors.items():
        if isinstance(v, torch.Tensor):
            if v.dtype == torch.bfloat16:
                arrays[k + "__bf16"] = v.contiguous().view(torch.int16).numpy()
            else:
                arrays[k] = v.contiguous().numpy()
        else:
            arrays[k] = np.asarray(v)
    path = os.path.join(GOLDEN_DIR, name + ".npz")
    np.savez_compressed(path, **arrays)
    return path


def load_case(name: str) -> dict:
    out = {}
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        for k in z.files:
            a = torch.from_numpy(z[k].copy())
            if k.endswith("__bf16"):
                out[k[: -len("__bf16")]] = a.view(torch.bfloat16)
            else:
                out[k] = a
    return out


def list_cases(prefix: str = "") -> list[str]:
    return sorted(
        f[:-4] for f in os.listdir(GOLDEN_DIR) if f.endswith(".npz") and f.startswith(prefix)
    )
