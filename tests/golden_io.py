"""Reader for the golden vectors in tests/golden/ (written by make_golden.py)."""
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def dtype_of(name) -> torch.dtype:
    return _DT[str(name)]


def tensor(arr: np.ndarray, dtype: torch.dtype = None) -> torch.Tensor:
    """numpy array of raw bits -> torch tensor (uint16 payloads become fp16/bf16)."""
    if arr.dtype == np.uint16:
        assert dtype in (torch.float16, torch.bfloat16)
        return torch.from_numpy(arr.view(np.int16).copy()).view(dtype)
    return torch.from_numpy(arr.copy())


def load(fname: str) -> dict:
    """{case name: {field: numpy array}}"""
    z = np.load(os.path.join(GOLDEN_DIR, fname))
    cases = {}
    for key in z.files:
        case, field = key.split("/")
        cases.setdefault(case, {})[field] = z[key]
    return cases
