"""Loader for tests/golden/golden.npz (written by tests/golden/make_golden.py)."""
import os
from collections import defaultdict

import numpy as np
import torch

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz")


def load_golden():
    """Returns {record_key: {name: tensor-or-scalar}}; bf16/f16 arrays are re-viewed from their bits."""
    out = defaultdict(dict)
    with np.load(_PATH) as z:
        for full in z.files:
            key, name = full.rsplit("/", 1)
            arr = z[full]
            if name.endswith("#bf16"):
                val = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
                name = name[:-5]
            elif name.endswith("#f16"):
                val = torch.from_numpy(arr.view(np.int16).copy()).view(torch.float16)
                name = name[:-4]
            elif arr.ndim == 0:
                val = arr.item()
            else:
                val = torch.from_numpy(arr.copy())
            out[key][name] = val
    return dict(out)


def records(golden, prefix):
    return sorted((k, v) for k, v in golden.items() if k.startswith(prefix))
