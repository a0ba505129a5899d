"""B200 (sm_100a) implementation of mcoplib's per-token inference hot path.

`mcoplib_b200.op` mirrors `mcoplib.op` (same function names, positional arguments and in-place
conventions) for the operators on the path; `mcoplib_b200.custom_ops` mirrors `mcoplib.custom_ops`;
the torch-library operators live under `torch.ops.<op.torch_namespace>` once `op` is imported.
Everything runs in hand-written CUDA kernels behind the C ABI of include/mcop_b200.h
(`libmcop_b200.so`, loadable on its own through `mcoplib_b200.cabi`).  There is no CPU fallback:
importing `op` without the built extension raises.
"""
import os as _os

import torch as _torch  # noqa: F401  (must be initialised before the extension module loads)

__version__ = "0.1.0"

PACKAGE_DIR = _os.path.dirname(_os.path.abspath(__file__))
LIBRARY_PATH = _os.path.join(PACKAGE_DIR, "libmcop_b200.so")


def _missing(name):
    raise ImportError(
        f"mcoplib_b200: native component '{name}' is not built. Run `python -m mcoplib_b200.build` "
        "(needs nvcc with sm_100a support); there is no fallback implementation.")


try:
    from . import op  # noqa: F401  (pybind11 + torch-library shims)
except ImportError as _e:  # pragma: no cover - exercised only on a broken install
    if not _os.path.exists(LIBRARY_PATH):
        _missing("libmcop_b200.so")
    raise
