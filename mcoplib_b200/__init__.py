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


_OP_NAME = "op" + (__import__("sysconfig").get_config_var("EXT_SUFFIX") or ".so")


def __getattr__(name):
    # `op` (the pybind11 + torch-library shims over libmcop_b200.so) is loaded on first use, not at package import:
    # the helper modules (workloads, sharding, perf_csv) are plain Python and a process that only wants them - the CPU
    # baseline of the benchmark, for one - must not map the native libraries.  `import mcoplib_b200.op` and
    # `from mcoplib_b200 import op` both end up here or in the regular submodule import.
    if name == "op":
        if not (_os.path.exists(LIBRARY_PATH) and _os.path.exists(_os.path.join(PACKAGE_DIR, _OP_NAME))):
            _missing("libmcop_b200.so" if not _os.path.exists(LIBRARY_PATH) else _OP_NAME)
        import importlib
        return importlib.import_module(".op", __name__)   # registers torch.ops.<namespace>.* as a side effect
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
