"""CPU-side checks of the C-ABI library: it loads, exports every symbol that include/mcop_b200.h declares,
the ctypes binding agrees with the header, and argument validation rejects bad calls before any launch
(no kernel runs here)."""
import ctypes
import os
import re

import pytest

from mcoplib_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "mcop_b200.h")


def _declarations():
    hdr = open(HEADER).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    decls = {}
    for m in re.finditer(r"\b(mcop_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", hdr, re.S):
        args = [a for a in m.group(2).split(",") if a.strip() and a.strip() != "void"]
        decls[m.group(1)] = len(args)
    return decls


def test_library_exports_every_declared_symbol():
    decls = _declarations()
    assert len(decls) >= 20
    lib = ctypes.CDLL(cabi.LIBRARY_PATH)
    for name in decls:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_ctypes_binding_matches_header():
    decls = _declarations()
    assert set(decls) == set(cabi.SIGNATURES)
    for name, nargs in decls.items():
        assert len(cabi.SIGNATURES[name][1]) == nargs, name


def test_every_declaration_cites_the_reference():
    hdr = open(HEADER).read()
    for name in _declarations():
        if name in ("mcop_version", "mcop_last_error", "mcop_moe_scatter_workspace_bytes", "mcop_moe_gather_workspace_bytes"):
            continue
        pos = hdr.index(name + "(")
        comment = hdr[hdr.rfind("/*", 0, pos):pos]
        assert re.search(r"\.(cu|cuh|h|cpp)\b.*:\d+", comment, re.S) or "no reference counterpart" in comment.lower() \
            or "no counterpart in the reference" in comment.lower() \
            or "No single reference operator" in comment, f"{name}: no reference citation"


def test_version_and_workspace_queries():
    lib = cabi.load()
    assert lib.mcop_version() >= 100
    # header + [tiles, E] histogram + the larger of the bitmaps (16 words per tile and expert) and the per-slot ranks
    assert lib.mcop_moe_scatter_workspace_bytes(8192, 8, 256) == (64 + 16 * 256 + max(16 * 256 * 16, 8192 * 8)) * 4
    assert lib.mcop_moe_scatter_workspace_bytes(512, 1, 1024) == (64 + 1024 + max(1024 * 16, 512)) * 4
    assert lib.mcop_moe_gather_workspace_bytes(1000, 2000) == (1024 + 1000 * 2) * 4
    assert lib.mcop_moe_gather_workspace_bytes(0, 0) == 0


@pytest.mark.parametrize("call", [
    lambda lib: lib.mcop_add_rmsnorm_quant_i8(None, None, None, 0, None, None, None, 4, 64, 1e-6, 1, None),
    lambda lib: lib.mcop_add_rmsnorm_quant_i8(16, 16, 16, 8, 16, None, None, 4, 64, 1e-6, 1, None),   # row stride < hidden
    lambda lib: lib.mcop_moe_softmax_topk(16, 16, 16, 4, 8, 9, None),                                # k > experts
    lambda lib: lib.mcop_moe_softmax_topk(16, 16, 16, 4, 2048, 2, None),                             # too many experts
    lambda lib: lib.mcop_moe_gate_grouped_sigmoid(16, 16, 16, 16, None, 4, 250, 8, 4, 8, 1, 1.0, 0, 0, 0, 0, None),  # experts % 32
    lambda lib: lib.mcop_moe_gate_grouped_sigmoid(16, 16, 16, 16, None, 4, 256, 8, 1, 40, 1, 1.0, 0, 0, 0, 0, None),  # topk too large
    lambda lib: lib.mcop_moe_gate_grouped_sigmoid(16, 16, 16, 16, None, 4, 256, 8, 4, 9, 1, 1.0, 1, 0, 0, 0, None),  # shared expert with type 0
    lambda lib: lib.mcop_moe_gate_grouped_sigmoid(16, 16, 16, 16, None, 4, 256, 8, 4, 9, 1, 1.0, 2, 1, 0, 0, None),  # two shared experts
    lambda lib: lib.mcop_moe_gate_grouped_sigmoid(16, 16, 16, 16, None, 4, 256, 8, 4, 8, 1, 1.0, 0, 2, 0, 0, None),  # moegate_type 2
    lambda lib: lib.mcop_moe_scatter_quant_i8(16, 16, 16, 16, 16, 16, 16, 16, 16, None, 4, 64, 2, 8, None, 0, None),  # no workspace
    lambda lib: lib.mcop_moe_gather(16, 16, 16, None, 0, 4, 8, 64, None, 0, None),                   # no workspace, no tok2row
    lambda lib: lib.mcop_rope_inplace(16, 16, 16, 16, 1, 64, 4, 8, 2, 128, 130, 1024, 256, 128, 1, 1, None),  # rot_dim > head_size
    lambda lib: lib.mcop_rope_inplace(16, 16, 16, 16, 1, 0, 4, 8, 2, 128, 128, 1024, 256, 128, 1, 1, None),   # empty cos/sin table
    lambda lib: lib.mcop_reshape_and_cache(16, 16, 256, 256, 16, 16, 16, 4, 2, 128, 16, 7, 8, 2, None),        # head_size % x
    lambda lib: lib.mcop_silu_mul_quant_i8_masked_pack(16, 1, 16, 0, 18, 2, 4, 64, 256, None),                 # out_packed not 4-byte aligned
    lambda lib: lib.mcop_silu_mul_quant_i8_masked_pack(16, 1, 16, 0, 16, 2, 4, 64, 255, None),                 # odd record stride
    lambda lib: lib.mcop_selftest_wait_timeout(0, None),                                                      # limit out of range
    lambda lib: lib.mcop_rmsnorm(16, 16, 16, 16, None, 4, 64, 1e-6, 0, 1, 1, None),                  # after_res without residual
])
def test_bad_arguments_are_rejected_without_a_launch(call):
    lib = cabi.load()
    rc = call(lib)
    assert rc < 0
    assert len(cabi.last_error(lib)) > 0


def test_zero_tokens_is_a_no_op():
    lib = cabi.load()
    assert lib.mcop_moe_softmax_topk(16, 16, 16, 0, 8, 2, None) == 0
    assert lib.mcop_add_rmsnorm_quant_i8(16, 16, 16, 64, 16, None, None, 0, 64, 1e-6, 1, None) == 0


def test_op_module_refuses_cpu_tensors():
    import torch
    from mcoplib_b200 import op
    with pytest.raises(RuntimeError, match="CUDA"):
        op.moe_softmax_topk(torch.zeros(2, 2), torch.zeros(2, 2, dtype=torch.int32), torch.zeros(2, 8), False)
    with pytest.raises(RuntimeError, match="CUDA"):
        op.rms_norm_dynamic_per_token_quant_custom(torch.zeros(2, 8, dtype=torch.int8), torch.zeros(2, 8), torch.zeros(8),
                                                   torch.zeros(2, 1), 1e-6, None, None)
    assert op.torch_namespace == "mcop_C"
    assert hasattr(torch.ops.mcop_C, "rms_norm_dynamic_per_token_quant")
    assert hasattr(torch.ops.mcop_C_cache_ops, "reshape_and_cache_flash")
    assert hasattr(torch.ops.mcop_C_cache_ops, "reshape_and_cache")
