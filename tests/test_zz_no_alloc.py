"""The allocation-free gather entry point, mcop_moe_gather_noalloc.

Some hosts of this library cannot give it scratch memory: a plugin loaded into a serving engine that has
already handed the whole device to its own memory pool, a plain C program that was only given input and
output buffers, a latency-critical loop that must not run into the device synchronisation an allocation
implies.  For them the library keeps a fixed 4 MiB table of its own and `mcop_moe_gather_noalloc` uses it
instead of a caller workspace.  This test calls it through the C ABI (ctypes, raw device pointers) and checks
that it writes exactly what the workspace-taking `mcop_moe_gather` writes - and what the CPU oracle computes - on two
calls in a row of different shapes (the table keeps the first call's contents, which must not leak into the second), and that a problem
too large for the table is refused before anything runs.

The file name sorts last so that a run which stops at the first failure has already executed every other test.
"""
import pytest
import torch

from mcoplib_b200 import cabi
from oracle import ref_ops as R

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _inputs(tokens, rows, hidden, seed):
    g = torch.Generator().manual_seed(seed)
    y = torch.randn(rows, hidden, generator=g).bfloat16().to(DEV)
    out0 = torch.randn(tokens, hidden, generator=g).bfloat16().to(DEV)
    # an arbitrary row -> token map: uneven counts, one token with no row, two entries that must be skipped
    r2t = torch.randint(0, tokens, (rows,), generator=g).to(torch.int32)
    r2t[r2t == 3] = 4
    r2t[0] = -1
    r2t[rows - 1] = tokens + 7
    return y, r2t.to(DEV), out0


def _with_workspace(lib, y, r2t, out0, tokens, rows, hidden, stream):
    out = out0.clone()
    nbytes = lib.mcop_moe_gather_workspace_bytes(tokens, rows)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    cabi.check(lib.mcop_moe_gather(y.data_ptr(), r2t.data_ptr(), out.data_ptr(), None, 0, tokens, rows, hidden,
                                   ws.data_ptr(), ws.numel(), stream), lib)
    return out


def _without_allocation(lib, y, r2t, out0, tokens, rows, hidden, stream):
    out = out0.clone()
    cabi.check(lib.mcop_moe_gather_noalloc(y.data_ptr(), r2t.data_ptr(), out.data_ptr(), tokens, rows, hidden, stream), lib)
    return out


def test_noalloc_gather_equals_workspace_gather_on_two_calls_in_a_row():
    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    # first a larger problem (takes the pipelined kernel), then a smaller one with fewer tokens and a different
    # rows-per-token ratio, so that stale counters or row lists from call one would corrupt call two
    for tokens, rows, hidden, seed in [(1500, 6000, 4096, 1), (300, 2100, 1024, 2)]:
        y, r2t, out0 = _inputs(tokens, rows, hidden, seed)
        expect = _with_workspace(lib, y, r2t, out0, tokens, rows, hidden, stream)
        got = _without_allocation(lib, y, r2t, out0, tokens, rows, hidden, stream)
        torch.cuda.synchronize()
        # integer-exact: both run the same kernels, only the home of the scratch table differs
        assert torch.equal(got.view(torch.int16), expect.view(torch.int16)), (tokens, rows, hidden)
        # and both are what the CPU oracle computes: fp32 sum in ascending row order, one rounding, bad entries skipped
        oracle = R.moe_gather(y.cpu(), r2t.cpu(), out0.cpu())
        assert torch.equal(got.cpu().view(torch.int16), oracle.view(torch.int16)), (tokens, rows, hidden)
        assert torch.equal(got[3].view(torch.int16), out0[3].view(torch.int16)), "a token without rows keeps its value"
        assert not torch.equal(got, out0)
    assert lib.mcop_device_error() == 0


def test_noalloc_gather_refuses_what_does_not_fit():
    lib = cabi.load()
    tokens, rows = 1 << 20, 1 << 21      # needs ~12 MiB of table
    assert lib.mcop_moe_gather_workspace_bytes(tokens, rows) > cabi.GATHER_NOALLOC_SCRATCH_BYTES
    dummy = torch.zeros(16, dtype=torch.int32, device=DEV)   # never dereferenced: the call is rejected first
    rc = lib.mcop_moe_gather_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), tokens, rows, 64,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    assert "built-in area" in cabi.last_error(lib)
    # the largest advertised case fits
    assert lib.mcop_moe_gather_workspace_bytes(65536, 65536 * 8) <= cabi.GATHER_NOALLOC_SCRATCH_BYTES
