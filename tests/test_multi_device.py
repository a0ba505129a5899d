"""One process driving two GPUs: the per-device state of the library (shared-memory attribute of the pipelined kernels,
error word, SM count, built-in scratch) must exist on every device that is used, not only on the first one."""
import pytest
import torch

from mcoplib_b200 import workloads as W
from oracle import compare as C
from oracle import ref_ops as R


@pytest.mark.gpu
def test_pipelined_kernels_run_on_a_second_device():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from mcoplib_b200 import op
    T, H, E, k = 4096, 7168, 8, 2
    d = W.norm_quant_inputs(T, H)
    q_ref, s_ref, res_ref = R.rms_norm_dynamic_per_token_quant(d["x"], d["weight"], 1e-6, residual=d["residual"])
    logits = W.router_inputs(T, E)["logits"]
    w_ref, ids_ref = R.moe_softmax_topk(logits, k)
    dd = W.dispatch_inputs(T, H, E, k, with_hidden=False)
    for dev in (0, 1, 0):
        device = torch.device("cuda", dev)
        with torch.cuda.device(dev):
            x, res, w = d["x"].to(device), d["residual"].to(device), d["weight"].to(device)
            codes = torch.empty(T, H, dtype=torch.int8, device=device)
            scales = torch.empty(T, 1, device=device)
            op.rms_norm_dynamic_per_token_quant_custom(codes, x, w, scales, 1e-6, None, res)
            C.assert_codes(codes, q_ref, f"norm codes on cuda:{dev}")
            tw = torch.empty(T, k, device=device); ti = torch.empty(T, k, dtype=torch.int32, device=device)
            op.moe_softmax_topk(tw, ti, logits.to(device), False)
            rows = torch.empty(T * k, H, dtype=torch.int8, device=device)
            rs = torch.empty(T * k, device=device); r2t = torch.empty(T * k, dtype=torch.int32, device=device)
            cnt = torch.empty(E, dtype=torch.int32, device=device); st = torch.empty(E, dtype=torch.int32, device=device)
            t2r = torch.empty(T, k, dtype=torch.int32, device=device)
            op.moe_scatter_dynamic_quant(x, ti, tw, dd["smooth"].to(device), rows, rs, r2t, cnt, st, E, 0, 0, t2r)
            out = torch.empty(T, H, dtype=torch.bfloat16, device=device)
            op.moe_gather_weighted(dd["y"].to(device), r2t, ti, tw, st, out, False, t2r)
            torch.cuda.synchronize(dev)
            rows_ref, rs_ref, r2t_ref, cnt_ref, st_ref, _ = R.moe_scatter_dynamic_quant(d["x"], ti.cpu(), tw.cpu(), dd["smooth"], E)
            C.assert_equal(r2t, r2t_ref, f"row2tok on cuda:{dev}")
            C.assert_codes(rows, rows_ref, f"scatter rows on cuda:{dev}")
            out_ref = R.moe_gather_weighted(dd["y"], r2t_ref, ti.cpu(), tw.cpu(), st_ref, torch.empty(T, H, dtype=torch.bfloat16), False)
            assert torch.equal(out.cpu(), out_ref), f"gather on cuda:{dev}"
