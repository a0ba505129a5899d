"""torch.ops._moe_C.topk_softmax (vLLM's softmax top-k router: optional renormalisation, token_expert_indices, fp32 /
bf16 / f16 logits): the oracle against the golden vectors of the reference benchmark's own check, and the CUDA kernel
against the oracle (ids exact up to the float64-margin rule, weights to 1e-5)."""
import pytest
import torch

from oracle import compare as C
from oracle import ref_ops as R
from tests.golden_io import records


def test_oracle_renormalised_form_matches_the_benchmark_check(golden):
    recs = records(golden, "formula:benchmark/runners/mcoplib_mxbenchmark_topk_softmax_runners.py:38-49")
    assert len(recs) == 4
    for key, r in recs:
        w, ids, src = R.topk_softmax(r["gating"], int(r["k"]), True)
        C.assert_equal(ids, r["ids"], key)
        assert torch.allclose(w, r["weights"], rtol=1e-5, atol=1e-6), key
        n, k = ids.shape
        assert src[3 % n, k - 1] == (k - 1) * n + 3 % n


def test_oracle_unnormalised_weights_are_the_softmax_probabilities():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(40, 60, generator=g)
    w, ids, _ = R.topk_softmax(x, 6, False)
    p = torch.softmax(x, dim=-1)
    assert torch.allclose(w, torch.gather(p, 1, ids.long()), rtol=1e-5, atol=1e-7)
    w2, ids2, _ = R.topk_softmax(x, 6, True)
    assert torch.equal(ids, ids2) and torch.allclose(w2.sum(-1), torch.ones(40), atol=1e-5)
    assert torch.allclose(w2, R.moe_softmax_topk(x, 6)[0])


@pytest.mark.gpu
@pytest.mark.parametrize("n,E,k,dtype", [(1000, 8, 2, torch.float32), (333, 64, 6, torch.bfloat16), (64, 256, 8, torch.float16),
                                         (17, 60, 4, torch.float32), (9, 384, 8, torch.bfloat16), (5, 1024, 32, torch.float32),
                                         (262144, 8, 2, torch.float32)])
@pytest.mark.parametrize("renorm", [True, False])
def test_kernel_matches_oracle(n, E, k, dtype, renorm):
    import mcoplib_b200  # noqa: F401  (registers the torch library)
    from mcoplib_b200 import op
    from tests.gpu_util import DEV, Canary
    g = torch.Generator().manual_seed(n + E)
    x = torch.randn(n, E, generator=g).to(dtype)
    w_ref, ids_ref, src_ref = R.topk_softmax(x, k, renorm)
    w = Canary((n, k), torch.float32); ids = Canary((n, k), torch.int32); src = Canary((n, k), torch.int32)
    xd = x.to(DEV)
    if n % 2:   # both entry points: the pybind function and the torch-library operator
        op.topk_softmax(w.t, ids.t, src.t, xd, renorm)
    else:
        getattr(torch.ops, op.torch_moe_namespace).topk_softmax(w.t, ids.t, src.t, xd, renorm)
    torch.cuda.synchronize()
    w.check(); ids.check(); src.check()
    excused = C.assert_ids_with_margin(ids.t, ids_ref, R.softmax_topk_margin(x.float(), k), x.float().abs().amax(-1), "topk_softmax ids")
    assert excused <= max(2, n // 20000)
    same = (ids.t.cpu() == ids_ref).all(-1)
    C.assert_close(w.t.cpu()[same], w_ref[same], "topk_softmax weights", rel=1e-5, abs_=1e-7)
    C.assert_equal(src.t, src_ref, "token_expert_indices")


@pytest.mark.gpu
def test_rejects_wrong_dtypes():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    x = torch.randn(4, 16, device=DEV)
    w = torch.empty(4, 2, device=DEV); i = torch.empty(4, 2, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        op.topk_softmax(w, i, i.clone(), x.double(), True)
    with pytest.raises(RuntimeError):
        op.topk_softmax(w, i.long(), i.clone(), x, True)
