"""MCOP_DEBUG_TRACE / MCOP_DEBUG_PARAMS_DUMP of the operator shims (the reference's debug aids,
common/mcoplib_ops_params_info.hpp and common/mcoplib_ops_params_dump.hpp).  The environment is read once per
process, so every case runs in a child process; CPU tensors are enough because the trace is the first statement of
a shim (the operator itself then refuses the CPU tensors, as it should)."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import sys
    sys.path.insert(0, %r)
    import torch
    from mcoplib_b200 import op
    x = torch.arange(40, dtype=torch.float32).reshape(4, 10)
    w = torch.zeros(4, 2); i = torch.arange(8, dtype=torch.int32).reshape(4, 2)
    try:
        op.moe_softmax_topk(w, i, x, True)
    except RuntimeError as e:
        print("raised:", str(e).splitlines()[0])
    try:
        op.rms_norm(torch.zeros(2, 8, dtype=torch.bfloat16), torch.ones(2, 8, dtype=torch.bfloat16),
                    torch.ones(8, dtype=torch.bfloat16), 1e-6, None, None, False)
    except RuntimeError as e:
        print("raised:", str(e).splitlines()[0])
""") % ROOT


def _run(tmp_path, **env):
    e = {k: v for k, v in os.environ.items() if not k.startswith("MCOP_")}
    e.update(env)
    r = subprocess.run([sys.executable, "-c", CHILD], cwd=tmp_path, env=e, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    return r.stdout


def test_silent_by_default(tmp_path):
    out = _run(tmp_path)
    assert "[MCOP_DEBUG]" not in out and out.count("raised:") == 2
    assert not list(tmp_path.glob("*.json"))


def test_trace_prints_the_call_and_every_argument(tmp_path):
    out = _run(tmp_path, MCOP_DEBUG_TRACE="1")
    assert "[MCOP_DEBUG] Call: moe_softmax_topk\n" in out
    assert "  topk_weights = Tensor(Shape=[4, 2], Dtype=Float, Device=cpu),\n" in out
    assert "  gating_output = Tensor(Shape=[4, 10], Dtype=Float, Device=cpu),\n" in out
    assert "  pre_softmax = 1\n" in out
    assert "[MCOP_DEBUG] Call: rms_norm\n" in out and "  after_res = Optional(nullopt),\n" in out and "  rms_div = 0\n" in out
    # the trace comes before the operator's own argument checks
    assert out.index("Call: moe_softmax_topk") < out.index("raised: gating_output must be a CUDA tensor")
    assert not list(tmp_path.glob("*.json"))
    assert "[MCOP_DEBUG]" in _run(tmp_path, MCOP_DEBUG_TRACE="ON") and "[MCOP_DEBUG]" not in _run(tmp_path, MCOP_DEBUG_TRACE="0")


def test_dump_writes_one_json_file_per_operator(tmp_path):
    out = _run(tmp_path, MCOP_DEBUG_PARAMS_DUMP="1", MCOP_TENSOR_DUMP_SAMPLE_SIZE="3")
    assert "[MCOP_DEBUG]" not in out
    d = json.loads((tmp_path / "moe_softmax_topk.json").read_text())
    assert d["function"] == "moe_softmax_topk"
    p = {q["name"]: q for q in d["parameters"]}
    assert list(p) == ["topk_weights", "topk_indices", "gating_output", "pre_softmax"]
    assert p["gating_output"] == {"name": "gating_output", "type": "at::Tensor", "dtype": "Float", "shape": "[4, 10]",
                                  "value": "[0, 1, 2, ..., 37, 38, 39]", "bytes": 160}
    assert p["topk_indices"]["value"] == "[0, 1, 2, ..., 5, 6, 7]" and p["topk_indices"]["dtype"] == "Int"
    assert p["pre_softmax"]["value"] == "1" and p["pre_softmax"]["type"] == "bool"
    r = {q["name"]: q for q in json.loads((tmp_path / "rms_norm.json").read_text())["parameters"]}
    assert r["after_res"]["value"] == "nullopt" and r["weight"]["value"] == "[1, 1, 1, ..., 1, 1, 1]"


def test_dump_of_all_values(tmp_path):
    _run(tmp_path, MCOP_DEBUG_PARAMS_DUMP="1", MCOP_TENSOR_DUMP_FULL="1")
    d = json.loads((tmp_path / "moe_softmax_topk.json").read_text())
    v = {q["name"]: q for q in d["parameters"]}["gating_output"]["value"]
    assert v == "[" + ", ".join(str(i) for i in range(40)) + "]"
