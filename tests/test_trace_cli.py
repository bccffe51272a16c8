"""The inline-expression tracer and the ``compile`` / ``run`` command line.

CPU part: the tracer must produce, for the expressions the golden fixtures were generated from, the same Torch-IR
records the reference's tracer produced (``tests/golden/graphs/*.json``, written by ``tests/golden/make_golden.py``
through ``emmy/commands/trace.py:114`` ``graph_from_code``); ``compile`` prints one launch per op; the accuracy rule is
the reference's (``emmy/commands/run.py:1452-1491``). GPU part: ``run -c`` end to end, exit code 0 iff PASS.
"""

from __future__ import annotations

import importlib.util
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from deplodock_b200.__main__ import accuracy_verdict, main, render_table
from deplodock_b200.backend import B200Backend, LoweringError
from deplodock_b200.trace import bind_inputs, graph_from_code, trace_inline_code

GOLDEN = Path(__file__).parent / "golden"


def _golden_codes() -> dict[str, str]:
    spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return {**mod.CASES, **mod.RECORD_ONLY}


CODES = _golden_codes()
_KERNEL_OPS = {"RmsNormOp", "SoftmaxOp", "LinearOp", "MatmulOp", "SdpaOp"}


@pytest.mark.parametrize("name", list(CODES))
def test_tracer_matches_reference_records(name):
    ref = json.loads((GOLDEN / "graphs" / f"{name}.json").read_text())
    got = trace_inline_code(CODES[name]).graph.to_dict()
    assert got["inputs"] == ref["inputs"]
    assert got["outputs"] == ref["outputs"]

    def essentials(d):
        out = {}
        for nid, n in d["nodes"].items():
            if n["op"] in _KERNEL_OPS or n["op"] in ("InputOp", "ElementwiseOp") or (
                    n["op"] == "ConstantOp" and n["op_fields"].get("source_path")):
                fields = {k: v for k, v in n["op_fields"].items() if k in ("eps", "axis", "is_causal", "has_bias",
                                                                           "source_path", "op")}
                out[nid] = (n["op"], fields, n["inputs"], n["output"]["shape"], n["output"]["dtype"])
        return out

    assert essentials(got) == essentials(ref)


def test_perf_suite_expressions_lower_to_gemms_and_one_pointwise_launch():
    """The expressions the reference's perf suite drives (``tests/perf/cases.py:60-74``)."""
    g, _, _ = graph_from_code(CODES["swiglu_f32"])
    assert {n.op for n in g.nodes.values()} == {"InputOp", "MatmulOp", "ElementwiseOp"}
    plan = B200Backend().compile(g)
    assert [s.entry for s in plan.steps] == ["emk_linear_f32_simt", "emk_linear_f32_simt", "emk_elementwise"]
    assert plan.steps[2].attrs["op"] == "silu_multiply"
    # bf16 matmul + residual: the add becomes the GEMM's residual epilogue
    plan = B200Backend().compile(trace_inline_code(
        "x=torch.randn(16,64).bfloat16(); w=torch.randn(64,96).bfloat16(); r=torch.randn(16,96).bfloat16(); "
        "torch.matmul(x,w)+r").graph)
    assert [s.entry for s in plan.steps] == ["emk_linear_bf16"] and plan.steps[0].attrs["residual"]
    assert plan.aliases["add"] == "matmul"
    # fp32: GEMM then a pointwise add
    plan = B200Backend().compile(trace_inline_code(
        "x=torch.randn(16,64); w=torch.randn(64,96); r=torch.randn(16,96); torch.matmul(x,w)+r").graph)
    assert [s.entry for s in plan.steps] == ["emk_linear_f32_simt", "emk_elementwise"]
    # broadcasting adds have no kernel
    with pytest.raises(LoweringError):
        B200Backend().compile(trace_inline_code("torch.matmul(torch.randn(4,8), torch.randn(8,4)) + torch.randn(4)").graph)


def test_grammar_errors():
    with pytest.raises(ValueError, match="must end with an expression"):
        trace_inline_code("x = torch.randn(4)")
    with pytest.raises(ValueError, match="no tensor inputs"):
        trace_inline_code("1 + 2")


def test_module_fast_path_and_binding():
    tr = trace_inline_code("m = nn.Linear(16, 8); m(torch.randn(4, 16))")
    assert isinstance(tr.module, torch.nn.Linear)
    data = bind_inputs(tr.graph, tr.module, tr.args, tr.kwargs, tr.const_sources)
    assert set(data) == set(tr.graph.inputs) | {"p_weight", "p_bias"}
    assert data["p_weight"].shape == (8, 16)
    assert tr.slug == "m"


def test_wrapper_path_names_inputs():
    tr = trace_inline_code("q=torch.randn(1,2,8,16); F.scaled_dot_product_attention(q, q, torch.randn(1,2,8,16))")
    assert tr.graph.inputs == ["q", "x"]
    tr = trace_inline_code("torch.matmul(torch.randn(4, 8), torch.randn(8, 4))")
    assert tr.graph.inputs == ["x0", "x1"]
    tr = trace_inline_code("x=torch.randn(4, 8); torch.matmul(x, torch.randn(8, 4))")
    assert tr.graph.inputs == ["x", "x_"]


def test_casts_alias_their_input():
    plan = B200Backend().compile(trace_inline_code(
        "torch.softmax(torch.randn(4, 8).contiguous().to(torch.float32).reshape(2, 16), dim=-1)").graph)
    assert [s.entry for s in plan.steps] == ["emk_softmax_lastdim"]


def test_compile_cli_prints_plan(capsys):
    assert main(["compile", "-c", CODES["cfg3_linear_bf16"]]) == 0
    out = capsys.readouterr().out
    assert "emk_linear_bf16" in out and "k_linear_" in out
    assert main(["compile", str(GOLDEN / "graphs" / "cfg4_sdpa_bf16.json")]) == 0
    assert "emk_sdpa_causal_gqa_bf16" in capsys.readouterr().out
    assert main(["compile", "--ir", "torch", "-c", CODES["softmax_f32"]]) == 0
    rec = json.loads(capsys.readouterr().out)
    assert rec["nodes"]["softmax"]["op"] == "SoftmaxOp"


def test_dump_dir_writes_rerunnable_per_kernel_records(tmp_path, capsys):
    """``compile --dump-dir`` leaves one stand-alone Torch-IR record per launch; each compiles back to the same entry."""
    from deplodock_b200.graph import Graph

    code = "m = nn.Linear(64, 96, bias=True); torch.softmax(m(torch.randn(8, 64)), dim=-1)"
    assert main(["compile", "-c", code, "--dump-dir", str(tmp_path)]) == 0
    plan_text = capsys.readouterr().out
    assert (tmp_path / "00_torch.json").exists() and (tmp_path / "50_cuda.kernels.txt").read_text().strip() == plan_text.strip()
    whole = B200Backend().compile(Graph.from_json(tmp_path / "00_torch.json"))
    assert [s.entry for s in whole.steps] == ["emk_linear_f32_simt", "emk_softmax_lastdim"]
    for step in whole.steps:
        rec = tmp_path / "50_cuda.kernels" / f"{step.kernel_name}.torch.json"
        sub = B200Backend().compile(Graph.from_json(rec))
        assert [s.entry for s in sub.steps] == [step.entry]
        assert sub.steps[0].attrs == step.attrs
        head = (tmp_path / "50_cuda.kernels" / f"{step.kernel_name}.torch.txt").read_text()
        assert "1/1" in head and step.out in head
    # the softmax record reads the linear's output as a plain input of the same shape
    soft = Graph.from_json(tmp_path / "50_cuda.kernels" / f"{whole.steps[1].kernel_name}.torch.json")
    assert soft.inputs == ["linear"] and soft.nodes["linear"].output.shape == (8, 96)


def test_compile_cli_unsupported_op_exit_code(capsys):
    assert main(["compile", "-c", "torch.relu(torch.randn(4, 4))"]) == 1
    assert "LoweringError" in capsys.readouterr().err


def test_cli_needs_exactly_one_input(capsys):
    assert main(["compile"]) == 1
    assert main(["compile", "-c", "torch.relu(torch.randn(2))", "x.json"]) == 1


def test_accuracy_rule():
    eager = np.linspace(-1, 1, 1000)
    ok, mx, mean, tol = accuracy_verdict(eager + 0.05, eager, False)
    assert ok and abs(mx - 0.05) < 1e-9 and abs(tol - 0.08) < 1e-9
    # one outlier above 8 % of peak: passes on the mean clause
    v = eager.copy()
    v[0] += 0.5
    assert accuracy_verdict(v, eager, False)[0]
    # systematic 10 % corruption fails both clauses
    assert not accuracy_verdict(eager + 0.1, eager, False)[0]
    # fp16 outputs: the wide budget of the reference
    assert accuracy_verdict(eager + 0.5, eager, True)[0]
    # tiny outputs: the absolute floor
    assert accuracy_verdict(np.zeros(4) + 5e-4, np.zeros(4), False)[0]


def test_table_rows():
    lines = render_table({"Eager PyTorch": 200.0, "Emmy": 50.0})
    assert lines[0].split() == ["Backend", "Latency", "(us)", "vs", "Eager"]
    assert lines[2].split()[-1] == "1.00x" and lines[3].split() == ["Emmy", "50", "4.00x"]


# ------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("name", ["rmsnorm_readme_shape", "softmax_f32", "linear_bias_f32", "matmul_f32",
                                  "sdpa_causal_gqa_d128_f32", "sdpa_full_f32", "swiglu_f32"])
def test_run_cli_passes_on_golden_expressions(name, capsys):
    assert main(["run", "-c", CODES[name]]) == 0
    assert capsys.readouterr().out.strip().endswith("PASS")


@pytest.mark.gpu
def test_run_cli_bf16_and_bench(tmp_path, capsys):
    code = "nn.Linear(512, 768, bias=False).bfloat16()(torch.randn(256, 512).bfloat16())"
    assert main(["run", "-c", code, "--bench", "--warmup", "2", "--iters", "5", "--dump-dir", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "PASS" in out and "Eager PyTorch" in out and "Emmy" in out and "vs Eager" in out
    rec = json.loads((tmp_path / "60_bench_compare.json").read_text())
    assert rec["warmup"] == 2 and rec["iters"] == 5
    assert set(rec["backends"]) == {"Eager PyTorch", "Emmy"}
    assert rec["backends"]["Emmy"]["latency_us"] > 0 and "speedup_vs_eager" in rec["backends"]["Emmy"]


@pytest.mark.gpu
def test_run_cli_reruns_dumped_kernel_records(tmp_path, capsys):
    code = "q=torch.randn(1,4,160,128); k=torch.randn(1,2,160,128); F.scaled_dot_product_attention(q,k,k,is_causal=True,enable_gqa=True)"
    assert main(["run", "-c", code, "--dump-dir", str(tmp_path)]) == 0
    capsys.readouterr()
    recs = sorted((tmp_path / "50_cuda.kernels").glob("*.torch.json"))
    assert len(recs) == 1
    assert main(["run", "--ir", str(recs[0]), "--bench", "--warmup", "1", "--iters", "3"]) == 0
    out = capsys.readouterr().out
    assert "Emmy" in out and "k_scaled_dot_product_attention" in out


@pytest.mark.gpu
@pytest.mark.parametrize("code", [
    "x=torch.randn(512,1024).bfloat16(); w=(0.03*torch.randn(1024,768)).bfloat16(); r=torch.randn(512,768).bfloat16(); "
    "torch.matmul(x,w)+r",
    "x=torch.randn(40,64); w=torch.randn(64,96); r=torch.randn(40,96); torch.matmul(x,w)+r",
    "x=torch.randn(256,512).bfloat16(); wg=(0.05*torch.randn(512,384)).bfloat16(); wu=(0.05*torch.randn(512,384)).bfloat16(); "
    "F.silu(torch.matmul(x,wg))*torch.matmul(x,wu)",
])
def test_run_cli_perf_suite_expressions(code, capsys):
    assert main(["run", "-c", code]) == 0
    assert capsys.readouterr().out.strip().endswith("PASS")


@pytest.mark.gpu
def test_run_cli_json_record(capsys):
    assert main(["run", "--ir", str(GOLDEN / "graphs" / "rmsnorm_f32.json"), "--seed", "3"]) == 0
    assert "no eager reference" in capsys.readouterr().out


@pytest.mark.gpu
def test_run_cli_detects_wrong_answer(monkeypatch, capsys):
    """A corrupted kernel result must give FAIL and exit code 1."""
    from deplodock_b200 import ops

    real = ops.softmax_lastdim
    monkeypatch.setattr(ops, "softmax_lastdim", lambda x: real(x) * 3.0)
    assert main(["run", "-c", "torch.softmax(torch.randn(64, 256), dim=-1)"]) == 1
    assert "FAIL" in capsys.readouterr().out
