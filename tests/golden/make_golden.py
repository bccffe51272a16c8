"""Generates the golden fixtures under ``tests/golden/`` by running the REFERENCE itself (test infrastructure).

Run in a container where the reference checkout is importable:

    PYTHONPATH=<reference root> python tests/golden/make_golden.py

For every case the reference's tracer (``emmy/commands/trace.py:114`` ``graph_from_code``) builds the Torch-IR graph of
a small seeded PyTorch expression and the reference's ``NumpyBackend`` (``emmy/compiler/backend/numpy/backend.py:18``,
default ``Backend.run`` of ``emmy/compiler/backend/base.py:139-205``) evaluates it; inputs, bound constants and outputs
are stored in ``<case>.npz`` and the graph record (``Graph.to_dict``, ``emmy/compiler/graph.py:953-997``) in
``graphs/<case>.json``. The fixtures pin ``oracle/np_ref.py`` and ``oracle/cpu_ref.py`` and feed the record loader of
the backend shim. The GPU box has no reference checkout; it reads only these files.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _trace_and_run(code: str):
    from emmy.commands.run import _bind_inputs
    from emmy.commands.trace import graph_from_code
    from emmy.compiler.backend.numpy.backend import NumpyBackend

    torch.manual_seed(0)
    graph, _, (module, args, kwargs) = graph_from_code(code)
    backend = NumpyBackend()
    compiled = backend.compile(graph)
    input_data = _bind_inputs(compiled, module, args, kwargs)
    result, _ = backend.run(compiled, input_data=input_data)
    return graph, input_data, result.outputs


CASES = {
    # name: code (the --code grammar of the reference CLI: preamble; final call)
    "rmsnorm_f32": "nn.RMSNorm(256, eps=1e-6)(torch.randn(2, 5, 256))",
    "rmsnorm_readme_shape": "nn.RMSNorm(2048, eps=1e-6)(torch.randn(1, 32, 2048))",
    "softmax_f32": "torch.nn.Softmax(dim=-1)(torch.randn(2, 3, 16, 200) * 3)",
    "linear_f32": "nn.Linear(64, 96, bias=False)(torch.randn(40, 64))",
    "linear_bias_f32": "nn.Linear(64, 96, bias=True)(torch.randn(3, 8, 64))",
    "matmul_f32": "torch.matmul(torch.randn(24, 64), torch.randn(64, 40))",
    "sdpa_causal_gqa_f32": (
        "q=torch.randn(1, 4, 48, 32); k=torch.randn(1, 2, 48, 32); v=torch.randn(1, 2, 48, 32); "
        "F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)"
    ),
    "sdpa_causal_gqa_d128_f32": (
        "q=torch.randn(1, 4, 160, 128); k=torch.randn(1, 2, 160, 128); v=torch.randn(1, 2, 160, 128); "
        "F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)"
    ),
    "sdpa_full_f32": (
        "q=torch.randn(2, 2, 20, 16); k=torch.randn(2, 2, 24, 16); v=torch.randn(2, 2, 24, 16); "
        "F.scaled_dot_product_attention(q, k, v)"
    ),
    "swiglu_f32": (
        "x=torch.randn(16, 64); wg=torch.randn(64, 96); wu=torch.randn(64, 96); "
        "F.silu(torch.matmul(x, wg)) * torch.matmul(x, wu)"
    ),
}

# graph records only (too large to store tensors): the benchmark configurations as the reference traces them
RECORD_ONLY = {
    "cfg1_rmsnorm": "nn.RMSNorm(2048, eps=1e-6)(torch.randn(1, 32, 2048))",
    "cfg2_softmax": "torch.nn.Softmax(dim=-1)(torch.randn(1, 28, 2048, 2048))",
    "cfg3_linear_bf16": "nn.Linear(2048, 6144, bias=False).bfloat16()(torch.randn(4096, 2048).bfloat16())",
    "cfg4_sdpa_bf16": (
        "q=torch.randn(4, 16, 2048, 128).bfloat16(); k=torch.randn(4, 8, 2048, 128).bfloat16(); "
        "v=torch.randn(4, 8, 2048, 128).bfloat16(); "
        "F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)"
    ),
}


def _to_np(v):
    a = np.asarray(v)
    return a


def _qwen3_layer_case():
    """One-layer Qwen3-shaped trunk (hidden 1024, 16/8 heads of 128, intermediate 3072, vocab 64) wrapped by the
    reference's ``build_full_model_wrapper`` (``emmy/compiler/trace/huggingface.py:17-186``: additive causal mask and
    precomputed rotary tables as buffers) and run EAGERLY in fp32 — the module the reference traces and checks
    against. The traced graph is stored as an op histogram only. The reference's NumpyBackend cannot pin this case:
    its ``SdpaOp.forward`` reads q, k, v and ignores the additive-mask input (``emmy/compiler/ir/frontend/ir.py:253-275``),
    so on this graph it attends non-causally and differs from the eager module by O(1).
    Only ids and the output are stored: the weights are regenerated from the seed by
    ``oracle.inputs.embed_model_weights``."""
    sys.path.insert(0, str(HERE.parent.parent))
    from emmy.compiler.trace.huggingface import build_full_model_wrapper
    from emmy.compiler.trace.torch import trace_module

    from oracle import cpu_ref, inputs

    cfg = inputs.EmbedModelConfig(vocab_size=64, num_hidden_layers=1)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg, seed=0, dtype=torch.float32), seed=1)
    S = 24
    model = cpu_ref.build_hf_model(cfg, sd, dtype=torch.float32)
    wrapper = build_full_model_wrapper(model, S, torch.float32)
    ids = inputs.token_ids(1, S, cfg.vocab_size, seed=3)
    with torch.no_grad():
        out = wrapper(ids).numpy()
    graph = trace_module(wrapper, (ids,))
    np.savez_compressed(HERE / "qwen3_layer_f32.npz", ids=ids.numpy(), hidden=np.asarray(out, dtype=np.float32))
    ops = {}
    for n in graph.nodes.values():
        ops[type(n.op).__name__] = ops.get(type(n.op).__name__, 0) + 1
    (HERE / "graphs").mkdir(exist_ok=True)
    (HERE / "graphs" / "qwen3_layer_f32.ophist.json").write_text(json.dumps(ops, indent=1, sort_keys=True))
    print("qwen3_layer_f32", out.shape, ops)


def _qwen3_trunk_record():
    """Two-layer Qwen3-shaped trunk in bf16 (hidden 1024, 16/8 heads of 128, intermediate 3072, vocab 64, 48 tokens)
    behind the reference's ``build_full_model_wrapper``, traced by the reference's ``trace_module``: the graph record is
    stored whole (``graphs/qwen3_trunk_2layer_bf16.json``: shapes and wiring only, no tensors) together with the ids
    and the hidden states the wrapper module returns when run eagerly (``qwen3_trunk_2layer_bf16.npz``). Weights are
    regenerated from the seed by ``oracle.inputs.embed_model_weights`` + ``perturb_norm_weights``; the constants of the
    record name them by ``source_path``."""
    sys.path.insert(0, str(HERE.parent.parent))
    from emmy.compiler.trace.huggingface import build_full_model_wrapper
    from emmy.compiler.trace.torch import trace_module

    from oracle import cpu_ref, inputs

    cfg = inputs.EmbedModelConfig(vocab_size=64, num_hidden_layers=2)
    sd = inputs.perturb_norm_weights(inputs.embed_model_weights(cfg, seed=0, dtype=torch.bfloat16), seed=1)
    S = 48
    model = cpu_ref.build_hf_model(cfg, sd, dtype=torch.bfloat16)
    wrapper = build_full_model_wrapper(model, S, torch.bfloat16)
    ids = inputs.token_ids(1, S, cfg.vocab_size, seed=3)
    with torch.no_grad():
        out = wrapper(ids).float().numpy()
    graph = trace_module(wrapper, (ids,))
    (HERE / "graphs" / "qwen3_trunk_2layer_bf16.json").write_text(json.dumps(graph.to_dict(), indent=0))
    np.savez_compressed(HERE / "qwen3_trunk_2layer_bf16.npz", ids=ids.numpy(), hidden=out)
    print("qwen3_trunk_2layer_bf16", out.shape, len(graph.nodes), "nodes")


def main() -> None:
    (HERE / "graphs").mkdir(exist_ok=True)
    if "--only-qwen3" in sys.argv:
        _qwen3_layer_case()
        return
    if "--only-trunk-record" in sys.argv:
        _qwen3_trunk_record()
        return
    if "--only-loop-records" in sys.argv:
        import emmy

        _loop_records(Path(emmy.__file__).resolve().parent.parent)
        return
    for name, code in CASES.items():
        graph, input_data, outputs = _trace_and_run(code)
        arrays = {f"in__{k}": _to_np(v) for k, v in input_data.items()}
        arrays.update({f"out__{k}": _to_np(v) for k, v in outputs.items()})
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        (HERE / "graphs" / f"{name}.json").write_text(json.dumps(graph.to_dict(), indent=1))
        print(name, {k: v.shape for k, v in arrays.items()})
    from emmy.commands.trace import graph_from_code

    for name, code in RECORD_ONLY.items():
        torch.manual_seed(0)
        graph, _, _ = graph_from_code(code)
        (HERE / "graphs" / f"{name}.json").write_text(json.dumps(graph.to_dict(), indent=1))
        print(name, "record only")
    _qwen3_layer_case()
    _qwen3_trunk_record()
    import emmy

    _loop_records(Path(emmy.__file__).resolve().parent.parent)


def _loop_records(reference_root: Path):
    """The reference's shipped Loop-IR kernel records (``kernels/*.json``): copied as fixtures, and for each one the
    output of the reference's own LoopOp -> C++ renderer (``emmy/compiler/ir/loop/runner.py:56-78``) compiled with g++
    on the seeded inputs of ``oracle.inputs.loop_record_inputs``. The outputs are up to 2 MB each, so a strided sample
    (every ``stride``-th element) and two checksums are stored."""
    import ctypes
    import shutil
    import subprocess
    import tempfile

    from emmy.compiler.graph import Graph
    from emmy.compiler.ir.loop.runner import PRELUDE, render_loopop_cpp

    sys.path.insert(0, str(HERE.parent.parent))
    from oracle.inputs import loop_record_inputs

    dst = HERE / "loop_records"
    dst.mkdir(exist_ok=True)
    for i, path in enumerate(sorted((reference_root / "kernels").glob("*.json"))):
        shutil.copyfile(path, dst / path.name)
        record = json.loads(path.read_text())
        graph = Graph.from_dict(record)
        nid, node = next((n, v) for n, v in graph.nodes.items() if type(v.op).__name__ == "LoopOp")
        loop = node.op
        shapes = {name: tuple(int(d.as_static()) for d in graph.nodes[name].output.shape) for name in loop.inputs}
        out_shape = tuple(int(d.as_static()) for d in node.output.shape)
        text = PRELUDE + render_loopop_cpp(loop, "k", shapes, out_shape)
        data = loop_record_inputs(record, seed=i)
        with tempfile.TemporaryDirectory() as td:
            src, lib = Path(td) / "k.cpp", Path(td) / "k.so"
            src.write_text(text)
            subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-o", str(lib), str(src)], check=True)
            fn = ctypes.CDLL(str(lib)).k
            out = np.zeros(out_shape, dtype=np.float32)
            args = [np.ascontiguousarray(data[name]) for name in loop.inputs]
            fn(*[a.ctypes.data_as(ctypes.c_void_p) for a in args], out.ctypes.data_as(ctypes.c_void_p))
        flat = out.ravel()
        stride = max(1, flat.size // 4096)
        np.savez_compressed(dst / f"{path.stem}.npz", sample=flat[::stride], stride=np.int64(stride), seed=np.int64(i),
                            sum=np.float64(flat.astype(np.float64).sum()),
                            abs_sum=np.float64(np.abs(flat.astype(np.float64)).sum()))
        print(path.stem, out_shape, "stride", stride, "sum", float(flat.astype(np.float64).sum()))


if __name__ == "__main__":
    main()
