"""Recipe for ``oracle/_ref/``: the reference compiler's own emitted CUDA kernels for the four kernel configurations
and for one fp32 projection of its perf suite.

TEST AND REFERENCE-TIMING INFRASTRUCTURE, not product code. Run where the reference checkout is importable (it is not on the GPU
box; the outputs travel there):

    python oracle/build_ref_kernels.py /path/to/reference

For each configuration the reference traces the expression (``emmy/commands/trace.py:114`` ``graph_from_code``), lowers it
through its full pipeline with the compile-time target set to sm_100 (``emmy/compiler/target.py:41`` ``set_target``;
``emmy/compiler/pipeline/__init__.py:47`` ``CUDA_PASSES``) and hands back one ``CudaOp`` per graph
(``emmy/compiler/ir/cuda/ir.py:56-62``: ``kernel_source``, ``kernel_name``, ``arg_order``, ``grid``, ``block``,
``smem_bytes``, ``tma_descriptors``). The emitted source is compiled exactly as the reference's runtime does
(``emmy/compiler/backend/cuda/nvcc.py:118-151``: ``nvcc --cubin -arch=sm_<cc>[a] --use_fast_math``). Outputs, all under
``oracle/_ref/`` (git-ignored): ``<config>.cu`` (generated text), ``<config>.cubin`` and ``manifest.json`` with what a
launcher needs. Nothing of the reference's source tree is copied.
"""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

# the four single-kernel configurations, in the --code grammar of the reference CLI
CONFIGS = {
    "rmsnorm": "nn.RMSNorm(2048, eps=1e-6)(torch.randn(1, 32, 2048))",
    "softmax": "torch.nn.Softmax(dim=-1)(torch.randn(1, 28, 2048, 2048))",
    "linear": "nn.Linear(2048, 6144, bias=False).bfloat16()(torch.randn(4096, 2048).bfloat16())",
    "sdpa": ("q=torch.randn(4, 16, 2048, 128).bfloat16(); k=torch.randn(4, 8, 2048, 128).bfloat16(); "
             "v=torch.randn(4, 8, 2048, 128).bfloat16(); "
             "F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)"),
    # the fp32 tier the reference's own perf suite drives (tests/perf/cases.py:60-74): the Qwen3 q_proj at 512 tokens
    "matmul_f32": "a=torch.randn(512,1024); b=torch.randn(1024,2048); torch.matmul(a,b)",
}


def _static(dim) -> int:
    return int(dim.as_static()) if hasattr(dim, "as_static") else int(dim)


def _dim3(spec) -> list[int]:
    out = []
    for factors in spec:
        n = 1
        for f in factors:
            n *= int(f)
        out.append(n)
    return out


def build(reference_root: str) -> dict:
    sys.path.insert(0, reference_root)
    import emmy.compiler.target as target
    from emmy.commands.trace import graph_from_code
    from emmy.compiler.pipeline import CUDA_PASSES, Pipeline

    target.set_target((10, 0))
    OUT.mkdir(parents=True, exist_ok=True)
    manifest: dict[str, dict] = {}
    for name, code in CONFIGS.items():
        graph, _, _ = graph_from_code(code)
        lowered = Pipeline.build(CUDA_PASSES).run(graph)
        kernels = [(nid, n) for nid, n in lowered.nodes.items() if type(n.op).__name__ == "CudaOp"]
        if len(kernels) != 1:
            raise RuntimeError(f"{name}: expected one emitted kernel, got {len(kernels)}")
        nid, node = kernels[0]
        op = node.op
        buffers = {}
        for bid, bn in lowered.nodes.items():
            info = {"op": type(bn.op).__name__, "shape": [_static(d) for d in bn.output.shape],
                    "dtype": str(bn.output.dtype)}
            if type(bn.op).__name__ == "ConstantOp":
                info["value"] = getattr(bn.op, "value", None)
                info["source_path"] = getattr(bn.op, "source_path", None)
            buffers[bid] = info
        uses_tma = bool(op.tma_descriptors)
        cu = OUT / f"{name}.cu"
        cu.write_text(op.kernel_source)
        cubin = OUT / f"{name}.cubin"
        subprocess.run(["nvcc", "--cubin", "-arch=sm_100a", "--use_fast_math", "-o", str(cubin), str(cu)], check=True)
        manifest[name] = {
            "code": code, "kernel_name": op.kernel_name, "output": nid, "arg_order": list(op.arg_order),
            "grid": _dim3(op.grid), "block": _dim3(op.block), "smem_bytes": int(op.smem_bytes),
            "zero_outputs": list(op.zero_outputs), "uses_tma": uses_tma,
            "tma_descriptors": [{"name": d.name, "src_buf": d.src_buf, "box_extents": [int(b) for b in d.box_extents],
                                 "swizzle": d.swizzle} for d in op.tma_descriptors],
            "buffers": buffers,
        }
        print(f"{name}: {op.kernel_name} grid={manifest[name]['grid']} block={manifest[name]['block']} "
              f"smem={op.smem_bytes} args={list(op.arg_order)}")
    (OUT / "manifest.json").write_text(json.dumps(manifest, indent=1, default=str))
    return manifest


def find_reference() -> str | None:
    """The reference checkout: ``$EMMY_REFERENCE_ROOT``, else a ``reference`` directory beside this repository."""
    import os

    for cand in (os.environ.get("EMMY_REFERENCE_ROOT"), HERE.parent.parent / "reference"):
        if cand and (Path(cand) / "emmy" / "compiler").is_dir():
            return str(cand)
    return None


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else find_reference()
    if root is None:
        raise SystemExit("reference checkout not found: pass its path or set EMMY_REFERENCE_ROOT")
    build(root)
