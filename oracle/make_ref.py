"""Recipe for oracle/_ref: the reference's own GPU kernels for this path, kept beside the oracle.

TEST INFRASTRUCTURE.  kb-nano's FP8 activation kernels and its grouped GEMM are Triton kernels that live in
the kb-nano tree itself (only DeepGEMM and vLLM's compiled ops are third party), and Triton ships with the
torch wheel.  This script puts the files that hold them, unmodified, under oracle/_ref/ (git-ignored), from
where `tests/test_triton_ref_gpu.py` runs them on the GPU as a second oracle (bit-for-bit for the two
quantisers, under the bf16 tolerance for the grouped GEMM) and `bench.py` times them as the GPU competitor
of the same operation.  Nothing in the product path imports oracle/_ref.

    python oracle/make_ref.py [TREE]     # kb-nano tree: the argument, else $KB_NANO_REF, else the default mount point

  silu_mul_quant_fp8.py    tasks/baseline/L1/silu_mul_quant_fp8.py, whole file (torch + triton only)
  moe_grouped_gemm.py      tasks/baseline/L1/moe_grouped_gemm.py, whole file (deep_gemm import is optional there)
  fp8_group_quant.py       the `_fp8_group_quant_kernel` Triton function of tasks/baseline/L1/fp8_linear.py
                           (:181-215) alone, because that file imports deep_gemm at module level

Without a kb-nano tree the script does nothing and says so (the tests that need oracle/_ref then skip).
"""
from __future__ import annotations

import ast
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


DEFAULT_TREE = os.path.join(os.sep, "root", "reference")      # where the build container mounts the kb-nano tree


def ref_root() -> str | None:
    for cand in (sys.argv[1] if len(sys.argv) > 1 else None, os.environ.get("KB_NANO_REF"), DEFAULT_TREE):
        if cand and os.path.isfile(os.path.join(cand, "tasks", "baseline", "L1", "silu_mul_quant_fp8.py")):
            return cand
    return None


def extract_function(path: str, name: str) -> str:
    """Source text of the top-level function `name` of the file at `path`, decorators included."""
    src = open(path).read()
    for node in ast.parse(src).body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            first = min([node.lineno] + [d.lineno for d in node.decorator_list])
            return "\n".join(src.splitlines()[first - 1: node.end_lineno]) + "\n"
    raise RuntimeError(f"{name} not found in {path}")


def build() -> bool:
    root = ref_root()
    if root is None:
        print("oracle/make_ref.py: no kb-nano tree (argument, $KB_NANO_REF or the default mount point); oracle/_ref left as it is")
        return os.path.isdir(OUT)
    l1 = os.path.join(root, "tasks", "baseline", "L1")
    os.makedirs(OUT, exist_ok=True)
    for name in ("silu_mul_quant_fp8.py", "moe_grouped_gemm.py"):
        shutil.copyfile(os.path.join(l1, name), os.path.join(OUT, name))
    kernel = extract_function(os.path.join(l1, "fp8_linear.py"), "_fp8_group_quant_kernel")
    with open(os.path.join(OUT, "fp8_group_quant.py"), "w") as f:
        f.write("# extracted by oracle/make_ref.py from tasks/baseline/L1/fp8_linear.py (function text unchanged)\n"
                "import triton\nimport triton.language as tl\n\n\n" + kernel)
    with open(os.path.join(OUT, "__init__.py"), "w") as f:
        f.write("")
    print(f"oracle/_ref: 3 files from {root}")
    return True


if __name__ == "__main__":
    sys.exit(0 if build() else 1)
