"""Build the reference's own NVFP4 quantization kernels into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY. The product never imports anything from ``oracle/``.

The reference ships three CUDA quantization entry points in
``sageattention3_blackwell/sageattn4/quantization/fp4_quantization_4d.cu``
(``scaled_fp4_quant``, ``scaled_fp4_quant_permute``, ``scaled_fp4_quant_trans``;
pybind block at :650-654).  They only use ``cvt.rn.satfinite.e2m1x2.f32`` and
compile for sm_100a, so they are the bit-exact checker for the FP4 codes and
E4M3 scales on a B200.  The sources are compiled where they lie in the
read-only reference checkout, with the reference's own nvcc flags
(``sageattention3_blackwell/setup.py:111-133``: ``-O3 --use_fast_math`` ...);
nothing is copied into this repository and the output directory is git-ignored.

Usage:  python oracle/build_ref.py [path-to-reference-checkout]
The checkout is looked for at the argument, else at $SAGE_REFERENCE_ROOT, else at the default below.
"""
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
MODULE = "sage_ref_quant_cuda"


DEFAULT_REFERENCE_ROOT = "/root/reference"


def reference_root() -> str:
    return os.environ.get("SAGE_REFERENCE_ROOT") or DEFAULT_REFERENCE_ROOT


def build(reference_root_: str = "", verbose: bool = False):
    src = Path(reference_root_ or reference_root()) / "sageattention3_blackwell" / "sageattn4" / "quantization"
    cu = src / "fp4_quantization_4d.cu"
    if not cu.exists():
        raise FileNotFoundError(f"reference quantization source not found: {cu}")
    OUT.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils.cpp_extension import load
    flags = [
        "-O3", "-std=c++17", "--use_fast_math", "-lineinfo", "-DNDEBUG",
        "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
        "--expt-relaxed-constexpr", "--expt-extended-lambda",
        "-gencode", "arch=compute_100a,code=sm_100a",
    ]
    load(name=MODULE, sources=[str(cu)], extra_include_paths=[str(src)],
         extra_cflags=["-O3", "-std=c++17"], extra_cuda_cflags=flags,
         build_directory=str(OUT), verbose=verbose, is_python_module=False)
    return OUT / f"{MODULE}.so"


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "", verbose=True))
