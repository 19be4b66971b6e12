"""Compile csrc/*.cu|.cpp for sm_100a with ninja (torch.utils.cpp_extension) and place the shared object in-tree."""
import os
import shutil
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
CSRC = ROOT / "csrc"
TARGET = Path(__file__).resolve().parent / "_C.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--use_fast_math", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xptxas", "-v", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF_OPERATORS__",
              "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__"]


def sources():
    return sorted(str(p) for p in CSRC.iterdir() if p.suffix in (".cu", ".cpp"))


def build_extension(verbose=False):
    from torch.utils.cpp_extension import load
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    build_dir = ROOT / "build" / "q38_C"
    build_dir.mkdir(parents=True, exist_ok=True)
    load(name="q38_C", sources=sources(), extra_cflags=["-O3", "-std=c++17"], extra_cuda_cflags=NVCC_FLAGS,
         extra_include_paths=[str(CSRC)], build_directory=str(build_dir), is_python_module=False, verbose=verbose)
    built = build_dir / "q38_C.so"
    if not TARGET.exists() or built.stat().st_mtime > TARGET.stat().st_mtime or built.stat().st_size != TARGET.stat().st_size:
        shutil.copyfile(built, TARGET)
    return TARGET
