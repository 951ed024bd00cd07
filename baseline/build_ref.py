"""Builds the reference's generic CUDA kernels, unchanged, into `baseline/_ref/` for sm_100a.

    python baseline/build_ref.py REFERENCE_ROOT        (or TAU_REFERENCE_ROOT=... python baseline/build_ref.py)

taurs-ai/tau.rs is a Rust workspace and cannot be built here, but four of its kernel sources need only the CUDA
headers and export C launchers: `greedy_argmax.cu` (the one kernel on its dense Qwen3 path), `silu_and_mul.cu`,
`decode_attention.cu` and `centered_rms_norm.cu` (crates/cuda-kernels/src/kernels/).  They are compiled as they
are, one shared object each, next to a copy of the header they include; nothing of this library is linked in.
`baseline/_ref/` is not part of the repository.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
KERNELS = ("greedy_argmax.cu", "silu_and_mul.cu", "decode_attention.cu", "centered_rms_norm.cu")
HEADERS = ("fp32_precision.cuh",)


def main() -> int:
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TAU_REFERENCE_ROOT")
    if not root:
        print(__doc__)
        return 2
    source_dir = os.path.join(root, "crates", "cuda-kernels", "src", "kernels")
    os.makedirs(OUT, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    for name in HEADERS + KERNELS:
        shutil.copyfile(os.path.join(source_dir, name), os.path.join(OUT, name))
    for name in KERNELS:
        target = os.path.join(OUT, os.path.splitext(name)[0] + ".so")
        command = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
                   "-o", target, os.path.join(OUT, name)]
        print(" ".join(command), flush=True)
        subprocess.run(command, check=True)
    print(f"built {len(KERNELS)} reference kernel libraries in {OUT}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
