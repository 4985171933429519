"""Build recipe for the reference's own sparse MoE extension -- TEST / BENCH INFRASTRUCTURE.

Compiles sparse_fp4_kernel/sparse_fp4_v7.cu of a checkout of Avarok-Cybersecurity/dgx-vllm, from
where it lies, into oracle/_ref/ as the Python extension module `sparse_fp4_v7`.  It is the
reference's setup_v7.py (sparse_fp4_kernel/setup_v7.py:7-17: CUDAExtension, -O3 --use_fast_math)
with one change: the architecture flag is sm_100 instead of sm_120 (setup_v7.py:13); the source is
compiled unmodified.  nvcc is called directly with torch's include and library paths, which is what
BuildExtension would do.

    python oracle/build_ref_v7.py /path/to/dgx-vllm [--force]

The result is used in two places only: one GPU parity test (a second yardstick beside the CPU
oracle) and bench.py's `parts.reference_v7_gpu` (the kernel to beat).  No product code loads it.
The built module needs the same torch build it was compiled against.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

_HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(_HERE, "_ref")
SRC_REL = os.path.join("sparse_fp4_kernel", "sparse_fp4_v7.cu")


def module_path() -> str:
    return os.path.join(OUT_DIR, "sparse_fp4_v7" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference_root: str, force: bool = False) -> str:
    src = os.path.join(reference_root, SRC_REL)
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    out = module_path()
    if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    import logging
    logging.getLogger("torch.utils.cpp_extension").setLevel(logging.ERROR)
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [sysconfig.get_paths()["include"]] + list(ce.include_paths("cuda"))
    libs = list(ce.library_paths("cuda"))
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-O3", "--use_fast_math", "-gencode", "arch=compute_100,code=sm_100", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-DTORCH_EXTENSION_NAME=sparse_fp4_v7",
           "-DTORCH_API_INCLUDE_EXTENSION_H"]
    for i in inc:
        cmd += ["-I", i]
    cmd += [src, "-o", out]
    for l in libs:
        cmd += ["-L", l]
    cmd += ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the reference extension failed:\n{r.stdout}\n{r.stderr}")
    return out


def load():
    """Import the built module (torch must be imported first) or return None when it was not built."""
    path = module_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against torch's libraries)
    spec = importlib.util.spec_from_file_location("sparse_fp4_v7", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    print(build(sys.argv[1], force="--force" in sys.argv))
