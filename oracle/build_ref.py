"""Compile upstream's own CUDA extension (its sm_75-era kernels, unmodified) for the B200 so
that it can be timed and compared on the GPU box.  TEST / BASELINE INFRASTRUCTURE ONLY.

    python oracle/build_ref.py            # needs the upstream checkout and ~10 minutes

Sources are compiled where they lie: the cuda/ directory of the upstream checkout, named by the
environment variable RFA_REFERENCE_CUDA or, without it, looked for in a directory "reference"
beside this repository; nothing is copied.  The only accommodation is an include
directory holding an empty THC/THC.h, a header PyTorch no longer ships and upstream does not
actually use.  Flags follow upstream's setup.py:21-27 except the target architecture
(compute_100 instead of compute_75).  Output: oracle/_ref/rfa_cuda_ref.so, a PyTorch
extension module exposing upstream's forward(q,k,v) and backward(q,k,v,grad_attn).
"""
import os
import subprocess
import sys
import sysconfig

import torch
from torch.utils import cpp_extension

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.environ.get("RFA_REFERENCE_CUDA") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference",
                                                            "random_feature_attention", "cuda")
OUT = os.path.join(HERE, "_ref")


def main():
    if not os.path.isdir(SRC):
        print(f"upstream sources not found at {SRC}; nothing built")
        return 0
    os.makedirs(OUT, exist_ok=True)
    inc = ["-I" + os.path.join(HERE, "stub")] + ["-I" + p for p in cpp_extension.include_paths(device_type="cuda")]
    inc.append("-I" + sysconfig.get_paths()["include"])
    common = ["-DTORCH_EXTENSION_NAME=rfa_cuda_ref", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
              "-std=c++17", "-O3"]
    nvcc_flags = ["-DCUDA_HAS_FP16=1", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                  "-D__CUDA_NO_HALF2_OPERATORS__", "-gencode", "arch=compute_100,code=sm_100", "-use_fast_math",
                  "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
    objs, procs = [], []
    for name in ("forward.cu", "backward.cu", "utils.cu"):
        obj = os.path.join(OUT, name[:-3] + ".o")
        objs.append(obj)
        procs.append(subprocess.Popen(["nvcc", *common, *nvcc_flags, *inc, "-c", os.path.join(SRC, name), "-o", obj]))
    obj = os.path.join(OUT, "rfa_cuda.o")
    objs.append(obj)
    procs.append(subprocess.Popen(["g++", *common, "-fPIC", *inc, "-c", os.path.join(SRC, "rfa_cuda.cpp"), "-o", obj]))
    if any(p.wait() != 0 for p in procs):
        print("compilation of the upstream extension failed")
        return 1
    lib_dirs = cpp_extension.library_paths(device_type="cuda")
    link = ["g++", "-shared", "-o", os.path.join(OUT, "rfa_cuda_ref.so"), *objs]
    link += ["-L" + d for d in lib_dirs] + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    r = subprocess.run(link)
    print("built" if r.returncode == 0 else "link failed", os.path.join(OUT, "rfa_cuda_ref.so"))
    return r.returncode


if __name__ == "__main__":
    sys.exit(main())
