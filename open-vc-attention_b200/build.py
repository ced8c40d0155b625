"""Build libovc.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python open-vc-attention_b200/build.py

The library is written to open-vc-attention_b200/lib/libovc.so.  Only nvcc is needed; the
kernels are cross-compiled, so no GPU has to be present.
"""

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SOURCES = ["prep.cu", "attn.cu", "vsmooth.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", os.path.join(ROOT, "include"),
]


def nvcc_path():
    found = shutil.which("nvcc")
    if found:
        return found
    candidate = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(candidate):
        return candidate
    raise RuntimeError("nvcc not found; set CUDA_HOME")


def library_path():
    return os.path.join(HERE, "lib", "libovc.so")


def build(verbose=False, force=False):
    out = library_path()
    sources = [os.path.join(HERE, "csrc", name) for name in SOURCES]
    deps = sources + [os.path.join(HERE, "csrc", n) for n in os.listdir(os.path.join(HERE, "csrc")) if n.endswith(".cuh")]
    deps.append(os.path.join(ROOT, "include", "ovc.h"))
    if not force and os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    objects = []
    for src in sources:
        obj = os.path.join(HERE, "lib", os.path.basename(src) + ".o")
        cmd = [nvcc_path(), *FLAGS, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.run(cmd, check=True)
        objects.append(obj)
    subprocess.run([nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", out, *objects, "-lcudart"],
                   check=True)
    return out


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force=True))
