"""Builds libcwk_attn.so (every CUDA source under csrc/) for sm_100a with nvcc.

The library is built in-tree next to this file so that it travels with the
source tree; nothing is installed. `python -m cwick_b200.build` rebuilds it.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcwk_attn.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]
# Sources whose results are compared bit for bit with the reference (exact summation orders, quantisers, codecs,
# recurrences) are compiled WITHOUT fast-math: IEEE division and square root, no flush-to-zero, no contraction of
# a*b+c across statements that the source keeps apart. Everything else (the tensor-core attention kernels, whose
# bar is a tolerance) takes --use_fast_math for its exp2/division forms.
EXACT_SOURCES = {"dsa.cu", "ds_compress.cu", "prep_ds.cu", "mm_index.cu", "cache_io.cu", "kda.cu", "gdn.cu", "gdn_chunk.cu"}


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        flags = NVCC_FLAGS + ([] if os.path.basename(src) in EXACT_SOURCES else ["--use_fast_math"])
        cmd = [nvcc] + flags + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-lcudart"]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
