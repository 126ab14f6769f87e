"""Builds libmkda.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

    python -m mogankda_b200.build [--force] [-v]

Objects are cached under ``build/`` and recompiled only when their source or a header is newer.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ("host.cu", "entry.cu", "prologue.cu", "combine.cu", "selftest.cu", "tc_chunk.cu", "tc_recur.cu", "tc_intra.cu")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Wno-deprecated-gpu-targets"]


def lib_path():
    return os.path.join(HERE, "libmkda.so")


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False):
    """Compiles (only what is stale) and links; returns the library path."""
    nvcc = os.environ.get("NVCC", "nvcc")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "mkda.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs, objs = [], []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        path = os.path.join(CSRC, src)
        if not force and _newer(obj, [path, *headers]):
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-c", path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        jobs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in jobs:
        log, _ = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{log}")
        if verbose:
            print(log)
    out = lib_path()
    if force or jobs or not _newer(out, objs):
        subprocess.check_call([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", out, *objs])
    return out


def main(argv):
    print(build(force="--force" in argv, verbose="-v" in argv))


if __name__ == "__main__":
    main(sys.argv[1:])
