"""Builds libmkda.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

    python -m mogankda_b200.build [--force] [-v] [--variant DIGITS]

Every chunk contraction is compiled either as plain TF32 (1) or as the error-compensated three-product TF32 split (3);
the choice per kernel is a compile-time macro.  ``--variant`` takes one digit per macro, in the order of ``PREC_MACROS``,
and builds ``libmkda_<digits>.so`` beside the default library (used to measure where operand rounding matters).
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
# source file -> precision macros it understands
SOURCES = {
    "host.cu": (),
    "prologue.cu": (),
    "intra_fwd.cu": ("MKDA_PREC_INTRA",),
    "recur.cu": ("MKDA_PREC_STATE", "MKDA_PREC_OUT", "MKDA_PREC_DH"),
    "bwd_post.cu": ("MKDA_PREC_WY", "MKDA_PREC_SGRAD"),
    "intra_bwd.cu": ("MKDA_PREC_INTRA_BWD",),
    "selftest.cu": (),
    "tc_chunk.cu": (),
    "tc_recur.cu": (),
    "tc_intra.cu": (),
}
PREC_MACROS = ("MKDA_PREC_INTRA", "MKDA_PREC_STATE", "MKDA_PREC_OUT", "MKDA_PREC_DH", "MKDA_PREC_WY", "MKDA_PREC_SGRAD",
               "MKDA_PREC_INTRA_BWD")
# shipped configuration (see DESIGN.md for the measurements behind it)
DEFAULT_PREC = dict(MKDA_PREC_INTRA=3, MKDA_PREC_STATE=1, MKDA_PREC_OUT=1, MKDA_PREC_DH=1, MKDA_PREC_WY=3,
                    MKDA_PREC_SGRAD=3, MKDA_PREC_INTRA_BWD=3)
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Wno-deprecated-gpu-targets"]


def lib_path(variant=""):
    return os.path.join(HERE, f"libmkda{variant}.so")


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, variant="", prec=None, verbose=False):
    """Compiles (only what is stale) and links.  ``prec`` maps macro -> 1 | 3 (default: DEFAULT_PREC)."""
    nvcc = os.environ.get("NVCC", "nvcc")
    prec = dict(DEFAULT_PREC, **(prec or {}))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "mkda.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs, objs = [], []
    for src, macros in SOURCES.items():
        tag = "".join(str(prec[m]) for m in macros)
        obj = os.path.join(objdir, src.replace(".cu", f"_{tag}.o" if tag else ".o"))
        objs.append(obj)
        path = os.path.join(CSRC, src)
        if not force and _newer(obj, [path, *headers]):
            continue
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{m}={prec[m]}" for m in macros], "-c", path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        jobs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in jobs:
        log, _ = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{log}")
        if verbose:
            print(log)
    out = lib_path(variant)
    if force or jobs or not _newer(out, objs):
        subprocess.check_call([nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", out, *objs])
    return out


def build_variant(digits, force=False):
    assert len(digits) == len(PREC_MACROS) and set(digits) <= {"1", "3"}, "one digit (1 or 3) per macro"
    return build(force=force, variant="_" + digits, prec={m: int(d) for m, d in zip(PREC_MACROS, digits)})


def main(argv):
    force = "--force" in argv
    print(build(force=force, verbose="-v" in argv))
    for i, a in enumerate(argv):
        if a == "--variant":
            print(build_variant(argv[i + 1], force=force))


if __name__ == "__main__":
    main(sys.argv[1:])
