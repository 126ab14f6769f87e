"""ctypes binding of libmkda.so.

The parameter structs are generated from ``include/mkda.h`` (the header is the single source of truth) and their
sizes are checked against ``mkda_struct_sizes`` when the library is loaded.  There is no fallback: if the library is
missing or stale the import of the kernels fails with the build command in the message.
"""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "mkda.h")
ENTRY_POINTS = (
    "mkda_gate_cumsum_fwd", "mkda_gate_bwd", "mkda_reduce_partials", "mkda_l2norm_rstd", "mkda_intra_fwd",
    "mkda_recur_fwd", "mkda_out_fwd", "mkda_epilogue_bwd", "mkda_epilogue_bwd_tiles", "mkda_bwd_dh", "mkda_bwd_chunk",
    "mkda_qk_grad_finish", "mkda_state_combine", "mkda_warmup_chunks", "mkda_selftest_umma", "mkda_selftest_wait", "mkda_epilogue_bwd_noalloc",
)
ENUMS = {}
STRUCTS = {}


def _parse_header(path=HEADER):
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    for name, val in re.findall(r"^#define\s+(MKDA_\w+)\s+(\d+)\s*$", text, flags=re.M):
        ENUMS[name] = int(val)
    for body in re.findall(r"enum\s*\{(.*?)\}", text, flags=re.S):
        for item in body.split(","):
            if "=" in item:
                name, val = item.split("=")
                ENUMS[name.strip()] = int(val.strip())
    order = []
    for body, name in re.findall(r"typedef\s+struct\s*\{(.*?)\}\s*(\w+)\s*;", text, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = " ".join(decl.split())
            if not decl:
                continue
            m = re.match(r"^(.*?)(\w+)$", decl)
            ctype_s, fname = m.group(1).strip(), m.group(2)
            if "*" in ctype_s:
                ct = ctypes.c_void_p
            elif ctype_s == "int":
                ct = ctypes.c_int
            elif ctype_s == "float":
                ct = ctypes.c_float
            elif ctype_s in STRUCTS:
                ct = STRUCTS[ctype_s]
            else:
                raise RuntimeError(f"mkda.h: cannot map type {ctype_s!r} of field {fname}")
            fields.append((fname, ct))
        STRUCTS[name] = type(name, (ctypes.Structure,), {"_fields_": fields})
        order.append(name)
    return order


STRUCT_ORDER = _parse_header()
globals().update(ENUMS)


class MkdaError(RuntimeError):
    pass


_libs = {}


def load():
    """Returns the loaded library (cached)."""
    variant = ""
    if variant in _libs:
        return _libs[variant]
    path = os.path.join(HERE, "libmkda.so")
    if not os.path.exists(path):
        raise MkdaError(f"{path} is missing: build it with `python -m mogankda_b200.build` (no CPU or library fallback exists)")
    lib = ctypes.CDLL(path)
    lib.mkda_last_error.restype = ctypes.c_char_p
    for name in ENTRY_POINTS:
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    n = len(STRUCT_ORDER)
    sizes = (ctypes.c_int * n)()
    cnt = lib.mkda_struct_sizes(sizes, n)
    if cnt != n or any(sizes[i] != ctypes.sizeof(STRUCTS[s]) for i, s in enumerate(STRUCT_ORDER)):
        raise MkdaError(f"{path} does not match include/mkda.h (struct sizes differ): rebuild with `python -m mogankda_b200.build --force`")
    _libs[variant] = lib
    return lib


def call(name, params, stream):
    lib = load()
    rc = getattr(lib, name)(ctypes.byref(params), ctypes.c_void_p(stream))
    if rc != 0:
        raise MkdaError(f"{name} failed ({rc}): {lib.mkda_last_error().decode()}")


def device_status():
    """Synchronises the current device and returns 0 unless a bounded wait inside a tensor-core kernel ever expired (the
    kernels then ran on to their exit and their results are not to be trusted)."""
    lib = load()
    lib.mkda_device_status.restype = ctypes.c_int
    lib.mkda_device_status.argtypes = []
    return int(lib.mkda_device_status())



def device_status_clear():
    """Synchronises the current device and clears the expired-wait flag (restores the long wait limit)."""
    lib = load()
    lib.mkda_device_status_clear.restype = ctypes.c_int
    lib.mkda_device_status_clear.argtypes = []
    return int(lib.mkda_device_status_clear())
