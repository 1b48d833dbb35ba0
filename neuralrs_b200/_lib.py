"""ctypes binding of libnrs_b200.so (the C ABI in include/nrs.h and include/nrs_graph.h).

The library is the product; this module only loads it and declares argument
types.  There is no fallback: if the shared object is missing the import of
:func:`lib` raises, and every compute entry point fails with NRS_ERR_CUDA when
no sm_100 device is present.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libnrs_b200.so"
INCLUDE_DIR = _PKG.parent / "include"

_lib = None

c_float_p = C.POINTER(C.c_float)
c_i32_p = C.POINTER(C.c_int32)
c_i64_p = C.POINTER(C.c_int64)
VP = C.c_void_p

STATUS_NAMES = {0: "NRS_OK", 1: "NRS_ERR_ARG", 2: "NRS_ERR_SHAPE", 3: "NRS_ERR_ALLOC", 4: "NRS_ERR_CUDA",
                5: "NRS_ERR_NCCL", 6: "NRS_ERR_TIMEOUT", 7: "NRS_ERR_UNSUPPORTED"}

MATH_3XTF32, MATH_TF32, MATH_FP32 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2


class NrsError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {msg}")
        self.code = code


POLL_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)     # nrs_poll_fn

_C_TYPES = {
    "int": C.c_int, "float": C.c_float, "double": C.c_double, "size_t": C.c_size_t, "int64_t": C.c_int64,
    "uint64_t": C.c_uint64, "nrs_poll_fn": POLL_FN, "void": None,
}


def _ctype_of(type_str: str):
    """ctypes type of a C type spelled without a parameter name."""
    stars = type_str.count("*")
    base = type_str.replace("*", " ").replace("const", " ").split()
    if stars:
        return VP   # every pointer crosses as an address
    return _C_TYPES[base[-1]]


def _param_type(param: str):
    m = re.match(r"^(.*?)(\w+)$", param.strip(), flags=re.S)
    return _ctype_of(m.group(1))


def declared_functions() -> dict[str, tuple[str, list[str]]]:
    """Parses include/*.h: name -> (return decl, [param decls])."""
    out = {}
    for h in sorted(INCLUDE_DIR.glob("*.h")):
        txt = h.read_text()
        txt = re.sub(r"/\*.*?\*/", " ", txt, flags=re.S)
        txt = re.sub(r"//[^\n]*", " ", txt)
        for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(nrs_\w+)\s*\(([^;{}]*?)\)\s*;", txt):
            ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
            if "typedef" in ret or "struct" in ret or "enum" in ret:
                continue
            plist = [] if params in ("", "void") else [p.strip() for p in params.split(",")]
            out[name] = (ret, plist)
    return out


def lib() -> C.CDLL:
    """Loads the shared library and sets argtypes/restype from the headers."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m neuralrs_b200.build` "
            "(there is no CPU or pure-Python fallback)")
    l = C.CDLL(str(LIB_PATH))
    for name, (ret, params) in declared_functions().items():
        fn = getattr(l, name)   # AttributeError here means a declared symbol is not exported
        fn.restype = C.c_char_p if name == "nrs_last_error" else _ctype_of(ret)
        fn.argtypes = [_param_type(p) for p in params]
    _lib = l
    return l


def check(ctx, status: int) -> None:
    if status != 0:
        msg = lib().nrs_last_error(ctx)
        raise NrsError(status, msg.decode() if msg else "")
