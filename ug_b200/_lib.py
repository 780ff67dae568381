"""ctypes loader for libugb200.so.

The library is the product: there is no Python or CPU fallback.  If the
shared object is missing, importing this module raises with the build command.
Prototypes are read from ``include/ugb200.h`` so the header stays the single
source of truth for the ABI.
"""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libugb200.so")
HEADER = os.path.join(HERE, "..", "include", "ugb200.h")

_CTYPES = {
    "int32_t": C.c_int32,
    "uint64_t": C.c_uint64,
    "uint32_t": C.c_uint32,
    "size_t": C.c_size_t,
    "float": C.c_float,
    "void": None,
}


def _ctype(decl):
    """Map a C parameter / return declaration to a ctypes type."""
    decl = decl.replace("const", "").strip()
    stars = decl.count("*")
    base = decl.replace("*", "").split()
    base = base[0] if base else "void"
    if stars == 0:
        return _CTYPES[base]
    if base == "char" and stars == 1:
        return C.c_char_p
    return C.c_void_p  # every handle / buffer crosses as an opaque pointer


def parse_header(path=HEADER):
    """Return {name: (restype_decl, [param_decl, ...])} for every UGB_API prototype."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = {}
    for m in re.finditer(r"UGB_API\s+([^;(]+?)\s*\b(ug[bh]_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        ret, name, params = m.group(1), m.group(2), m.group(3)
        params = [p.strip() for p in params.replace("\n", " ").split(",")]
        if params == ["void"]:
            params = []
        protos[name] = (ret.strip(), params)
    return protos


def _param_type(p):
    # drop the parameter name (last identifier) unless the declaration is a bare type
    m = re.match(r"^(.*?)(\w+)$", p.strip())
    return _ctype(m.group(1) if m and m.group(1).strip() else p)


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ug_b200.build` "
            "(nvcc, sm_100a).  ug_b200 has no fallback path.")
    lib = C.CDLL(LIB_PATH)
    for name, (ret, params) in parse_header().items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch
        fn.restype = _ctype(ret)
        fn.argtypes = [_param_type(p) for p in params]
    return lib


lib = load()
