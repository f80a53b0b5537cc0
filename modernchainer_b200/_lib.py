"""ctypes loader for libmcb.so.  Prototypes are parsed from include/mcb.h so the Python
binding can never drift from the C ABI.  Loading fails loudly if the library is missing:
there is no Python or CPU fallback for any compute entry point."""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
HEADER = os.path.join(ROOT, "include", "mcb.h")
LIB_PATH = os.path.join(HERE, "libmcb.so")

_SCALARS = {"int32_t": C.c_int32, "int64_t": C.c_int64, "double": C.c_double, "float": C.c_float,
            "size_t": C.c_size_t, "mcb_status": C.c_int32, "uint64_t": C.c_uint64, "uint32_t": C.c_uint32}


def parse_header(path=HEADER):
    """Returns {name: (restype, [argtypes])} for every function declared in the header."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    protos = {}
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(mcb_\w+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if ret.startswith("typedef"):
            continue
        if "*" in ret:
            restype = C.c_char_p if "char" in ret else C.c_void_p
        elif ret == "void":
            restype = None
        else:
            restype = _SCALARS[ret.replace("const", "").strip()]
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    argtypes.append(C.c_void_p)
                else:
                    t = a.replace("const", "").split()[0]
                    argtypes.append(_SCALARS[t])
        protos[name] = (restype, argtypes)
    return protos


_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m modernchainer_b200.build` "
                               "(the CUDA library is the only implementation; there is no fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in parse_header().items():
            fn = getattr(lib, name)  # AttributeError here means the .so does not export a declared symbol
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib
