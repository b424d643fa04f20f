"""ctypes binding of libgsb200.so (the C ABI declared in include/gsb200.h).

Loading is strict: if the shared library is missing or does not export every declared symbol the
import fails — there is no Python or CPU fallback for any operator.
"""
import ctypes
import os
import re
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libgsb200.so")
HEADER_PATH = os.path.join(os.path.dirname(_PKG), "include", "gsb200.h")

c_i64 = ctypes.c_int64
c_u64 = ctypes.c_uint64
c_int = ctypes.c_int
c_vp = ctypes.c_void_p
c_i64p = ctypes.POINTER(ctypes.c_int64)


class GsbError(RuntimeError):
    def __init__(self, status, where, detail=""):
        self.status = status
        super().__init__(f"{where}: gsb status {status} ({status_string(status)}) {detail}".rstrip())


_lib = None
_lock = threading.Lock()


def declared_symbols(header_path=HEADER_PATH):
    """Names of all GSB_API functions declared in the public header."""
    text = open(header_path).read()
    return sorted(set(re.findall(r"GSB_API\s+[\w\s\*]+?\b(gsb_\w+)\s*\(", text)))


_CTYPES = {"int": ctypes.c_int, "int64_t": ctypes.c_int64, "uint64_t": ctypes.c_uint64, "size_t": ctypes.c_size_t,
           "double": ctypes.c_double, "float": ctypes.c_float}


def declared_prototypes(header_path=HEADER_PATH):
    """{name: (restype, [argtypes])} for every GSB_API function of the public header.  Pointers of any kind
    become c_void_p (callers pass raw device addresses, ctypes arrays or byref objects); `const char*` results
    become c_char_p.  Binding with explicit argument types makes a call with the wrong number of arguments raise
    instead of corrupting the stack."""
    text = re.sub(r"/\*.*?\*/", " ", open(header_path).read(), flags=re.S)
    protos = {}
    for ret, name, args in re.findall(r"GSB_API\s+([\w\s\*]+?)\b(gsb_\w+)\s*\(([^)]*)\)\s*;", text):
        ret = " ".join(ret.split())
        restype = ctypes.c_char_p if ret == "const char*" else _CTYPES[ret]
        argtypes = []
        for a in [x.strip() for x in args.split(",")]:
            if a in ("void", ""):
                continue
            if "*" in a:
                argtypes.append(ctypes.c_void_p)
            else:
                argtypes.append(_CTYPES[a.replace("const ", "").split()[0]])
        protos[name] = (restype, argtypes)
    return protos


def load():
    """Loads the library once; raises if it is absent (build with `python -m graph_sampling_b200.build`)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found: the CUDA kernel library is not built. "
                "Run `python -m graph_sampling_b200.build`; there is no CPU fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        missing = [s for s in declared_symbols() if not hasattr(lib, s)]
        if missing:
            raise ImportError(f"{LIB_PATH} lacks symbols declared in gsb200.h: {missing}")
        for name, (restype, argtypes) in declared_prototypes().items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
        return lib


def status_string(status):
    return load().gsb_status_string(int(status)).decode()


def version():
    return load().gsb_version().decode()
