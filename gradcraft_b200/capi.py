"""ctypes view of include/gradc_b200.h (used by the tests, the smoke check and the bench driver).

The prototypes are read from the header itself, so this file cannot drift from the C ABI.  Loading fails loudly
when the shared library has not been built: there is no Python or CPU fallback for any entry point.
"""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "..", "include", "gradc_b200.h")
LIB_PATH = os.path.join(HERE, "libgradc_b200.so")

OK, INVALID_ARG, UNSUPPORTED, OOM, CUDA_ERROR, NCCL_ERROR, TIMEOUT = range(7)
U = dict(IDENTITY=0, NEG=1, SQUARE=2, SQRT=3, GELU=4, SILU=5, EXP=6, LOG=7, RELU=8, SIGMOID=9, TANH=10)
B = dict(ADD=0, SUB=1, MUL=2, DIV=3, BGELU=4, ISUB=5, IDIV=6)
IDX_I64, IDX_I32 = 0, 1
OP_N, OP_T = 0, 1
ADAMW_CHUNK = 1024
DP_ID_BYTES = 128

_SCALARS = {"int": ctypes.c_int, "int64_t": ctypes.c_int64, "float": ctypes.c_float, "size_t": ctypes.c_size_t, "double": ctypes.c_double}


class GcbError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("gradc_b200 status %d: %s" % (status, message))
        self.status = status


def parse_header(path=HEADER):
    """[(name, restype, [argtype, ...])] for every GCB_API declaration."""
    text = re.sub(r"/\*.*?\*/", " ", open(path).read(), flags=re.S)
    out = []
    for m in re.finditer(r"GCB_API\s+([\w\s\*]+?)\s*\b(gcb_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                if "*" in a or "[" in a:
                    argtypes.append(ctypes.c_void_p)
                else:
                    argtypes.append(_SCALARS[a.replace("const ", "").split()[0]])
        if "*" in ret:
            restype = ctypes.c_char_p if "char" in ret else ctypes.c_void_p
        else:
            restype = _SCALARS[ret.split()[-1]]
        out.append((name, restype, argtypes))
    return out


def _ptr(x):
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return ctypes.c_void_p(x.data_ptr())
    if hasattr(x, "ctypes"):
        return ctypes.c_void_p(x.ctypes.data)
    return x


class Lib:
    """Attribute access gives the raw entry points (gcb_ prefix dropped); status codes other than OK raise GcbError."""

    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise RuntimeError("%s is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` (there is no fallback path)" % path)
        self.cdll = ctypes.CDLL(path)
        self.names = []
        for name, restype, argtypes in parse_header():
            fn = getattr(self.cdll, name)  # AttributeError here means the header declares a symbol the library lacks
            fn.restype, fn.argtypes = restype, argtypes
            self.names.append(name)
            checked = restype is ctypes.c_int and name not in ("gcb_ctx_device", "gcb_ctx_last_gemm_engine", "gcb_ctx_gemm_split_mode")
            setattr(self, name[4:], self._wrap(fn, checked))

    def _wrap(self, fn, checked):
        def call(*args):
            r = fn(*[_ptr(a) for a in args])
            if checked and r != OK:
                raise GcbError(r, self.cdll.gcb_last_error_string().decode())
            return r

        return call


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = Lib()
    return _LIB


class Context:
    """One device context bound to a CUDA stream (by default the current torch stream, so that torch tensors used as
    device buffers are ordered with the kernels)."""

    def __init__(self, device=0, stream=None, own_stream=False):
        self.lib = lib()
        h = ctypes.c_void_p()
        if own_stream:
            self.lib.ctx_create(device, ctypes.byref(h))
        else:
            if stream is None:
                import torch

                stream = torch.cuda.current_stream(device).cuda_stream
            self.lib.ctx_create_on_stream(device, ctypes.c_void_p(stream), ctypes.byref(h))
        self.h = h

    def __getattr__(self, name):
        fn = getattr(self.lib, name, None) or getattr(self.lib, "ctx_" + name)
        return lambda *a: fn(self.h, *a)

    def close(self):
        if self.h:
            self.lib.ctx_destroy(self.h)
            self.h = None
