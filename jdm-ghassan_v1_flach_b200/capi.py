"""ctypes binding of libb200ops.so generated from include/b200ops.h.

The header is the single source of truth: every `int b200_*(...)` prototype in it
is parsed into ctypes argtypes, so the Python side cannot drift from the C ABI.
Arguments may be torch CUDA tensors (their data pointer is passed), None (NULL),
ints or floats.  A non-zero status raises B200Error carrying b200_last_error().
There is no fallback: if the shared library is missing, loading fails loudly.
"""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB_PATH = os.path.join(HERE, "libb200ops.so")
HEADERS = [os.path.join(ROOT, "include", "b200ops.h"), os.path.join(ROOT, "include", "b200step.h"),
           os.path.join(ROOT, "include", "b200gguf.h"), os.path.join(ROOT, "include", "b200ep.h")]

_SCALARS = {
    "int": C.c_int, "float": C.c_float, "int64_t": C.c_int64, "uint64_t": C.c_uint64,
    "size_t": C.c_size_t, "int32_t": C.c_int32, "double": C.c_double,
}


# int-returning functions whose result is a value, not a status code
VALUE_RETURNING = {"b200_version", "b200_fp16_gemm_enabled", "b200_bf16_gemm_enabled"}


class B200Error(RuntimeError):
    def __init__(self, name, code, message):
        super().__init__(f"{name}: status {code}: {message}")
        self.code = code
        self.message = message


def _ctype_of(decl):
    decl = decl.strip()
    if decl == "void":
        return None
    if "*" in decl:
        if re.match(r"^const\s+char\s*\*", decl):
            return C.c_char_p
        return C.c_void_p
    base = re.sub(r"\bconst\b", "", decl).split()
    # drop the parameter name
    ty = base[0] if len(base) >= 1 else ""
    if ty not in _SCALARS:
        raise ValueError(f"unhandled C type in header: {decl!r}")
    return _SCALARS[ty]


def parse_header(path):
    """-> {name: (restype_name, [ctypes...])} for every b200_* prototype."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    protos = {}
    for m in re.finditer(r"\b(int|size_t|uint64_t|const\s+char\s*\*)\s*(b200_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, args = m.group(1), m.group(2), m.group(3)
        args = args.strip()
        if args in ("", "void"):
            argtypes = []
        else:
            argtypes = [_ctype_of(a) for a in args.split(",")]
        protos[name] = (re.sub(r"\s+", " ", ret), argtypes)
    return protos


def declared_symbols():
    out = {}
    for h in HEADERS:
        if os.path.exists(h):
            out.update(parse_header(h))
    return out


def _to_c(v):
    if v is None:
        return None
    if hasattr(v, "data_ptr"):
        return v.data_ptr()
    return v


class Library:
    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is missing: build it with `make -C {os.path.join(HERE, 'csrc')}` "
                "(or __graft_entry__.build()); there is no CPU or PyTorch fallback")
        self.path = path
        self.cdll = C.CDLL(path)
        self.protos = declared_symbols()
        for name, (ret, argtypes) in self.protos.items():
            fn = getattr(self.cdll, name)          # AttributeError = symbol not exported
            fn.argtypes = argtypes
            fn.restype = {"int": C.c_int, "size_t": C.c_size_t, "uint64_t": C.c_uint64}.get(ret, C.c_char_p)

    def last_error(self):
        return self.cdll.b200_last_error().decode(errors="replace")

    def raw(self, name, *args):
        """Call without raising; returns the status code."""
        return getattr(self.cdll, name)(*[_to_c(a) for a in args])

    def call(self, name, *args):
        rc = self.raw(name, *args)
        if self.protos[name][0] == "int" and rc != 0 and name not in VALUE_RETURNING:
            raise B200Error(name, rc, self.last_error())
        return rc

    def __getattr__(self, name):
        if name.startswith("b200_"):
            return lambda *a: self.call(name, *a)
        raise AttributeError(name)


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
