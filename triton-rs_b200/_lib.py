"""ctypes binding of libb200_kernels.so.

The C prototypes are read from include/b200_kernels.h, so the Python side cannot
drift from the header: every function the header declares is bound with the
argument types written there, and a missing export is an error at load time.
There is no fallback of any kind: if the shared object is absent or a call is made
without a CUDA device, an exception says so.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

HERE = Path(__file__).resolve().parent
HEADER = HERE.parent / "include" / "b200_kernels.h"
LIB_PATH = HERE / "libb200_kernels.so"

_SCALARS = {
    "int": ctypes.c_int,
    "float": ctypes.c_float,
    "size_t": ctypes.c_size_t,
    "b200k_stream": ctypes.c_void_p,
    "uint64_t": ctypes.c_uint64,
    "int64_t": ctypes.c_int64,
}
# int-returning functions whose value is a count, not a status
_NOT_STATUS = {"b200k_layer_launches_per_forward"}
_RET = {"int": ctypes.c_int, "size_t": ctypes.c_size_t, "const char *": ctypes.c_char_p, "void": None}


class B200KError(RuntimeError):
    def __init__(self, name: str, code: int, message: str):
        super().__init__(f"{name} failed with status {code}: {message}")
        self.code = code
        self.message = message


def parse_header(path: Path = HEADER):
    """-> {name: (restype_key, [(ctype_key, argname), ...])} for every prototype."""
    text = path.read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    text = re.sub(r"^\s*#.*$", " ", text, flags=re.M)
    protos = {}
    pat = re.compile(r"\b(const\s+char\s*\*\s*|int\s+|size_t\s+|void\s+)(\w+)\s*\(([^;{}]*?)\)\s*;", re.S)
    for m in pat.finditer(text):
        ret, name, args = m.group(1), m.group(2), m.group(3)
        ret = "const char *" if "char" in ret else ret.strip()
        parsed = []
        args = " ".join(args.split())
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                am = re.match(r"^(.*?)(\w+)$", a)
                ty, an = am.group(1).strip(), am.group(2)
                if "*" in ty:
                    parsed.append(("ptr", an))
                else:
                    ty = ty.replace("const ", "").strip()
                    if ty not in _SCALARS:
                        raise ValueError(f"{name}: unknown C type {ty!r}")
                    parsed.append((ty, an))
        protos[name] = (ret, parsed)
    return protos


class Library:
    def __init__(self, path: Path = LIB_PATH):
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is missing: build it with `python {HERE.name}/build.py` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        self._dll = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
        self.protos = parse_header()
        self._fns = {}
        missing = []
        for name, (ret, args) in self.protos.items():
            try:
                fn = getattr(self._dll, name)
            except AttributeError:
                missing.append(name)
                continue
            fn.restype = _RET[ret]
            fn.argtypes = [ctypes.c_void_p if t == "ptr" else _SCALARS[t] for t, _ in args]
            self._fns[name] = fn
        if missing:
            raise ImportError(f"{path} does not export: {', '.join(missing)}")

    def last_error(self) -> str:
        return self._fns["b200k_last_error"]().decode()

    def raw(self, name: str):
        return self._fns[name]

    def call(self, name: str, *args):
        """Call `name`; torch tensors become device pointers; a non-zero status raises."""
        ret, proto = self.protos[name]
        if len(args) != len(proto):
            raise TypeError(f"{name} takes {len(proto)} arguments ({', '.join(n for _, n in proto)}), got {len(args)}")
        conv = []
        for (ty, an), a in zip(proto, args):
            if ty == "ptr":
                if a is None:
                    conv.append(None)
                elif hasattr(a, "data_ptr"):
                    if not a.is_cuda and not an.startswith("host"):
                        raise ValueError(f"{name}: argument {an} must be a CUDA tensor (no CPU fallback exists)")
                    conv.append(a.data_ptr())
                else:
                    conv.append(int(a))
            elif ty == "b200k_stream":
                conv.append(None if a in (None, 0) else int(getattr(a, "cuda_stream", a)))
            elif ty == "float":
                conv.append(float(a))
            else:
                conv.append(int(a))
        rc = self._fns[name](*conv)
        if ret == "int" and rc != 0 and name not in _NOT_STATUS:
            raise B200KError(name, rc, self.last_error())
        return rc


_LIB = None


def lib() -> Library:
    global _LIB
    if _LIB is None:
        _LIB = Library()
    return _LIB
