"""ctypes binding of the C ABI declared in include/*.h.

The headers are the single source of truth: every `rfk_*` prototype is parsed from them and
bound with matching argtypes, so a symbol that is declared but not exported (or the reverse)
shows up as a load error rather than as a silent fallback. There is no CPU or PyTorch
fallback behind these bindings: if the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
INCLUDE = PKG.parent / "include"

_SCALARS = {
    "int": ctypes.c_int,
    "float": ctypes.c_float,
    "long long": ctypes.c_longlong,
    "unsigned long long": ctypes.c_ulonglong,
    "size_t": ctypes.c_size_t,
    "unsigned short": ctypes.c_ushort,
    "int64_t": ctypes.c_int64,
    "uint64_t": ctypes.c_uint64,
    "rfk_stream_t": ctypes.c_void_p,
    "void": None,
}


def _ctype_of(decl: str):
    """Map one C parameter / return declaration (name stripped) to a ctypes type."""
    t = " ".join(decl.replace("*", " * ").split())
    if t.count("*") >= 2:
        return ctypes.POINTER(ctypes.c_void_p)          # host array of device pointers
    if t.endswith("*"):
        base = t[:-1].replace("const", "").strip()
        if base == "char":
            return ctypes.c_char_p
        if base == "int":
            return ctypes.POINTER(ctypes.c_int)          # host array of ints
        return ctypes.c_void_p                           # device pointer
    base = t.replace("const", "").strip()
    if base not in _SCALARS:
        raise ValueError(f"unmapped C type in header: {decl!r}")
    return _SCALARS[base]


_PROTO = re.compile(r"([A-Za-z_][\w\s\*]*?)\b(rfk_\w+)\s*\(([^;{}]*?)\)\s*;", re.S)


def parse_header(path: Path) -> dict[str, tuple]:
    """Return {symbol: (restype, [argtypes], [argnames])} for every rfk_* prototype."""
    text = path.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for ret, name, args in _PROTO.findall(text):
        ret = ret.strip()
        if ret.startswith("typedef") or "enum" in ret:
            continue
        argtypes, argnames = [], []
        args = args.strip()
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                m = re.match(r"(.*?)(\w+)$", a, re.S)
                argtypes.append(_ctype_of(m.group(1)))
                argnames.append(m.group(2))
        out[name] = (_ctype_of(ret), argtypes, argnames)
    return out


_HEADER_LIB = {"rfk.h": "librfk.so", "rfk_layers.h": "librfk_layers.so", "rfk_io.h": "librfk_io.so"}


def declared_symbols() -> dict[str, dict[str, tuple]]:
    """{header file name: {symbol: signature}} for the C-ABI headers under include/
    (rfk_compat.h is a C++ convenience layer over rfk.h and declares no symbols of its own)."""
    return {name: parse_header(INCLUDE / name) for name in sorted(_HEADER_LIB) if (INCLUDE / name).exists()}
_loaded: dict[str, ctypes.CDLL] = {}


def library_path(header: str) -> Path:
    return PKG / _HEADER_LIB[header]


def load(header: str = "rfk.h") -> ctypes.CDLL:
    """Load the shared library that implements `header` and bind every declared symbol."""
    if header in _loaded:
        return _loaded[header]
    path = library_path(header)
    if not path.exists():
        raise RuntimeError(
            f"{path.name} is not built ({path}); run `python {PKG.name}/build.py`. "
            "There is no fallback implementation.")
    if header == "rfk_layers.h":
        load("rfk.h")  # dependency; RTLD_GLOBAL so the layer library resolves rfk_* symbols
    lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    for name, (restype, argtypes, _) in parse_header(INCLUDE / header).items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise RuntimeError(f"{path.name} does not export {name} declared in {header}") from e
        fn.restype = restype
        fn.argtypes = argtypes
    _loaded[header] = lib
    return lib
