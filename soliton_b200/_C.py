"""ctypes binding of libsoliton_b200.so, generated from the C header.

`include/soliton_b200.h` is the single statement of the ABI; this module reads its declarations and derives the
ctypes signature of every function from them, so binding and header cannot drift apart. Every declared symbol is
resolved when the module is imported: a library that lacks one fails here and not in the middle of a step (the
reference binds eagerly too, python/soliton/_C.py:68-70). There is no fallback: without the built library the import
raises.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsoliton_b200.so")
_HEADER = os.path.join(os.path.dirname(_HERE), "include", "soliton_b200.h")

if not os.path.exists(_LIB_PATH):
    raise ImportError(f"soliton_b200: {_LIB_PATH} is not built; run `python -m soliton_b200.build` (needs nvcc)")
lib = ctypes.CDLL(_LIB_PATH)

_SCALARS = {
    "void": None, "int": ctypes.c_int, "unsigned": ctypes.c_uint, "float": ctypes.c_float, "double": ctypes.c_double,
    "int64_t": ctypes.c_int64, "size_t": ctypes.c_size_t,
}


def _ctype(decl):
    """C type text of a parameter or result -> ctypes type. Strings travel as c_char_p; every other pointer as
    c_void_p, which takes device addresses (ints), ctypes arrays and byref() alike."""
    words = [w for w in re.sub(r"\bconst\b", " ", decl).replace("*", " * ").split()]
    stars = words.count("*")
    base = [w for w in words if w != "*"]
    if stars:
        return ctypes.c_char_p if base[:1] == ["char"] else ctypes.c_void_p
    return _SCALARS[base[0]]


def _declarations(text):
    """(name, result type text, [parameter type texts]) of every function declared in the header."""
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"^\s*#.*$", " ", text, flags=re.M)
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(slb?_\w+)\s*\(([^)]*)\)\s*;", text):
        result, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        if result.startswith("extern"):
            continue
        args = []
        if params and params != "void":
            for p in params.split(","):
                p = p.strip()
                # drop the parameter name: the last identifier, unless the parameter is a bare type
                m2 = re.match(r"^(.*?[\*\s])([A-Za-z_]\w*)$", p)
                args.append(m2.group(1).strip() if m2 and m2.group(1).strip() else p)
        yield name, result, args


_SIGS = {}
with open(_HEADER) as _f:
    for _name, _result, _args in _declarations(_f.read()):
        _SIGS[_name] = (_ctype(_result), [_ctype(a) for a in _args])
for _name, (_res, _argtypes) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _argtypes


def longs(values):
    """A C array of int64 (at least one element, so that an empty list still yields a valid pointer)."""
    values = list(values)
    return (ctypes.c_int64 * max(len(values), 1))(*values)


def set_option(name, value):
    if lib.slb_set_option(name.encode(), int(value)) != 0:
        raise KeyError(f"soliton_b200: unknown option {name!r}")


def counter(name):
    return lib.slb_get_counter(name.encode())
