"""ctypes loader of libeisen_b200.so.

Argument types are taken from include/eisen_b200.h, so the Python side cannot drift from the
C ABI.  There is no fallback: if the library is missing, or a call returns a non-zero status,
an exception is raised.
"""
import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "libeisen_b200.so")
HEADER_PATH = os.path.join(_ROOT, "include", "eisen_b200.h")

_CTYPES = {
    "void*": C.c_void_p,
    "const void*": C.c_void_p,
    "float*": C.c_void_p,
    "const float*": C.c_void_p,
    "double*": C.c_void_p,
    "const double*": C.c_void_p,
    "int*": C.c_void_p,
    "const int*": C.c_void_p,
    "long long*": C.c_void_p,
    "const long long*": C.c_void_p,
    "const char*": C.c_char_p,
    "long long": C.c_longlong,
    "unsigned long long": C.c_ulonglong,
    "int": C.c_int,
    "float": C.c_float,
    "double": C.c_double,
    "void**": C.c_void_p,
    "const void* const*": C.c_void_p,
    "void* const*": C.c_void_p,
    "eisen_block_cb": C.c_void_p,
}

_DECL = re.compile(r"^\s*(const char\*|int|long long|void|eisen_\w+_t)\s+(eisen_\w+)\s*\(([^;{]*?)\)\s*;", re.M | re.S)


class EisenError(RuntimeError):
    pass


def _strip_comments(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def parse_header(path=HEADER_PATH):
    """Returns {name: (restype_str, [(type_str, arg_name), ...])} for every declaration."""
    text = _strip_comments(open(path).read())
    out = {}
    for m in _DECL.finditer(text):
        ret, name, args = m.group(1), m.group(2), m.group(3)
        parsed = []
        args = " ".join(args.split())
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                mm = re.match(r"^(.*?)(\w+)$", a)
                ty = mm.group(1).strip().replace(" *", "*")
                parsed.append((ty, mm.group(2)))
        out[name] = (ret, parsed)
    return out


_lib = None
_decls = None


def declarations():
    global _decls
    if _decls is None:
        _decls = parse_header()
    return _decls


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise EisenError(
                "libeisen_b200.so is not built (%s missing): run `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `python eisen_b200/build.py`; there is no fallback path" % LIB_PATH
            )
        L = C.CDLL(LIB_PATH)
        for name, (ret, args) in declarations().items():
            fn = getattr(L, name)  # AttributeError here means the header and the library disagree
            fn.restype = {"int": C.c_int, "long long": C.c_longlong, "const char*": C.c_char_p, "void": None}.get(ret, C.c_void_p)
            fn.argtypes = [_CTYPES[t] for t, _ in args]
        _lib = L
    return _lib


def check(rc, what=""):
    if rc != 0:
        msg = lib().eisen_last_error().decode("utf-8", "replace")
        raise EisenError("%s failed with status %d: %s" % (what or "eisen call", rc, msg))


def call(name, *args):
    """Calls an int-returning entry point and raises on a non-zero status."""
    rc = getattr(lib(), name)(*args)
    check(rc, name)
