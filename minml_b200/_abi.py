"""ctypes view of libminml_b200.so.

The prototypes are not typed in by hand: they are parsed from include/minml_b200.h, so every symbol the header
declares is bound (and `declared_symbols()` lets a test check that the shared library exports each of them).
Descriptor structs mirror include/minml/backend/backend_types.h:30-75 of the reference.
"""
import ctypes
import os
import re

_ROOT = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(_ROOT, "..", "include", "minml_b200.h")
LIBRARY = os.path.join(_ROOT, "libminml_b200.so")

(DTYPE_UNKNOWN, DTYPE_FLOAT8, DTYPE_FLOAT16, DTYPE_FLOAT32, DTYPE_FLOAT64, DTYPE_UINT8, DTYPE_INT8, DTYPE_INT16,
 DTYPE_INT32) = range(9)
(ACTIVATION_LINEAR, ACTIVATION_SIGMOID, ACTIVATION_TANH, ACTIVATION_RELU, ACTIVATION_LEAKY_RELU, ACTIVATION_EXP) = range(6)


class mlShape_t(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("dim", ctypes.c_int * 6)]


class mlQuantizationData_t(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_float), ("shift", ctypes.c_float)]


class mlTensor_t(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int), ("rank", ctypes.c_int), ("dim", ctypes.c_int * 6)]


_SCALARS = {
    "void": None, "int": ctypes.c_int, "float": ctypes.c_float, "double": ctypes.c_double, "bool": ctypes.c_bool,
    "char": ctypes.c_char, "size_t": ctypes.c_size_t, "unsigned long long": ctypes.c_ulonglong,
    "mlContext_t": ctypes.c_void_p, "mlEvent_t": ctypes.c_void_p, "mlDataType_t": ctypes.c_int,
    "mlActivationType_t": ctypes.c_int, "mlShape_t": mlShape_t, "mlTensor_t": mlTensor_t,
    "mlQuantizationData_t": mlQuantizationData_t,
}


def _ctype(text):
    t = text.replace("const", " ").strip()
    t = re.sub(r"\s+", " ", t)
    if t.endswith("*"):
        base = t[:-1].strip()
        if base == "void":
            return ctypes.c_void_p
        if base == "char":
            return ctypes.c_char_p
        return ctypes.POINTER(_SCALARS[base])
    return _SCALARS[t]


_DECL = re.compile(r"^([A-Za-z_][\w \*]*?)\s*\b((?:cud[an]n?|mb200)_\w+)\((.*)\);")


def parse_header(path=HEADER):
    """Returns [(name, restype, [argtypes], tag)] for every function the header declares."""
    out = []
    with open(path) as f:
        for line in f:
            m = _DECL.match(line.strip())
            if not m:
                continue
            ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
            tag = re.search(r"\[(hot|infra|stub)\]", line)
            argtypes = []
            if args and args != "void":
                for a in args.split(","):
                    a = a.strip()
                    # drop the parameter name: the last identifier not preceded by '*' glued to it
                    m2 = re.match(r"^(.*?)(\w+)$", a)
                    argtypes.append(_ctype(m2.group(1)))
            out.append((name, _ctype(ret), argtypes, tag.group(1) if tag else "ext"))
    return out


def declared_symbols():
    return [name for name, _, _, _ in parse_header()]


def load(path=LIBRARY):
    """Loads the shared library and attaches prototypes.  Raises when the library has not been built: there is
    no fallback implementation."""
    if not os.path.exists(path):
        raise RuntimeError("libminml_b200.so is missing (%s): run `python -m minml_b200.build`" % path)
    lib = ctypes.CDLL(path)
    for name, restype, argtypes, _ in parse_header():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib
