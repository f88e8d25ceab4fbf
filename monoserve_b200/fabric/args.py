"""Operand blocks of model tiles, packed with the field offsets the native
library reports, so Python never hard-codes a C++ layout
(the contract of monoserve/fabric/args.py:11-31)."""
import struct

_LAYOUTS = None
_FMT = {"u64": "<Q", "u32": "<I", "f32": "<f"}


def layouts():
    global _LAYOUTS
    if _LAYOUTS is None:
        from monoserve_b200 import _C
        _LAYOUTS = _C.struct_layouts()
    return _LAYOUTS


def pack(name, **fields):
    """Bytes of struct `name` with the given fields set and all others zero.
    A tensor given for a u64 field contributes its device address."""
    size, spec = layouts()[name]
    buf = bytearray(size)
    for f, v in fields.items():
        if f not in spec:
            raise KeyError(f"{name} has no field {f}")
        off, t = spec[f]
        if t == "u64" and hasattr(v, "data_ptr"):
            v = v.data_ptr()
        struct.pack_into(_FMT[t], buf, off, v)
    return bytes(buf)
