"""Operand blocks of model tiles.  The native library reports every operand
struct's size and field offsets (monofab_struct_layouts_json); Python packs by
those offsets and never hard-codes a C++ layout - the contract of the
reference's monoserve/fabric/args.py:11-31, whose names `layouts` and `pack`
this module keeps.

Each struct gets a small packer built once from the reported layout: a zeroed
template of the struct's size and, per field, a pre-compiled `struct.Struct`
with its offset.
"""
import struct

_CODES = {"u64": struct.Struct("<Q"), "u32": struct.Struct("<I"), "f32": struct.Struct("<f")}
_packers = {}
_table = None


def layouts():
    """{struct name: (sizeof, {field: (offset, "u64" | "u32" | "f32")})} as the library reports it."""
    global _table
    if _table is None:
        from monoserve_b200 import _C
        _table = _C.struct_layouts()
    return _table


class _Packer:
    def __init__(self, name):
        size, spec = layouts()[name]
        self.name = name
        self.blank = bytes(size)
        self.fields = {field: (_CODES[kind], offset, kind == "u64") for field, (offset, kind) in spec.items()}

    def __call__(self, values):
        block = bytearray(self.blank)
        for field, value in values.items():
            try:
                code, offset, is_address = self.fields[field]
            except KeyError:
                raise KeyError(f"{self.name} has no field {field}") from None
            if is_address and hasattr(value, "data_ptr"):   # a tensor stands for its device address
                value = value.data_ptr()
            code.pack_into(block, offset, value)
        return bytes(block)


def pack(name, **fields):
    """Bytes of struct `name` with the given fields set and all others zero."""
    packer = _packers.get(name)
    if packer is None:
        packer = _packers[name] = _Packer(name)
    return packer(fields)
