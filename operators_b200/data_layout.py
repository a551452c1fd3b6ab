"""ctypes image of the C `DataLayout` bit-field (include/infiniop.h; reference
include/data_type.h:4-47, mirrored by reference operatorspy/data_layout.py)."""
import ctypes


class DataLayout(ctypes.LittleEndianStructure):
    _fields_ = [
        ("packed", ctypes.c_ushort, 8),
        ("sign", ctypes.c_ushort, 1),
        ("size", ctypes.c_ushort, 7),
        ("mantissa", ctypes.c_ushort, 8),
        ("exponent", ctypes.c_ushort, 8),
    ]

    def bits(self):
        return int.from_bytes(bytes(self), "little")

    def __eq__(self, other):
        return isinstance(other, DataLayout) and self.bits() == other.bits()

    def __hash__(self):
        return self.bits()


def _dl(packed, sign, size, mantissa, exponent):
    return DataLayout(packed, sign, size, mantissa, exponent)


I8, I16, I32, I64 = _dl(1, 1, 1, 7, 0), _dl(1, 1, 2, 15, 0), _dl(1, 1, 4, 31, 0), _dl(1, 1, 8, 63, 0)
U8, U16, U32, U64 = _dl(1, 0, 1, 8, 0), _dl(1, 0, 2, 16, 0), _dl(1, 0, 4, 32, 0), _dl(1, 0, 8, 64, 0)
F16, BF16 = _dl(1, 1, 2, 10, 5), _dl(1, 1, 2, 7, 8)
F32, F64 = _dl(1, 1, 4, 23, 8), _dl(1, 1, 8, 52, 11)
