"""Scalar types of the loop language and NumPy-style promotion.

Array elements and NumPy scalars are *strong* types; Python literals and Python
scalar arguments are *weak* (NEP 50): a weak operand adopts the kind-compatible type
of the strong operand it meets (``np.float32(x) * 2.5`` stays float32), and only
falls back to int64 / float64 when no strong operand decides.  The reference's Triton
lowering instead turns every float literal into float64
(appy/backends/triton/passes/device_passes/lower_constants.py:22-38) and passes Python
floats as float32; for expressions made of a single operation the two agree.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Ty:
    kind: str          # 'b' bool, 'i' signed, 'u' unsigned, 'f' float
    bits: int
    weak: bool = False

    @property
    def c(self) -> str:
        return C_NAME[(self.kind, self.bits)]

    @property
    def np(self):
        return np.dtype({("b", 8): "bool", ("i", 8): "int8", ("i", 16): "int16", ("i", 32): "int32",
                         ("i", 64): "int64", ("u", 8): "uint8", ("u", 16): "uint16", ("u", 32): "uint32",
                         ("u", 64): "uint64", ("f", 32): "float32", ("f", 64): "float64"}[(self.kind, self.bits)])

    @property
    def is_float(self):
        return self.kind == "f"

    @property
    def is_int(self):
        return self.kind in "iu"

    @property
    def is_bool(self):
        return self.kind == "b"

    def strong(self) -> "Ty":
        return Ty(self.kind, self.bits, False)

    def __str__(self):
        return ("weak " if self.weak else "") + self.c


C_NAME = {("b", 8): "bool", ("i", 8): "signed char", ("i", 16): "short", ("i", 32): "int", ("i", 64): "i64",
          ("u", 8): "unsigned char", ("u", 16): "unsigned short", ("u", 32): "unsigned int", ("u", 64): "u64",
          ("f", 32): "float", ("f", 64): "double"}

BOOL = Ty("b", 8)
I32 = Ty("i", 32)
I64 = Ty("i", 64)
F32 = Ty("f", 32)
F64 = Ty("f", 64)
WEAK_INT = Ty("i", 64, True)
WEAK_FLOAT = Ty("f", 64, True)


def from_numpy(dt) -> Ty:
    dt = np.dtype(dt)
    if dt == np.bool_:
        return BOOL
    if dt.kind in "iuf" and dt.itemsize * 8 in (8, 16, 32, 64) and not (dt.kind == "f" and dt.itemsize < 4):
        return Ty(dt.kind, dt.itemsize * 8)
    raise TypeError(f"Unsupported element type: {dt}")


def from_torch(tdtype) -> Ty:
    import torch
    table = {torch.bool: BOOL, torch.int8: Ty("i", 8), torch.int16: Ty("i", 16), torch.int32: I32,
             torch.int64: I64, torch.uint8: Ty("u", 8), torch.float32: F32, torch.float64: F64}
    if tdtype not in table:
        raise TypeError(f"Unsupported element type: {tdtype}")
    return table[tdtype]


def promote(a: Ty, b: Ty) -> Ty:
    """Result type of an arithmetic operation on a and b."""
    if a.weak and b.weak:
        if a.is_float or b.is_float:
            return WEAK_FLOAT
        return WEAK_INT
    if a.weak or b.weak:
        w, s = (a, b) if a.weak else (b, a)
        if w.is_float:
            return s if s.is_float else F64
        # weak int
        if s.is_bool:
            return I64
        return s
    return from_numpy(np.result_type(a.np, b.np))


def join(a: Ty | None, b: Ty) -> Ty:
    """Type of a local variable that is assigned values of type a and b."""
    if a is None:
        return b
    return promote(a, b)


def finalize(t: Ty) -> Ty:
    return t.strong()


def float_of(t: Ty) -> Ty:
    """Type of a math function (exp, sqrt, ...) applied to t, and of true division."""
    if t.is_float:
        return t
    if t.weak:
        return WEAK_FLOAT
    return F64
