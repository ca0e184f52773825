"""`DType` with the reference's `#[repr(u8)]` discriminants
(crates/hodu_core/src/types/dtype.rs:6-30) and its `Display` names (:31-58)."""
from __future__ import annotations

import enum


class DType(enum.IntEnum):
    BOOL = 0
    F8E4M3 = 1
    F8E5M2 = 2
    BF16 = 3
    F16 = 4
    F32 = 5
    F64 = 6
    U8 = 7
    U16 = 8
    U32 = 9
    U64 = 10
    I8 = 11
    I16 = 12
    I32 = 13
    I64 = 14

    def __str__(self) -> str:  # "bf16", "f8e4m3", ... as the kernel names use them
        return self.name.lower()

    @property
    def size_in_bytes(self) -> int:
        return _SIZES[self]


_SIZES = {DType.BOOL: 1, DType.F8E4M3: 1, DType.F8E5M2: 1, DType.BF16: 2, DType.F16: 2, DType.F32: 4,
          DType.F64: 8, DType.U8: 1, DType.U16: 2, DType.U32: 4, DType.U64: 8, DType.I8: 1,
          DType.I16: 2, DType.I32: 4, DType.I64: 8}


def from_torch(dt) -> DType:
    import torch
    table = {torch.float8_e4m3fn: DType.F8E4M3, torch.bfloat16: DType.BF16, torch.float16: DType.F16,
             torch.float32: DType.F32, torch.float64: DType.F64, torch.int8: DType.I8,
             torch.int32: DType.I32, torch.int64: DType.I64, torch.uint8: DType.U8, torch.bool: DType.BOOL,
             torch.int16: DType.I16}
    try:
        return table[dt]
    except KeyError:
        raise TypeError(f"no Hodu dtype for {dt}") from None


def to_torch(dt: DType):
    import torch
    table = {DType.F8E4M3: torch.float8_e4m3fn, DType.BF16: torch.bfloat16, DType.F16: torch.float16,
             DType.F32: torch.float32, DType.F64: torch.float64, DType.I8: torch.int8,
             DType.I32: torch.int32, DType.I64: torch.int64, DType.U8: torch.uint8, DType.BOOL: torch.bool,
             DType.I16: torch.int16}
    return table[DType(dt)]
