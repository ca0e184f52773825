"""`Layout` = shape + element strides + element offset, as in the reference
(crates/hodu_core/src/types/layout.rs): transpose and broadcast are stride
tricks that share storage (layout.rs:291-380)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, Tuple


@dataclass(frozen=True)
class Layout:
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    offset: int = 0

    @staticmethod
    def from_shape(shape: Sequence[int]) -> "Layout":
        """Row-major contiguous layout (Layout::from_shape)."""
        shape = tuple(int(s) for s in shape)
        strides, acc = [], 1
        for s in reversed(shape):
            strides.append(acc)
            acc *= s
        return Layout(shape, tuple(reversed(strides)), 0)

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def is_contiguous(self) -> bool:
        acc = 1
        for s, st in zip(reversed(self.shape), reversed(self.strides)):
            if s > 1 and st != acc:
                return False
            acc *= s
        return True

    def transpose(self, d0: int, d1: int) -> "Layout":
        n = self.ndim
        d0, d1 = d0 % n, d1 % n
        shape, strides = list(self.shape), list(self.strides)
        shape[d0], shape[d1] = shape[d1], shape[d0]
        strides[d0], strides[d1] = strides[d1], strides[d0]
        return Layout(tuple(shape), tuple(strides), self.offset)

    def broadcast_to(self, target: Sequence[int]) -> "Layout":
        """Right-aligned broadcast; broadcast dims get stride 0 (layout.rs:291-337)."""
        target = tuple(int(t) for t in target)
        if len(target) < self.ndim:
            raise ValueError(f"cannot broadcast {self.shape} to {target}")
        pad = len(target) - self.ndim
        strides = []
        for i, t in enumerate(target):
            if i < pad:
                strides.append(0)
                continue
            s, st = self.shape[i - pad], self.strides[i - pad]
            if s == t:
                strides.append(st)
            elif s == 1:
                strides.append(0)
            else:
                raise ValueError(f"cannot broadcast {self.shape} to {target}")
        return Layout(target, tuple(strides), self.offset)

    def reshape_contiguous(self, shape: Sequence[int]) -> "Layout":
        if not self.is_contiguous():
            raise ValueError("reshape of a non-contiguous layout needs a copy")
        new = Layout.from_shape(shape)
        if new.size() != self.size():
            raise ValueError(f"cannot reshape {self.shape} to {tuple(shape)}")
        return Layout(new.shape, new.strides, self.offset)
