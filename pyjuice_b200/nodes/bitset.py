"""Variable scopes as integer bitmasks.

Plays the role of PyJuice's ``BitSet`` (src/pyjuice/utils/bitset.py:6-160): a set of
variable ids with union / intersection / ordered iteration, hashable so that scopes can
key dictionaries.  A Python ``int`` is the whole representation, which makes ``|`` and
``&`` single big-integer operations instead of byte loops.
"""
from __future__ import annotations

from typing import Iterable, List


class BitSet:
    __slots__ = ("mask",)

    def __init__(self, mask: int = 0):
        self.mask = int(mask)

    @classmethod
    def from_array(cls, values: Iterable[int]) -> "BitSet":
        m = 0
        for v in values:
            m |= 1 << int(v)
        return cls(m)

    def add(self, value: int) -> None:
        self.mask |= 1 << int(value)

    def remove(self, value: int) -> None:
        self.mask &= ~(1 << int(value))

    def hasitem(self, value: int) -> bool:
        return (self.mask >> int(value)) & 1 == 1

    def to_list(self) -> List[int]:
        out, m, base = [], self.mask, 0
        while m:
            chunk = m & 0xFFFFFFFFFFFFFFFF
            while chunk:
                low = chunk & -chunk
                out.append(base + low.bit_length() - 1)
                chunk ^= low
            m >>= 64
            base += 64
        return out

    def contains_all(self, other: "BitSet") -> bool:
        return (self.mask & other.mask) == other.mask

    def contains_any(self, other: "BitSet") -> bool:
        return (self.mask & other.mask) != 0

    def __and__(self, other: "BitSet") -> "BitSet":
        return BitSet(self.mask & other.mask)

    def __or__(self, other: "BitSet") -> "BitSet":
        return BitSet(self.mask | other.mask)

    def __ior__(self, other: "BitSet") -> "BitSet":
        self.mask |= other.mask
        return self

    def __eq__(self, other) -> bool:
        return isinstance(other, BitSet) and self.mask == other.mask

    def __hash__(self) -> int:
        return hash(self.mask)

    def __len__(self) -> int:
        return bin(self.mask).count("1")

    def __iter__(self):
        return iter(self.to_list())

    def __contains__(self, value: int) -> bool:
        return self.hasitem(value)

    def __repr__(self) -> str:
        n = len(self)
        if n <= 16:
            return "BitSet([" + ",".join(str(v) for v in self) + "])"
        return f"BitSet(num_elements={n})"
