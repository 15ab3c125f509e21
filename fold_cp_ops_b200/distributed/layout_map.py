"""Strided index maps: multidimensional index <-> flat index, with slicing.

Mirrors the public surface of the reference's ``fold_cp_ops/distributed/layout_map.py:41-359``
(``LayoutMap``, ``LayoutRightMap``, ``LayoutLeftMap``): the semantics are those of C++
``std::layout_stride::mapping`` plus the inverse map.  Used by :mod:`pe_map` to flatten the cp
mesh axes row-major into one peer index.
"""
from __future__ import annotations

import numbers
from typing import Sequence, Tuple, Union

import numpy as np

__all__ = ["LayoutMap", "LayoutRightMap", "LayoutLeftMap"]


def _is_int(v) -> bool:
    return isinstance(v, numbers.Integral) and not isinstance(v, bool)


class LayoutMap:
    """``flat = offset + sum(ids[k] * strides[k])`` over a box ``shape``.

    Raises ``ValueError`` when strides are not positive integers, when the shape has a zero or
    negative extent, when the lengths differ, or when two indices would map to the same flat
    index (the layout must be unique).
    """

    def __init__(self, strides: Sequence[int], shape: Sequence[int], offset: int = 0):
        strides = tuple(strides)
        shape = tuple(shape)
        if not all(_is_int(s) and s > 0 for s in strides):
            raise ValueError(f"Input strides contain non-integer or negative values: {strides}")
        if any(s < 0 for s in shape):
            raise ValueError(f"Input shape contain negative values: {shape}")
        if any(s == 0 for s in shape):
            raise ValueError(f"Input shape contain zero values: {shape}")
        if len(shape) != len(strides):
            raise ValueError(f"Shape {shape} and strides {strides} must have the same length")
        self._strides = tuple(int(s) for s in strides)
        self._shape = tuple(int(s) for s in shape)
        self._offset = int(offset)
        # axes from the fastest (smallest stride) to the slowest; ties broken by extent
        self._ascending = sorted(range(len(shape)), key=lambda a: (self._strides[a], self._shape[a]))
        self.is_unique, self.is_exhaustive = self._classify()
        if not self.is_unique:
            raise ValueError(f"Input strides {strides} and shape {shape} do not give unique layout.")

    def _classify(self) -> Tuple[bool, bool]:
        """unique: every stride is at least the span of all faster axes; exhaustive: exactly it."""
        need = 1
        unique = exhaustive = True
        for a in self._ascending:
            if self._strides[a] < need:
                unique = False
            if self._strides[a] != need:
                exhaustive = False
            need = self._strides[a] * self._shape[a]
        return unique, exhaustive

    # ---- properties -------------------------------------------------------------------------
    @property
    def offset(self) -> int:
        return self._offset

    @property
    def shape(self) -> Tuple[int, ...]:
        return self._shape

    @property
    def strides(self) -> Tuple[int, ...]:
        return self._strides

    @property
    def numel(self) -> int:
        return int(np.prod(self._shape)) if self._shape else 1

    @property
    def required_span_size(self) -> int:
        """Smallest contiguous buffer (in elements, past ``offset``) that holds the layout."""
        return 1 + sum((n - 1) * s for n, s in zip(self._shape, self._strides))

    # ---- forward / inverse -------------------------------------------------------------------
    def __call__(self, ids: Sequence[int]) -> int:
        ids = tuple(ids)
        if len(ids) != len(self._shape):
            raise ValueError(f"Expected {len(self._shape)} elements in ids but got only {len(ids)}")
        for axis, (i, n) in enumerate(zip(ids, self._shape)):
            if i < 0 or i >= n:
                raise ValueError(
                    f"Expected ids to satisfy 0 <= ids[{axis}] <= {n - 1} but found ids[{axis}] == {i}")
        return self._offset + sum(int(i) * s for i, s in zip(ids, self._strides))

    def ravel(self, ids: Sequence[int]) -> int:
        return self(ids)

    def unravel(self, flat_index: int) -> Tuple[int, ...]:
        if not _is_int(flat_index):
            raise TypeError(f"Expected arg to be an int, but instead got type {type(flat_index)}")
        rem = int(flat_index) - self._offset
        if rem < 0 or rem >= self.required_span_size:
            raise ValueError(
                f"Expected flat_index in range [{self._offset}, {self._offset + self.required_span_size - 1}], "
                f"but instead got {flat_index}")
        ids = [0] * len(self._shape)
        for a in reversed(self._ascending):  # slowest axis first
            q = min(rem // self._strides[a], self._shape[a] - 1)
            ids[a] = q
            rem -= q * self._strides[a]
        if rem != 0:
            msg = f"Input flat_index {flat_index} is out of the valid range of span."
            if not self.is_exhaustive:
                msg += " Given the layout is not exhaustive, the input flat_index can fall into the unmapped region."
            raise ValueError(msg)
        return tuple(ids)

    # ---- slicing -----------------------------------------------------------------------------
    def __getitem__(self, slices: Union[int, slice, Tuple[Union[int, slice], ...]]) -> "LayoutMap":
        if not isinstance(slices, tuple):
            slices = (slices,)
        slices = slices + (slice(None),) * (len(self._shape) - len(slices))
        shape, strides, offset = [], [], self._offset
        for axis, s in enumerate(slices):
            if _is_int(s):
                offset += int(s) * self._strides[axis]
            elif isinstance(s, slice):
                start, stop, step = s.indices(self._shape[axis])
                if step <= 0:
                    raise ValueError("Unsupported slicing: Negative or zero steps")
                if start >= stop:
                    raise ValueError("Unsupported slicing: start not smaller than stop")
                shape.append((stop - start + step - 1) // step)
                strides.append(self._strides[axis] * step)
                offset += start * self._strides[axis]
            else:
                raise TypeError(f"Unsupported slice type: {type(s)}")
        return LayoutMap(tuple(strides), tuple(shape), offset)

    def __repr__(self) -> str:
        return f"{type(self).__name__}(strides={self._strides}, shape={self._shape}, offset={self._offset})"


class LayoutRightMap(LayoutMap):
    """Row-major (C-contiguous): the last axis is the fastest."""

    def __init__(self, shape: Sequence[int]):
        shape = tuple(int(s) for s in shape)
        strides, acc = [], 1
        for n in reversed(shape):
            strides.append(acc)
            acc *= n
        super().__init__(tuple(reversed(strides)), shape)


class LayoutLeftMap(LayoutMap):
    """Column-major (Fortran-contiguous): the first axis is the fastest."""

    def __init__(self, shape: Sequence[int]):
        shape = tuple(int(s) for s in shape)
        strides, acc = [], 1
        for n in shape:
            strides.append(acc)
            acc *= n
        super().__init__(tuple(strides), shape)
