"""Host-side compressed format, mirroring spbitnet::SparseTernaryTensor
(reference include/spbitnet/sparse_ternary_tensor.h:41-265) on numpy arrays."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import check, load

SPARSE_GROUP_SIZE = 4     # kSparseGroupSize
SPARSE_NON_ZEROS = 2      # kSparseNonZeros
META_GROUPS_PER_WORD = 8  # kMetaGroupsPerWord
VALUES_GROUPS_PER_WORD = 16  # kValuesGroupsPerWord


def meta_words_per_row(cols: int) -> int:
    return load().spb_meta_words_per_row(cols)


def values_words_per_row(cols: int) -> int:
    return load().spb_values_words_per_row(cols)


def _ptr(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


@dataclass
class SparseTernaryTensor:
    """rows x cols ternary matrix with 2:4 sparsity: meta (rows, meta_stride) uint32 bitmaps,
    values (rows, values_stride) uint32 sign pairs."""
    rows: int
    cols: int
    meta: np.ndarray
    values: np.ndarray

    @property
    def meta_row_stride(self) -> int:
        return self.meta.shape[1]

    @property
    def values_row_stride(self) -> int:
        return self.values.shape[1]

    @staticmethod
    def _empty(rows: int, cols: int) -> "SparseTernaryTensor":
        if cols % SPARSE_GROUP_SIZE != 0:
            raise ValueError("cols must be a multiple of 4 for 2:4 sparsity")
        return SparseTernaryTensor(rows, cols,
                                   np.zeros((rows, meta_words_per_row(cols)), np.uint32),
                                   np.zeros((rows, values_words_per_row(cols)), np.uint32))

    @staticmethod
    def pack_from_dense(weights: np.ndarray, mask: np.ndarray) -> "SparseTernaryTensor":
        """pack_from_dense (sparse_ternary_tensor.h:58-108): weights int8 {-1,0,1}, mask keeps
        exactly two entries per group of four; a kept zero is stored as +1."""
        w = np.ascontiguousarray(weights, np.int8)
        m = np.ascontiguousarray(mask).astype(np.uint8)
        rows, cols = w.shape
        t = SparseTernaryTensor._empty(rows, cols)
        check(load().spb_pack_from_dense(_ptr(w), _ptr(m), rows, cols, _ptr(t.meta), _ptr(t.values)))
        return t

    @staticmethod
    def pack_with_pruning(latent: np.ndarray) -> "SparseTernaryTensor":
        """pack_with_pruning (sparse_ternary_tensor.h:123-191)."""
        x = np.ascontiguousarray(latent, np.float32)
        rows, cols = x.shape
        t = SparseTernaryTensor._empty(rows, cols)
        check(load().spb_pack_with_pruning(_ptr(x), rows, cols, _ptr(t.meta), _ptr(t.values)))
        return t

    def unpack_to_int8(self) -> np.ndarray:
        """unpack_to_int8 (sparse_ternary_tensor.h:197-232)."""
        out = np.empty((self.rows, self.cols), np.int8)
        check(load().spb_unpack_to_int8_host(_ptr(self.meta), _ptr(self.values), self.rows, self.cols,
                                             self.meta_row_stride, self.values_row_stride, _ptr(out)))
        return out

    def validate(self) -> None:
        """Raises SpbError unless every bitmap has exactly two bits set."""
        check(load().spb_validate_packed(_ptr(self.meta), self.rows, self.cols, self.meta_row_stride))
