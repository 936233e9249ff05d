"""spbitnet_b200: the sparse-ternary (2:4, 1.5 bit/param) inference hot path of spbitnet,
written for NVIDIA B200 (sm_100a) behind the reference's kernel-wrapper API.

`kernels` mirrors include/spbitnet/{sparse_ternary,inference}_kernels.h of the reference
(same names, same argument order), `format` mirrors SparseTernaryTensor, `engine` mirrors
InferenceEngine.  Everything calls the C-ABI of libspbitnet_b200.so through ctypes; torch
is used only to own device memory and streams.
"""
from . import _lib  # noqa: F401
from ._lib import SpbError, load  # noqa: F401

__all__ = ["load", "SpbError"]
