"""The GEMV on prepared weights (the packed format re-laid once for the warp-level sparse MMA) against the CPU oracle
and against the GEMV on the packed format: integer results bit-exact on every configured shape, on row counts that
are not multiples of 16, on padded strides; the scaled half output bit for bit; what the entry points refuse."""
import numpy as np
import pytest
import torch

import oracle
from spbitnet_b200 import _lib, kernels as K, synth
from gpu_util import Guarded, dev

pytestmark = pytest.mark.gpu

SHAPES = [s for s in synth.GEMV_SHAPES if s[1] % 256 == 0]


def prepared(case):
    return K.prepare_weights(dev(case["meta"]), dev(case["values"]), case["rows"], case["cols"], case["meta_stride"],
                             case["values_stride"])


def run_prepared(case, prep=None, x=None):
    rows, cols = case["rows"], case["cols"]
    prep = prepared(case) if prep is None else prep
    assert prep.numel() == K.prepared_weights_bytes(rows, cols) == ((rows + 15) // 16) * (cols // 256) * 768
    y = Guarded(rows * 4)
    K.prepared_gemv_gpu(prep, dev(case["x"] if x is None else x), y.ptr, rows, cols)
    return y.read(np.int32)


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_config_shapes_bit_exact(rows, cols):
    case = synth.gemv_case(rows, cols, seed=0)
    want = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols, threads=8)
    prep = prepared(case)
    got = run_prepared(case, prep)
    assert (got == want).all()
    # extreme activations: every accumulator at its largest magnitude for this matrix
    for fill in (127, -127):
        x = np.full(cols, fill, np.int8)
        assert (run_prepared(case, prep, x) == oracle.sparse_gemv(case["meta"], case["values"], x, rows, cols, threads=8)).all()


@pytest.mark.parametrize("rows,cols", [(1, 256), (7, 256), (16, 512), (17, 768), (33, 1024), (100, 2560), (250, 6912),
                                       (8192, 8192), (1024, 8192), (2048, 28672)])
def test_ragged_rows_and_long_rows(rows, cols):
    case = synth.gemv_case(rows, cols, seed=rows + cols)
    want = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols, threads=8)
    assert (run_prepared(case) == want).all()


def test_padded_strides_and_packed_gemv_agree():
    rows, cols = 320, 1536
    case = synth.gemv_case(rows, cols, seed=3)
    ms, vs = case["meta_stride"] + 4, case["values_stride"] + 8
    meta = np.full((rows, ms), 0xDEADBEEF, np.uint32)
    values = np.full((rows, vs), 0xDEADBEEF, np.uint32)
    meta[:, :case["meta_stride"]] = case["meta"].reshape(rows, -1)[:, :case["meta_stride"]]
    values[:, :case["values_stride"]] = case["values"].reshape(rows, -1)[:, :case["values_stride"]]
    prep = K.prepare_weights(dev(meta), dev(values), rows, cols, ms, vs)
    y = Guarded(rows * 4)
    K.prepared_gemv_gpu(prep, dev(case["x"]), y.ptr, rows, cols)
    y2 = Guarded(rows * 4)
    K.sparse_ternary_gemv_gpu(dev(case["meta"]), dev(case["values"]), dev(case["x"]), y2.ptr, rows, cols,
                              case["meta_stride"], case["values_stride"])
    assert (y.read(np.int32) == y2.read(np.int32)).all()


def test_scaled_half_output_bit_for_bit():
    rows, cols = 2560, 2560
    case = synth.gemv_case(rows, cols, seed=4)
    prep = prepared(case)
    absmax = torch.tensor([3.25], dtype=torch.float32, device="cuda")
    gamma = np.float32(0.0371)
    meta, values, x = dev(case["meta"]), dev(case["values"]), dev(case["x"])
    a, b = Guarded(rows * 2), Guarded(rows * 2)
    K.prepared_bitlinear_q8_gpu(prep, x, a.ptr, absmax, gamma, rows, cols)
    import ctypes as C
    _lib.check(_lib.load().spb_sparse_bitlinear_q8(C.c_void_p(meta.data_ptr()), C.c_void_p(values.data_ptr()),
                                                   C.c_void_p(x.data_ptr()), C.c_void_p(b.ptr), C.c_void_p(absmax.data_ptr()),
                                                   C.c_float(gamma), rows, cols, case["meta_stride"], case["values_stride"], None))
    acc = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols, threads=8)
    dq = np.float32(np.float32(gamma * np.float32(3.25)) / np.float32(127.0))
    want = (acc.astype(np.float32) * dq).astype(np.float16).view(np.uint16)
    assert (b.read(np.uint16) == want).all()
    assert (a.read(np.uint16) == want).all()


def test_refusals():
    assert K.prepared_weights_bytes(64, 128) == 0  # not whole quads
    case = synth.gemv_case(64, 256, seed=1)
    prep = prepared(case)
    y = Guarded(64 * 4)
    lib = _lib.load()
    import ctypes as C
    rc = lib.spb_prepared_gemv(C.c_void_p(prep.data_ptr()), C.c_void_p(dev(case["x"]).data_ptr()), C.c_void_p(y.ptr), 64, 128, None)
    assert rc == _lib.SPB_E_UNSUPPORTED
    rc = lib.spb_prepared_gemv(None, C.c_void_p(dev(case["x"]).data_ptr()), C.c_void_p(y.ptr), 64, 256, None)
    assert rc == _lib.SPB_E_INVALID
    rc = lib.spb_prepare_weights(C.c_void_p(dev(case["meta"]).data_ptr()), C.c_void_p(dev(case["values"]).data_ptr()), 64, 256, 4, 4,
                                 C.c_void_p(prep.data_ptr()), None)
    assert rc == _lib.SPB_E_INVALID  # meta stride shorter than a row (8 words)
