"""GPU parity of the sparse-ternary GEMV / BitLinear / unpack / GEMM against the CPU oracle,
through the C-ABI.  Integer results must be bit-exact; the scaled fp32 and half outputs are
compared bit for bit too (tolerance allowed by the spec: 1 ulp)."""
import hashlib

import numpy as np
import pytest
import torch

import oracle
from spbitnet_b200 import _lib, kernels as K, synth
from gpu_util import Guarded, dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1, 4], ids=["auto", "pair-kernel", "warp-mma-kernel"], autouse=True)
def gemv_variant(request):
    """Every test in this file runs once per GEMV kernel variant."""
    old = K.set_gemv_variant(request.param)
    before = K.gemm_tc_timeouts()
    yield request.param
    K.set_gemv_variant(old)
    assert K.gemm_tc_timeouts() == before


def run_gemv(case, x=None, align=0):
    rows, cols = case["rows"], case["cols"]
    x = case["x"] if x is None else x
    y = Guarded(rows * 4, align_offset=align)
    K.sparse_ternary_gemv_gpu(dev(case["meta"]), dev(case["values"]), dev(x), y.ptr, rows, cols,
                              case["meta_stride"], case["values_stride"])
    return y.read(np.int32)


def test_reference_test_case_64x256(golden):
    # tests/test_sparse_ternary.cu:252-324 (GemvCorrectness, seed 42)
    g = golden("format_ref.npz")
    y = Guarded(64 * 4)
    K.sparse_ternary_gemv_gpu(dev(g["meta42"]), dev(g["values42"]), dev(g["x42"]), y.ptr, 64, 256,
                              g["meta42"].shape[1], g["values42"].shape[1])
    assert (y.read(np.int32) == g["y42"]).all()


def test_reference_test_case_2048(golden):
    # tests/test_sparse_ternary.cu:330-402 (GemvLargeDimension, seed 77)
    g = golden("format_ref.npz")
    w, m, x = oracle.testgen_gemv_case(77, 2048, 2048, -5, 5)
    meta, values = oracle.pack_from_dense(w, m)
    want = oracle.sparse_gemv(meta, values, x, 2048, 2048, threads=8)
    if hashlib.sha256(w.tobytes() + m.tobytes() + x.tobytes()).hexdigest() == str(g["sha77"]):
        assert (want == g["y77"]).all()
    case = dict(meta=meta, values=values, x=x, rows=2048, cols=2048, meta_stride=meta.shape[1],
                values_stride=values.shape[1])
    assert (run_gemv(case) == want).all()


@pytest.mark.parametrize("rows,cols", synth.GEMV_SHAPES)
def test_config_shapes_bit_exact(rows, cols):
    case = synth.gemv_case(rows, cols, seed=0)
    want = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols, threads=8)
    got = run_gemv(case)
    assert (got == want).all()
    assert (run_gemv(case) == got).all()  # run-to-run identical


def test_small_shapes_exhaustive():
    # every tail and stride situation: rows 1..17, cols 4..260 step 4 (generic path) and the
    # 128-multiples (unit path) with few rows
    rng = np.random.default_rng(5)
    for rows in (1, 2, 3, 7, 8, 9, 17):
        for cols in list(range(4, 264, 4)) + [384, 512, 640, 1152]:
            case = synth.gemv_case(rows, cols, seed=rows * 7919 + cols)
            x = rng.integers(-128, 128, cols, dtype=np.int8)  # includes -128
            want = oracle.sparse_gemv(case["meta"], case["values"], x, rows, cols)
            assert (run_gemv(case, x) == want).all(), (rows, cols)


@pytest.mark.parametrize("rows,cols", [(33, 2560), (700, 6912), (5, 28672), (301, 8192)])
def test_row_counts_that_do_not_fill_blocks(rows, cols):
    case = synth.gemv_case(rows, cols, seed=3)
    want = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols, threads=8)
    assert (run_gemv(case) == want).all()


def test_padded_strides_and_unaligned_pointers():
    rows, cols = 37, 640
    case = synth.gemv_case(rows, cols, seed=9)
    want = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols)
    ms, vs = case["meta_stride"], case["values_stride"]
    for pad_m, pad_v in [(4, 2), (1, 1), (3, 0)]:  # unit path keeps multiples of 4/2 words, others go generic
        meta = np.zeros((rows, ms + pad_m), np.uint32)
        values = np.zeros((rows, vs + pad_v), np.uint32)
        meta[:, :ms], values[:, :vs] = case["meta"], case["values"]
        meta[:, ms:], values[:, vs:] = 0xFFFFFFFF, 0xFFFFFFFF  # padding must never be visited
        y = Guarded(rows * 4)
        K.sparse_ternary_gemv_gpu(dev(meta), dev(values), dev(case["x"]), y.ptr, rows, cols, ms + pad_m, vs + pad_v)
        assert (y.read(np.int32) == want).all(), (pad_m, pad_v)
    # x at an odd address, meta at a 4-byte (not 16-byte) boundary
    xbuf = torch.zeros(cols + 16, dtype=torch.int8, device="cuda")
    xbuf[3:3 + cols] = dev(case["x"])
    mbuf = torch.zeros(case["meta"].size + 4, dtype=torch.int32, device="cuda")
    mbuf[1:1 + case["meta"].size] = dev(case["meta"]).flatten()
    y = Guarded(rows * 4)
    K.sparse_ternary_gemv_gpu(mbuf.data_ptr() + 4, dev(case["values"]), xbuf.data_ptr() + 3, y.ptr, rows, cols, ms, vs)
    assert (y.read(np.int32) == want).all()


@pytest.mark.parametrize("rows,cols", [(48, 16640), (100, 28672), (17, 32768), (1024, 28672), (33, 20480)])
def test_rows_longer_than_one_slab(rows, cols):
    # cols > 16384: the tensor-core kernel walks the row in double-buffered chunks of 4096 columns
    case = synth.gemv_case(rows, cols, seed=cols)
    want = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols, threads=8)
    assert (run_gemv(case) == want).all()
    # and the scaled half output of the BitLinear on a quantised vector
    out = Guarded(rows * 2)
    K.sparse_bitlinear_q8_gpu(dev(case["meta"]), dev(case["values"]), dev(case["x"]), out.ptr,
                              dev(np.array([1.7], np.float32)), 0.01, rows, cols, case["meta_stride"], case["values_stride"])
    wh = oracle.dequantize(want, np.float32(1.7), np.float32(0.01))
    assert (out.read(np.uint16) == wh.view(np.uint16)).all()


def test_invalid_bitmaps_are_memory_safe(gemv_variant):
    # src/kernels/sparse_ternary.cu:34-51 decodes any bitmap without exactly two bits as (0,0) while the
    # reference's CPU unpack yields as many non-zeros as bits: the result is unspecified there.  The kernels
    # here promise memory safety on such input (no fault, no write outside y), and exactness on the valid groups.
    cols = 128
    meta = np.array([[0x0F731248, 0x0, 0xEDB7FFFF, 0x33333333]], np.uint32)
    values = np.array([[0x9C3A5F01, 0x6E21D4B7]], np.uint32)
    x = np.random.default_rng(1).integers(-128, 128, cols, dtype=np.int8)
    lut = {3: (0, 1), 5: (0, 2), 6: (1, 2), 9: (0, 3), 10: (1, 3), 12: (2, 3)}
    acc = 0
    for g in range(cols // 4):
        b = (int(meta[0, g // 8]) >> ((g % 8) * 4)) & 0xF
        s = (int(values[0, g // 16]) >> ((g % 16) * 2)) & 3
        p0, p1 = lut.get(b, (0, 0))
        acc += (-1 if s & 1 else 1) * int(x[4 * g + p0]) + (-1 if s & 2 else 1) * int(x[4 * g + p1])
    case = dict(meta=meta, values=values, x=x, rows=1, cols=cols, meta_stride=4, values_stride=2)
    got = run_gemv(case)[0]  # Guarded output: canaries on either side are checked
    assert abs(int(got) - acc) <= 23 * 2 * 128  # the 23 invalid groups may each contribute anything two bytes can


def test_degenerate_and_bad_arguments():
    lib = _lib.load()
    y = torch.zeros(4, dtype=torch.int32, device="cuda")
    K.sparse_ternary_gemv_gpu(0, 0, 0, y, 0, 128, 4, 2)  # rows == 0: silent no-op
    K.sparse_ternary_gemv_gpu(0, 0, 0, y, 4, 0, 0, 0)
    with pytest.raises(_lib.SpbError):
        K.sparse_ternary_gemv_gpu(y, y, y, y, 4, 130, 5, 3)
    with pytest.raises(_lib.SpbError):
        K.sparse_ternary_gemv_gpu(y, y, y, y, 4, 256, 1, 1)  # stride shorter than a row
    assert lib.spb_last_error_string()


def test_scaled_fp32_output_is_exact():
    case = synth.gemv_case(2560, 2560, seed=0)
    rows, cols = 2560, 2560
    acc = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols, threads=8)
    for absmax, gamma in [(1.0, 1.0), (3.7251, 0.0213), (0.0917, 1.7)]:
        want = oracle.dequantize_f32(acc, absmax, gamma)
        y, ya = Guarded(rows * 4), Guarded(rows * 4)
        K.sparse_ternary_gemv_scaled_gpu(dev(case["meta"]), dev(case["values"]), dev(case["x"]), y.ptr, ya.ptr,
                                         dev(np.array([absmax], np.float32)), gamma, rows, cols,
                                         case["meta_stride"], case["values_stride"])
        got = y.read(np.float32)
        assert (ya.read(np.int32) == acc).all()
        ulp = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
        assert ulp.max() <= 1 and (got == want).all()


@pytest.mark.parametrize("rows,cols", [(2560, 2560), (640, 2560), (2560, 6912), (19, 132), (64, 256)])
def test_fused_bitlinear_matches_oracle(rows, cols):
    case = synth.gemv_case(rows, cols, seed=4)
    rng = np.random.default_rng(rows + cols)
    x = (rng.standard_normal(cols) * 2.5).astype(np.float16)
    x[::97] = 0
    absmax = oracle.absmax_reduce(x)
    gamma = 0.0317
    want = oracle.fused_bitlinear(case["meta"], case["values"], x, absmax, gamma, rows, cols)
    out = Guarded(rows * 2)
    K.fused_sparse_bitlinear_gpu(dev(case["meta"]), dev(case["values"]), dev(x), out.ptr,
                                 dev(np.array([absmax], np.float32)), gamma, rows, cols, case["meta_stride"],
                                 case["values_stride"])
    assert (out.read(np.uint16) == want.view(np.uint16)).all()
    # the pre-quantised form gives the same halfs
    q, a2 = oracle.absmax_quantize(x)
    out2 = Guarded(rows * 2)
    K.sparse_bitlinear_q8_gpu(dev(case["meta"]), dev(case["values"]), dev(q), out2.ptr,
                              dev(np.array([a2], np.float32)), gamma, rows, cols, case["meta_stride"],
                              case["values_stride"])
    assert (out2.read(np.uint16) == want.view(np.uint16)).all()


def test_fused_bitlinear_zero_input():
    case = synth.gemv_case(16, 256, seed=1)
    x = np.zeros(256, np.float16)
    out = Guarded(32)
    K.fused_sparse_bitlinear_gpu(dev(case["meta"]), dev(case["values"]), dev(x), out.ptr,
                                 dev(np.zeros(1, np.float32)), 0.5, 16, 256, case["meta_stride"],
                                 case["values_stride"])
    assert not out.read(np.uint16).any()


@pytest.mark.parametrize("rows,cols", [(8, 64), (3, 36), (5, 260), (64, 2560), (2560, 2560)])
def test_unpack_matches_oracle(rows, cols):
    # tests/test_sparse_ternary.cu:184-247 (GPU unpack == CPU unpack)
    case = synth.gemv_case(rows, cols, seed=123)
    want = oracle.unpack_to_int8(case["meta"], case["values"], rows, cols)
    for align in (0, 1):
        out = Guarded(rows * cols, align_offset=align)
        K.sparse_ternary_unpack_gpu(dev(case["meta"]), dev(case["values"]), out.ptr, rows, cols,
                                    case["meta_stride"], case["values_stride"])
        assert (out.read(np.int8).reshape(rows, cols) == want).all()


@pytest.fixture(params=[0, 1, 3], ids=["auto", "simt", "tcgen05sp"])
def gemm_variant(request):
    """0 = automatic (warp-level sparse MMA up to 32 batch rows, sparse tcgen05 above), 1 = SIMT form,
    3 = sparse tcgen05 form (forced for every n the layout allows)."""
    old = K.set_gemm_variant(request.param)
    before = K.gemm_tc_timeouts()
    yield request.param
    K.set_gemm_variant(old)
    assert K.gemm_tc_timeouts() == before


@pytest.mark.parametrize("rows,cols,n", [(64, 256, 16), (64, 256, 1), (37, 132, 5), (300, 2560, 4), (96, 6912, 19),
                                          (2048, 2048, 32), (128, 512, 64), (128, 128, 16), (129, 384, 257),
                                          (1000, 1024, 300), (256, 2560, 256), (100, 256, 8), (500, 2560, 9),
                                          (333, 512, 24), (64, 6912, 32), (2560, 6912, 17), (48, 768, 3)])
def test_gemm_matches_oracle(rows, cols, n, gemm_variant):
    # tests/test_cusparselt.cu:127-274: exact int32 vs the CPU int8 GEMM
    case = synth.gemm_case(rows, cols, n, seed=n)
    want = oracle.sparse_gemm(case["meta"], case["values"], case["X"], rows, cols)
    Y = Guarded(n * rows * 4)
    K.sparse_ternary_gemm_gpu(dev(case["meta"]), dev(case["values"]), dev(case["X"]), Y.ptr, rows, cols, n,
                              case["meta_stride"], case["values_stride"])
    assert (Y.read(np.int32).reshape(n, rows) == want).all()
    dense = oracle.unpack_to_int8(case["meta"], case["values"], rows, cols)
    assert (oracle.int8_gemm(dense[:8], case["X"].T.copy())[:, :n] == want.T[:8]).all()


@pytest.mark.parametrize("rows,cols", synth.GEMM_SHAPES)
def test_gemm_full_size_properties(rows, cols, gemm_variant):
    # full benchmark shapes: column j of the batch must equal the GEMV of row j (checked against
    # the oracle for a few rows), and the product is linear: W(a+b) = Wa + Wb
    n = 64
    case = synth.gemm_case(rows, cols, n, seed=1)
    X = (case["X"] // 2).astype(np.int8)
    X[2] = X[0] + X[1]
    d_meta, d_values = dev(case["meta"]), dev(case["values"])
    Y = torch.empty((n, rows), dtype=torch.int32, device="cuda")
    K.sparse_ternary_gemm_gpu(d_meta, d_values, dev(X), Y, rows, cols, n, case["meta_stride"], case["values_stride"])
    Yh = host(Y)
    for j in (0, 17, 63):
        assert (Yh[j] == oracle.sparse_gemv(case["meta"], case["values"], X[j], rows, cols, threads=8)).all()
    assert (Yh[2] == Yh[0] + Yh[1]).all()
    y1 = torch.empty(rows, dtype=torch.int32, device="cuda")
    K.sparse_ternary_gemv_gpu(d_meta, d_values, dev(X[5]), y1, rows, cols, case["meta_stride"], case["values_stride"])
    assert (host(y1) == Yh[5]).all()


def test_work_list_batch_matches_oracle():
    # one persistent launch over a list of GEMVs of mixed shapes == the same GEMVs one by one
    shapes = [(6912, 2560), (640, 2560), (2560, 6912), (33, 256), (2048, 2048), (1, 256), (700, 8192), (6912, 2560),
              (5, 512), (301, 2560), (8192, 2560), (6912, 2560)]
    rng = np.random.default_rng(0)
    items, wants, keep = [], [], []
    for i, (rows, cols) in enumerate(shapes):
        case = synth.gemv_case(rows, cols, seed=100 + i)
        x = rng.integers(-128, 128, cols, dtype=np.int8)
        wants.append(oracle.sparse_gemv(case["meta"], case["values"], x, rows, cols, threads=8))
        y = torch.full((rows + 64,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
        t = (dev(case["meta"]), dev(case["values"]), dev(x), y)
        keep.append(t)
        items.append((t[0], t[1], t[2], y.data_ptr() + 128, rows, cols, case["meta_stride"], case["values_stride"]))
    work = K.GemvWorkList(items)
    for _ in range(2):
        K.sparse_ternary_gemv_batch_gpu(work)
    torch.cuda.synchronize()
    for (rows, cols), want, t in zip(shapes, wants, keep):
        got = t[3].cpu().numpy()
        assert (got[32:32 + rows] == want).all(), (rows, cols)
        assert (got[:32] == 0x5A5A5A5A).all() and (got[32 + rows:] == 0x5A5A5A5A).all()
    with pytest.raises(_lib.SpbError):
        K.GemvWorkList([(keep[0][0], keep[0][1], keep[0][2], keep[0][3], 16, 128, 4, 2)])  # cols not a multiple of 256
