"""The batched product at the sizes of the benchmark's prefill configuration: both FFN shapes at N = 256 and 1024,
every output element compared with the CPU oracle (exact int32, as tests/test_cusparselt.cu:127-274 compares the
reference's batched path with its CPU GEMM), and the half epilogue of the batched BitLinear bit for bit.  The four
cases reach every branch of the tcgen05 launcher by shape alone: 256 batch rows per block with two re-encoding
groups on two stages (both shapes at N = 1024), 128 rows with one group on four stages (6912x2560, N = 256), 64
rows with two groups on four stages (2560x6912, N = 256).  Also here: the bounded-wait self-test and the work
list's skip of an oversize item."""
import numpy as np
import pytest
import torch

import oracle
from spbitnet_b200 import _lib, kernels as K, synth
from gpu_util import Guarded, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=synth.GEMM_SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def full_case(request):
    rows, cols = request.param
    case = synth.gemm_case(rows, cols, 1024, seed=3)
    case["want"] = oracle.sparse_gemm(case["meta"], case["values"], case["X"], rows, cols)  # [1024, rows] int32
    case["d_meta"], case["d_values"], case["d_X"] = dev(case["meta"]), dev(case["values"]), dev(case["X"])
    return case


@pytest.fixture(params=[0, 1, 2], ids=["rows-auto", "rows-128", "rows-256"])
def row_halves(request):
    """Weight rows per block of the tcgen05 form: automatic, 128, or 256 (two accumulators on one activation tile)."""
    old = K.set_gemm_row_halves(request.param)
    yield request.param
    K.set_gemm_row_halves(old)


@pytest.mark.parametrize("n", [256, 1024])
def test_gemm_int32_every_element(full_case, n, row_halves):
    c = full_case
    rows, cols = c["rows"], c["cols"]
    before = K.gemm_tc_timeouts()
    Y = Guarded(n * rows * 4)
    K.sparse_ternary_gemm_gpu(c["d_meta"], c["d_values"], c["d_X"], Y.ptr, rows, cols, n, c["meta_stride"],
                              c["values_stride"])
    got = Y.read(np.int32).reshape(n, rows)
    assert (got == c["want"][:n]).all()
    assert K.gemm_tc_timeouts() == before


@pytest.mark.parametrize("rows,cols,n", [(300, 512, 200), (256, 256, 129), (129, 384, 257), (1000, 1024, 300),
                                          (257, 2560, 240), (512, 128, 241)])
def test_two_row_halves_on_ragged_shapes(rows, cols, n):
    # 256-row blocks forced on shapes that do not fill them: row tails in either half, batch tails, one K step
    case = synth.gemm_case(rows, cols, n, seed=rows + n)
    want = oracle.sparse_gemm(case["meta"], case["values"], case["X"], rows, cols)
    before = K.gemm_tc_timeouts()
    old = K.set_gemm_row_halves(2)
    try:
        Y = Guarded(n * rows * 4)
        K.sparse_ternary_gemm_gpu(dev(case["meta"]), dev(case["values"]), dev(case["X"]), Y.ptr, rows, cols, n,
                                  case["meta_stride"], case["values_stride"])
        assert (Y.read(np.int32).reshape(n, rows) == want).all()
        absmax = case["absmax"]
        out = Guarded(n * rows * 2)
        K.sparse_bitlinear_gemm_gpu(dev(case["meta"]), dev(case["values"]), dev(case["X"]), out.ptr, dev(absmax), 0.05,
                                    rows, cols, n, case["meta_stride"], case["values_stride"])
        wh = np.stack([oracle.dequantize(want[j], absmax[j], np.float32(0.05)) for j in range(n)])
        assert (out.read(np.float16).reshape(n, rows).view(np.uint16) == wh.view(np.uint16)).all()
    finally:
        K.set_gemm_row_halves(old)
    assert K.gemm_tc_timeouts() == before


@pytest.mark.parametrize("n", [256, 1024])
def test_bitlinear_gemm_half_every_element(full_case, n, row_halves):
    c = full_case
    rows, cols = c["rows"], c["cols"]
    gamma = np.float32(0.0213)
    absmax = c["absmax"][:n].copy()
    absmax[n // 2] = 0.0  # an all-zero activation row: scale 0
    want = np.stack([oracle.dequantize(c["want"][j], absmax[j], gamma) for j in range(n)])
    before = K.gemm_tc_timeouts()
    out = Guarded(n * rows * 2)
    K.sparse_bitlinear_gemm_gpu(c["d_meta"], c["d_values"], c["d_X"], out.ptr, dev(absmax), gamma, rows, cols, n,
                                c["meta_stride"], c["values_stride"])
    got = out.read(np.float16).reshape(n, rows)
    assert (got.view(np.uint16) == want.view(np.uint16)).all()
    assert K.gemm_tc_timeouts() == before


def test_bounded_wait_runs_out_and_is_reported():
    """A wait of the tcgen05 product that nobody satisfies must end by itself: the block counts it, frees its
    tensor memory and returns, the host sees SPB_E_TIMEOUT, and the next product is exact."""
    before = K.gemm_tc_timeouts()
    for k in range(3):
        rc = K.debug_bounded_wait_selftest(4000)
        assert rc == _lib.SPB_E_TIMEOUT, _lib.load().spb_last_error_string()
        assert K.gemm_tc_timeouts() == before + k + 1
    case = synth.gemm_case(256, 512, 80, seed=5)
    Y = Guarded(80 * 256 * 4)
    K.sparse_ternary_gemm_gpu(dev(case["meta"]), dev(case["values"]), dev(case["X"]), Y.ptr, 256, 512, 80,
                              case["meta_stride"], case["values_stride"])
    want = oracle.sparse_gemm(case["meta"], case["values"], case["X"], 256, 512)
    assert (Y.read(np.int32).reshape(80, 256) == want).all()
    assert K.gemm_tc_timeouts() == before + 3  # the healthy product added nothing


def test_engine_reports_a_run_out_wait():
    """The engine compares the counter at its synchronisation points: a run-out between two of them turns the
    next one into SPB_E_TIMEOUT (once), after which the engine works as before."""
    from spbitnet_b200.engine import DeviceModel, InferenceEngine
    model = synth.random_model(synth.TINY, seed=4)
    eng = InferenceEngine(DeviceModel(model))
    prompt = np.array([5, 17, 300, 41], np.int32)
    first = eng.generate(prompt, 4)
    assert K.debug_bounded_wait_selftest(4000) == _lib.SPB_E_TIMEOUT
    eng.reset()
    with pytest.raises(_lib.SpbError) as err:
        eng.generate(prompt, 4)
    assert err.value.code == _lib.SPB_E_TIMEOUT
    eng.reset()
    assert (eng.generate(prompt, 4) == first).all()


def test_work_list_skips_an_item_wider_than_max_cols():
    """The work-list kernel sizes its shared-memory stages from max_cols; an item with more columns is skipped
    (its y untouched) instead of overrunning them."""
    small = synth.gemv_case(64, 512, seed=1)
    wide = synth.gemv_case(32, 2560, seed=2)
    keep = []
    items = []
    for case in (small, wide, small):
        y = torch.full((case["rows"],), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
        t = (dev(case["meta"]), dev(case["values"]), dev(case["x"]), y)
        keep.append(t)
        items.append((t[0], t[1], t[2], t[3], case["rows"], case["cols"], case["meta_stride"], case["values_stride"]))
    work = K.GemvWorkList(items)
    work.max_cols = 512  # a caller that understates the maximum
    K.sparse_ternary_gemv_batch_gpu(work)
    torch.cuda.synchronize()
    want = oracle.sparse_gemv(small["meta"], small["values"], small["x"], 64, 512)
    assert (keep[0][3].cpu().numpy() == want).all() and (keep[2][3].cpu().numpy() == want).all()
    assert (keep[1][3].cpu().numpy() == 0x5A5A5A5A).all()
