"""The allocation-free attention entry point against the caller-scratch one.

spb_decode_attention_noalloc exists for callers that cannot make room for the split-KV partial
results: an engine with a fixed buffer plan, code inside a stream capture, a serving loop that must
not stall the GPU on cudaMalloc.  It keeps the partial results in an array inside the library.
Here it is called through the C-ABI twice in a row (the second time with other inputs and a
shorter sequence, so stale partial results from the first call are lying in the array) and must
give exactly what spb_decode_attention_split gives with a fresh caller-owned buffer.  Collected
last on purpose: a run that stops at the first failure has then already run everything else."""
import ctypes as C

import numpy as np
import pytest
import torch

from spbitnet_b200 import _lib
from gpu_util import Guarded, dev

pytestmark = pytest.mark.gpu


def _inputs(nh, nkv, hd, mx, sl, seed):
    r = np.random.default_rng(seed)
    Q = r.standard_normal(nh * hd).astype(np.float16)
    Kc = np.zeros((nkv, mx, hd), np.float16)
    Vc = np.zeros((nkv, mx, hd), np.float16)
    Kc[:, :sl] = r.standard_normal((nkv, sl, hd)).astype(np.float16)
    Vc[:, :sl] = r.standard_normal((nkv, sl, hd)).astype(np.float16)
    return dev(Q), dev(Kc), dev(Vc)


def _p(t):
    return C.c_void_p(t if isinstance(t, int) else t.data_ptr())


def test_noalloc_matches_caller_scratch_twice_in_a_row():
    lib = _lib.load()
    nh, nkv, hd, mx = 20, 5, 128, 4096
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.spb_decode_attention_scratch_bytes(nh, hd, mx)
    assert 0 < need <= lib.spb_decode_attention_noalloc_capacity()
    for call, (sl, seed) in enumerate([(1500, 1), (130, 2)]):
        Q, Kc, Vc = _inputs(nh, nkv, hd, mx, sl, seed)
        scale = 1.0 / np.sqrt(hd)
        scratch = torch.full((need // 4,), float("nan"), dtype=torch.float32, device="cuda")
        want = Guarded(nh * hd * 2)
        _lib.check(lib.spb_decode_attention_split(_p(Q), _p(Kc), _p(Vc), _p(want.ptr), nh, nkv, hd, mx, sl,
                                                  C.c_float(scale), _p(scratch), need, stream))
        got = Guarded(nh * hd * 2)
        _lib.check(lib.spb_decode_attention_noalloc(_p(Q), _p(Kc), _p(Vc), _p(got.ptr), nh, nkv, hd, mx, sl,
                                                    C.c_float(scale), stream))
        a, b = got.read(np.uint16), want.read(np.uint16)
        assert np.isfinite(a.view(np.float16)).all(), call
        # same kernels, same order of operations: the tolerance of the attention tests (1e-3) is met with zero slack
        assert (a == b).all(), call


def test_noalloc_refuses_what_does_not_fit():
    lib = _lib.load()
    nh, nkv, hd, mx = 64, 8, 128, 16384  # 64 heads * 512 chunks * 130 floats = 17 MB of partial results
    assert lib.spb_decode_attention_scratch_bytes(nh, hd, mx) > lib.spb_decode_attention_noalloc_capacity()
    dummy = torch.zeros(16, dtype=torch.float16, device="cuda")
    rc = lib.spb_decode_attention_noalloc(_p(dummy), _p(dummy), _p(dummy), _p(dummy), nh, nkv, hd, mx, 1,
                                          C.c_float(1.0), C.c_void_p(0))
    assert rc == _lib.SPB_E_UNSUPPORTED
    msg = lib.spb_last_error_string().decode()
    assert "built-in scratch holds" in msg and "spb_decode_attention_split" in msg
