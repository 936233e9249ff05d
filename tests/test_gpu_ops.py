"""GPU parity of the decode-step kernels against the CPU oracle, through the C-ABI.
Tolerances: int8 quantised activations bit-exact; norm / softmax / attention / rope within
1e-3 relative (of the vector's scale); exact ops bit for bit."""
import numpy as np
import pytest
import torch

import oracle
from spbitnet_b200 import kernels as K
from gpu_util import Guarded, dev, host

pytestmark = pytest.mark.gpu
RTOL = 1e-3


def close(got, want, rtol=RTOL):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    scale = max(np.abs(want).max(), 1e-6)
    # one half ulp of slack on top of the relative bound: both sides round to half
    return np.abs(got - want).max() <= rtol * scale + np.abs(want).max() * 2.0 ** -10


@pytest.mark.parametrize("n", [64, 2560, 6912, 1000, 8192])
def test_rms_norm(n):
    # tests/test_inference_kernels.cu:51-117
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 1.3).astype(np.float16)
    w = (1 + 0.02 * rng.standard_normal(n)).astype(np.float32)
    out = Guarded(n * 2)
    K.rms_norm_gpu(dev(x), dev(w), out.ptr, n, 1e-5)
    assert close(out.read(np.float16), oracle.rms_norm(x, w, 1e-5))
    xd = dev(x)
    K.rms_norm_gpu(xd, dev(w), xd, n, 1e-5)  # in place, as src/inference.cu:212 uses it
    assert close(host(xd), oracle.rms_norm(x, w, 1e-5))
    xf = (rng.standard_normal(n) * 500).astype(np.float32)
    out = Guarded(n * 2)
    K.rms_norm_f32in_gpu(dev(xf), dev(w), out.ptr, n, 1e-5)
    assert close(out.read(np.float16), oracle.rms_norm_f32in(xf, w, 1e-5))


@pytest.mark.parametrize("n", [1, 100, 2560, 6912])
def test_absmax_quantize_bit_exact(n):
    # tests/test_inference_kernels.cu:123-182 only bounds q within 1.5; the contract here is exact
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 2).astype(np.float16)
    x[0] = np.float16(6.5)
    q_want, a_want = oracle.absmax_quantize(x)
    q, a = Guarded(n), Guarded(4)
    K.absmax_quantize_gpu(dev(x), q.ptr, a.ptr, n)
    assert a.read(np.float32)[0] == a_want
    assert (q.read(np.int8) == q_want).all()
    a2 = Guarded(4)
    K.absmax_reduce_gpu(dev(x), a2.ptr, n)
    assert a2.read(np.float32)[0] == a_want
    # exact halves exercise round-half-to-even
    t = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, -127.0], np.float16)
    q, a = Guarded(8), Guarded(4)
    K.absmax_quantize_gpu(dev(t), q.ptr, a.ptr, 8)
    assert q.read(np.int8).tolist() == [127, 0, 2, 2, 0, -2, -2, -127]


def test_dequantize_exact():
    rng = np.random.default_rng(0)
    acc = rng.integers(-200000, 200000, 2560, dtype=np.int32)
    out = Guarded(2560 * 2)
    K.dequantize_gpu(dev(acc), out.ptr, dev(np.array([3.11], np.float32)), 0.0271, 2560)
    assert (out.read(np.uint16) == oracle.dequantize(acc, 3.11, 0.0271).view(np.uint16)).all()


@pytest.mark.parametrize("heads,hd,pos,theta", [(2, 8, 3, 10000.0), (20, 128, 383, 500000.0), (5, 128, 0, 500000.0),
                                                 (64, 128, 575, 500000.0)])
def test_rope(heads, hd, pos, theta):
    # tests/test_inference_kernels.cu:188-226
    v = np.random.default_rng(pos).standard_normal(heads * hd).astype(np.float16)
    d = dev(v)
    K.rope_gpu(d, heads, hd, pos, theta)
    assert close(host(d), oracle.rope(v, heads, hd, pos, theta))


def test_scatter_kv():
    # tests/test_inference_kernels.cu:460-494
    src = np.arange(1, 9, dtype=np.float16)
    cache = dev(np.zeros((2, 8, 4), np.float16))
    K.scatter_kv_gpu(dev(src), cache, 2, 4, 8, 3)
    assert (host(cache) == oracle.scatter_kv(src, np.zeros((2, 8, 4), np.float16), 2, 4, 8, 3).reshape(2, 8, 4)).all()


def _attn_inputs(nh, nkv, hd, mx, sl, seed):
    r = np.random.default_rng(seed)
    Q = r.standard_normal(nh * hd).astype(np.float16)
    Kc = np.zeros((nkv, mx, hd), np.float16)
    Vc = np.zeros((nkv, mx, hd), np.float16)
    Kc[:, :sl] = r.standard_normal((nkv, sl, hd)).astype(np.float16)
    Vc[:, :sl] = r.standard_normal((nkv, sl, hd)).astype(np.float16)
    return Q, Kc, Vc


def test_attention_known_answer():
    # tests/test_inference_kernels.cu:376-454
    hd, mx, sl = 4, 8, 3
    Q = np.array([1, 0, 1, 0], np.float16)
    Kc = np.zeros((1, mx, hd), np.float16)
    Kc[0, 0, 0] = 1
    Kc[0, 1, 1] = Kc[0, 1, 3] = 1
    Kc[0, 2, 0] = Kc[0, 2, 2] = 1
    Vc = np.zeros((1, mx, hd), np.float16)
    Vc[0, 0, 0], Vc[0, 1, 1], Vc[0, 2, 2] = 10, 20, 30
    s = dev(np.zeros((1, mx), np.float32))
    K.attention_scores_gpu(dev(Q), dev(Kc), s, 1, 1, hd, mx, sl, 0.5)
    assert np.allclose(host(s)[0, :3], [0.5, 0.0, 1.0], atol=1e-3)
    K.softmax_gpu(s, 1, mx, sl)
    p = host(s)[0]
    assert abs(p[:3].sum() - 1) < 1e-4 and p[2] > p[0] > p[1]
    out = Guarded(hd * 2)
    K.attention_output_gpu(s, dev(Vc), out.ptr, 1, 1, hd, mx, sl)
    assert np.allclose(out.read(np.float16).astype(np.float32), [p[0] * 10, p[1] * 20, p[2] * 30, 0], atol=0.1)


@pytest.mark.parametrize("nh,nkv,hd,mx,sl", [(4, 2, 64, 32, 19), (20, 5, 128, 4096, 384), (20, 5, 128, 640, 1),
                                              (64, 8, 128, 1024, 577), (3, 3, 40, 16, 16), (20, 5, 128, 4096, 4096),
                                              (8, 2, 128, 300, 129), (6, 2, 256, 260, 257)])
def test_attention_three_kernels_and_fused(nh, nkv, hd, mx, sl):
    Q, Kc, Vc = _attn_inputs(nh, nkv, hd, mx, sl, sl)
    scale = 1.0 / np.sqrt(hd)
    s_want = oracle.attention_scores(Q, Kc, nh, nkv, hd, mx, sl, scale)
    p_want = oracle.softmax(s_want, sl)
    o_want = oracle.attention_output(p_want, Vc, nh, nkv, hd, mx, sl)
    s = dev(np.zeros((nh, mx), np.float32))
    K.attention_scores_gpu(dev(Q), dev(Kc), s, nh, nkv, hd, mx, sl, scale)
    assert close(host(s)[:, :sl], s_want[:, :sl])
    K.softmax_gpu(s, nh, mx, sl)
    assert close(host(s)[:, :sl], p_want[:, :sl]) and np.allclose(host(s)[:, :sl].sum(1), 1, atol=1e-4)
    out = Guarded(nh * hd * 2)
    K.attention_output_gpu(s, dev(Vc), out.ptr, nh, nkv, hd, mx, sl)
    assert close(out.read(np.float16), o_want)
    out2 = Guarded(nh * hd * 2)
    K.decode_attention_gpu(dev(Q), dev(Kc), dev(Vc), out2.ptr, nh, nkv, hd, mx, sl, scale)
    assert close(out2.read(np.float16), o_want)
    # split-KV form with caller-provided scratch (poisoned: it must need no initialisation)
    nbytes = K.decode_attention_scratch_bytes(nh, hd, mx)
    scratch = torch.full((nbytes // 4 + 8,), float("nan"), dtype=torch.float32, device="cuda")
    for _ in range(2):
        out3 = Guarded(nh * hd * 2)
        K.decode_attention_split_gpu(dev(Q), dev(Kc), dev(Vc), out3.ptr, nh, nkv, hd, mx, sl, scale, scratch[:nbytes // 4])
        assert close(out3.read(np.float16), o_want)
    assert torch.isnan(scratch[nbytes // 4:]).all()


def test_elementwise_exact():
    rng = np.random.default_rng(0)
    n = 6912
    g = (rng.standard_normal(n) * 4).astype(np.float16)
    u = (rng.standard_normal(n) * 4).astype(np.float16)
    o = Guarded(n * 2)
    K.relu2_mul_gpu(dev(g), dev(u), o.ptr, n)
    assert (o.read(np.uint16) == oracle.relu2_mul(g, u).view(np.uint16)).all()
    of = Guarded(n * 4)
    K.relu2_mul_f32_gpu(dev(g), dev(u), of.ptr, n)
    assert (of.read(np.float32) == oracle.relu2_mul_f32(g, u)).all()
    big = (g.astype(np.float32) * 300) ** 2  # beyond the half range: the fp32 path must keep it
    oh = Guarded(n * 2)
    K.float_to_half_gpu(dev(big), oh.ptr, n)
    assert (oh.read(np.uint16) == oracle.float_to_half(big).view(np.uint16)).all()
    orr = Guarded(n * 2)
    K.residual_add_gpu(dev(g), dev(u), orr.ptr, n)
    assert (orr.read(np.uint16) == oracle.residual_add(g, u).view(np.uint16)).all()


@pytest.mark.parametrize("rows,cols", [(32, 64), (48, 200), (1001, 2560), (7, 13)])
def test_half_gemv(rows, cols):
    # tests/test_inference_kernels.cu:339-370
    rng = np.random.default_rng(rows)
    W = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float16)
    x = rng.standard_normal(cols).astype(np.float16)
    y = Guarded(rows * 4)
    K.half_gemv_gpu(dev(W), dev(x), y.ptr, rows, cols)
    want = oracle.half_gemv(W, x)
    assert np.abs(y.read(np.float32) - want).max() <= 1e-3 * max(np.abs(want).max(), 1.0)
