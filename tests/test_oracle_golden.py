"""Pins the CPU oracle (oracle/spb_oracle.c) to the reference: its own header run through
oracle/_ref when that was built, the golden vectors generated from its Python code and
header (tests/golden/make_golden.py), and the known-answer cases in its tests and docs."""
import hashlib

import numpy as np
import pytest

import oracle


# ---- known answers written in the reference's tests and docs -----------------------------

def test_pack_with_pruning_known_answer():
    # tests/test_sparse_ternary.cu:115-141 (PackWithPruning)
    latent = np.array([[0.1, -0.9, 0.8, -0.2, -0.7, 0.3, -0.6, 0.05],
                       [0.95, -0.1, 0.02, -0.85, -0.4, 0.9, -0.8, 0.3]], np.float32)
    meta, values = oracle.pack_with_pruning(latent)
    got = oracle.unpack_to_int8(meta, values, 2, 8)
    want = np.array([[0, -1, 1, 0, -1, 0, -1, 0], [1, 0, 0, -1, 0, 1, -1, 0]], np.int8)
    assert (got == want).all()


def test_docs_worked_example():
    # docs/compression_format.md:229-261: [0,+1,0,-1] -> bitmap 0xA, signs 0x2
    w = np.array([[0, 1, 0, -1]], np.int8)
    mask = np.array([[0, 1, 0, 1]], np.uint8)
    meta, values = oracle.pack_from_dense(w, mask)
    assert meta[0, 0] == 0xA and values[0, 0] == 0x2
    assert (oracle.unpack_to_int8(meta, values, 1, 4) == w).all()


def test_roundtrip_mask_02():
    # tests/test_sparse_ternary.cu:38-84 (PackFromDenseRoundtrip): keep positions 0 and 2
    rows, cols = 4, 32
    w = np.tile(np.array([1, -1, 1, -1], np.int8), rows * cols // 4).reshape(rows, cols)
    mask = np.tile(np.array([1, 0, 1, 0], np.uint8), rows * cols // 4).reshape(rows, cols)
    got = oracle.unpack_to_int8(*oracle.pack_from_dense(w, mask), rows, cols)
    assert (got == w * mask).all()


def test_compression_ratio():
    # tests/test_sparse_ternary.cu:149-179: 1.5 bits/weight = 75 % of dense 2-bit
    cols = 1024
    sparse_words = oracle.meta_words_per_row(cols) + oracle.values_words_per_row(cols)
    dense_words = (cols + 15) // 16
    assert 0.70 <= sparse_words / dense_words <= 0.80


def test_kept_zero_packs_as_plus_one():
    # include/spbitnet/sparse_ternary_tensor.h:86-91
    w = np.array([[0, 0, -1, 0]], np.int8)
    mask = np.array([[1, 0, 1, 0]], np.uint8)
    got = oracle.unpack_to_int8(*oracle.pack_from_dense(w, mask), 1, 4)
    assert got.tolist() == [[1, 0, -1, 0]]


def test_attention_known_answer():
    # tests/test_inference_kernels.cu:376-454 (AttentionSingleHead)
    hd, mx, sl = 4, 8, 3
    Q = np.array([1, 0, 1, 0], np.float16)
    K = np.zeros((1, mx, hd), np.float16)
    K[0, 0, 0] = 1
    K[0, 1, 1] = K[0, 1, 3] = 1
    K[0, 2, 0] = K[0, 2, 2] = 1
    V = np.zeros((1, mx, hd), np.float16)
    V[0, 0, 0], V[0, 1, 1], V[0, 2, 2] = 10, 20, 30
    s = oracle.attention_scores(Q, K, 1, 1, hd, mx, sl, 0.5)
    assert np.allclose(s[0, :3], [0.5, 0.0, 1.0], atol=1e-3)
    p = oracle.softmax(s, sl)
    assert abs(p[0, :3].sum() - 1) < 1e-4 and p[0, 2] > p[0, 0] > p[0, 1]
    out = oracle.attention_output(p, V, 1, 1, hd, mx, sl).astype(np.float32)
    assert np.allclose(out, [p[0, 0] * 10, p[0, 1] * 20, p[0, 2] * 30, 0], atol=0.1)


def test_scatter_kv_known_answer():
    # tests/test_inference_kernels.cu:460-494
    src = np.arange(1, 9, dtype=np.float16)
    cache = oracle.scatter_kv(src, np.zeros((2, 8, 4), np.float16), 2, 4, 8, 3).reshape(2, 8, 4)
    assert cache[0, 3].tolist() == [1, 2, 3, 4] and cache[1, 3].tolist() == [5, 6, 7, 8]
    assert cache.sum() == 36


def test_quantize_ties_to_even_and_clamp():
    # src/kernels/inference_kernels.cu:105-112: __float2int_rn rounds half to even
    x = np.array([127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -127.0], np.float16)
    q, absmax = oracle.absmax_quantize(x)
    assert absmax == 127.0
    assert q.tolist() == [127, 0, 2, 2, 0, -2, -127]
    q0, a0 = oracle.absmax_quantize(np.zeros(8, np.float16))
    assert a0 == 0 and not q0.any()  # scale 0 when absmax 0 (:103)


# ---- golden vectors generated from the reference -----------------------------------------

def test_python_packer_golden(golden):
    g = golden("format_py.npz")
    meta, values = oracle.pack_from_dense(g["sparse"], g["mask"])
    assert (meta == g["meta"]).all() and (values == g["values"]).all()
    assert meta.shape[1] == int(g["meta_stride"]) and values.shape[1] == int(g["values_stride"])
    assert (oracle.unpack_to_int8(meta, values, *g["sparse"].shape) == g["sparse"]).all()


def test_reference_header_golden(golden):
    g = golden("format_ref.npz")
    meta, values = oracle.pack_from_dense(g["w42"], g["m42"])
    assert (meta == g["meta42"]).all() and (values == g["values42"]).all()
    assert (oracle.unpack_to_int8(meta, values, 64, 256) == g["dense42"]).all()
    # GemvCorrectness, 64x256 seed 42 (tests/test_sparse_ternary.cu:252-324)
    assert (oracle.sparse_gemv(meta, values, g["x42"], 64, 256) == g["y42"]).all()
    pm, pv = oracle.pack_with_pruning(g["latent"])
    assert (pm == g["pmeta"]).all() and (pv == g["pvalues"]).all()


def test_reference_large_gemv_golden(golden):
    # GemvLargeDimension, 2048x2048 seed 77 (tests/test_sparse_ternary.cu:330-402)
    g = golden("format_ref.npz")
    w, m, x = oracle.testgen_gemv_case(77, 2048, 2048, -5, 5)
    if hashlib.sha256(w.tobytes() + m.tobytes() + x.tobytes()).hexdigest() != str(g["sha77"]):
        pytest.skip("this libstdc++ draws a different mt19937/shuffle sequence than the one the golden was made with")
    meta, values = oracle.pack_from_dense(w, m)
    assert (oracle.sparse_gemv(meta, values, x, 2048, 2048) == g["y77"]).all()
    assert (oracle.sparse_gemv(meta, values, x, 2048, 2048, threads=4) == g["y77"]).all()


@pytest.mark.skipif(oracle.ref() is None, reason="oracle/_ref not built (no reference tree)")
def test_against_reference_header_live():
    rng = np.random.default_rng(1)
    from spbitnet_b200 import synth
    for rows, cols in [(1, 4), (3, 36), (5, 260), (17, 64), (9, 2560)]:
        w, mask = synth.ternary_weights_and_mask(rows, cols, rng)
        assert all((a == b).all() for a, b in zip(oracle.pack_from_dense(w, mask), oracle.ref_pack_from_dense(w, mask)))
        x = rng.integers(-128, 128, cols, dtype=np.int8)
        meta, values = oracle.pack_from_dense(w, mask)
        assert (oracle.sparse_gemv(meta, values, x, rows, cols) == oracle.ref_cpu_sparse_gemv(w, mask, x)).all()
        lat = rng.standard_normal((rows, cols)).astype(np.float32)
        lat[:, ::7] = 0.5
        assert all((a == b).all() for a, b in zip(oracle.pack_with_pruning(lat), oracle.ref_pack_with_pruning(lat)))


def _close(a, b, rtol, atol):
    return np.allclose(np.asarray(a, np.float32), np.asarray(b, np.float32), rtol=rtol, atol=atol)


def test_ops_against_baseline_pytorch(golden):
    g = golden("ops_py.npz")
    assert _close(oracle.rms_norm(g["norm_x"], g["norm_w"], 1e-5), g["norm_y"], 1e-3, 1e-3)
    assert _close(oracle.rms_norm_f32in(g["normf_x"], g["normf_w"], 1e-5), g["normf_y"], 1e-3, 1e-3)
    assert _close(oracle.rope(g["rope_x"], 4, 128, 37, 500000.0), g["rope_y"], 1e-3, 2e-3)
    y = oracle.attention(g["attn_q"], g["attn_k"], g["attn_v"], 4, 2, 64, 32, 19, 1.0 / 8.0)
    assert _close(y, g["attn_y"], 1e-3, 2e-3)
    assert (oracle.relu2_mul_f32(g["relu_g"], g["relu_u"]) == g["relu_y"]).all()
    assert _close(oracle.half_gemv(g["hg_w"], g["hg_x"]), g["hg_y"], 1e-4, 1e-4)
    # BitLinear: the Python reference forms its scales in float64, the CUDA source (which the
    # oracle follows) in fp32, so the half outputs may differ in the last place.
    from spbitnet_b200 import synth
    case = synth.gemv_case(64, 256, seed=11)
    absmax = oracle.absmax_reduce(g["bl_x"])
    y = oracle.fused_bitlinear(case["meta"], case["values"], g["bl_x"], absmax, g["bl_gamma"], 64, 256)
    assert _close(y, g["bl_y"], 2e-3, 1e-4)


def test_engine_against_baseline_pytorch(golden):
    g = golden("engine_py.npz")
    from spbitnet_b200 import synth
    model = synth.random_model(synth.TINY, seed=int(g["seed"]))
    eng = oracle.Engine(model)
    tokens, logits = eng.generate(g["prompt"], len(g["tokens"]))
    assert np.abs(np.stack(logits) - g["logits"]).max() < 1e-2
    assert (tokens == g["tokens"]).all()


def test_fused_equals_unfused():
    # fused_sparse_bitlinear_gpu == absmax_quantize -> gemv -> dequantize (src/inference.cu:106-117)
    from spbitnet_b200 import synth
    case = synth.gemv_case(32, 512, seed=2)
    x = (np.random.default_rng(0).standard_normal(512) * 3).astype(np.float16)
    q, absmax = oracle.absmax_quantize(x)
    acc = oracle.sparse_gemv(case["meta"], case["values"], q, 32, 512)
    a = oracle.dequantize(acc, absmax, 0.02)
    b = oracle.fused_bitlinear(case["meta"], case["values"], x, absmax, 0.02, 32, 512)
    assert (a.view(np.uint16) == b.view(np.uint16)).all()
