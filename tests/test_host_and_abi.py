"""CPU-only checks of the product's host side: the C-ABI library loads and exports every
symbol the header declares, the host packers equal the oracle bit for bit, argument errors
come back as status codes.  No kernel is launched here."""
import re
from pathlib import Path

import numpy as np
import pytest

import oracle
from spbitnet_b200 import _lib, format as F, synth

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    header = (ROOT / "include" / "spbitnet_b200.h").read_text()
    declared = set(re.findall(r"\b(spb_[a-z0-9_]+)\s*\(", header))
    declared -= {"spb_engine", "spb_model_config"}
    assert declared, "no declarations parsed"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert b"sm_100a" in lib.spb_version()


def test_cpp_dropin_headers_name_the_reference_functions():
    ref_names = ["sparse_ternary_unpack_gpu", "sparse_ternary_gemv_gpu", "fused_sparse_bitlinear_gpu",
                 "rms_norm_gpu", "absmax_quantize_gpu", "absmax_reduce_gpu", "dequantize_gpu", "rope_gpu",
                 "scatter_kv_gpu", "attention_scores_gpu", "softmax_gpu", "attention_output_gpu", "relu2_mul_gpu",
                 "relu2_mul_f32_gpu", "rms_norm_f32in_gpu", "float_to_half_gpu", "residual_add_gpu", "half_gemv_gpu"]
    text = "".join(p.read_text() for p in (ROOT / "include" / "spbitnet").glob("*.h"))
    from spbitnet_b200 import kernels
    for n in ref_names:
        assert re.search(rf"\b{n}\s*\(", text), n
        assert hasattr(kernels, n), n


@pytest.mark.parametrize("rows,cols", [(1, 4), (2, 8), (3, 36), (7, 132), (16, 256), (5, 2560)])
def test_host_packers_equal_oracle(rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    w, mask = synth.ternary_weights_and_mask(rows, cols, rng)
    t = F.SparseTernaryTensor.pack_from_dense(w, mask)
    om, ov = oracle.pack_from_dense(w, mask)
    assert (t.meta == om).all() and (t.values == ov).all()
    assert (t.unpack_to_int8() == oracle.unpack_to_int8(om, ov, rows, cols)).all()
    nm, nv = synth.pack_numpy(w, mask)
    assert (nm == om).all() and (nv == ov).all()
    lat = rng.standard_normal((rows, cols)).astype(np.float32)
    lat[:, ::5] = -0.5
    lat[:, 1::9] = lat[:, ::9][:, : lat[:, 1::9].shape[1]]
    p = F.SparseTernaryTensor.pack_with_pruning(lat)
    pm, pv = oracle.pack_with_pruning(lat)
    assert (p.meta == pm).all() and (p.values == pv).all()
    t.validate()


def test_host_packers_golden(golden):
    g = golden("format_py.npz")
    t = F.SparseTernaryTensor.pack_from_dense(g["sparse"], g["mask"])
    assert (t.meta == g["meta"]).all() and (t.values == g["values"]).all()
    r = golden("format_ref.npz")
    p = F.SparseTernaryTensor.pack_with_pruning(r["latent"])
    assert (p.meta == r["pmeta"]).all() and (p.values == r["pvalues"]).all()


def test_synthetic_distribution():
    w, mask = synth.ternary_weights_and_mask(256, 1024, np.random.default_rng(0))
    assert abs((w == 0).mean() - 0.42) < 0.01 and abs((w == 1).mean() - 0.29) < 0.01
    assert (mask.reshape(256, 256, 4).sum(-1) == 2).all()
    kept_nz = (mask & (w != 0)).reshape(256, 256, 4).sum(-1)
    all_nz = (w != 0).reshape(256, 256, 4).sum(-1)
    assert (kept_nz == np.minimum(all_nz, 2)).all()  # never drops a non-zero while a zero is kept
    assert synth.gemv_algorithmic_bytes(6912, 2560) == 3347968
    assert synth.gemv_algorithmic_bytes(2560, 2560) == 1241600


def test_errors_are_status_codes():
    lib = _lib.load()
    with pytest.raises(_lib.SpbError) as ei:
        F.SparseTernaryTensor.pack_from_dense(np.ones((1, 4), np.int8), np.array([[1, 1, 1, 0]], np.uint8))
    assert ei.value.code == _lib.SPB_E_FORMAT and "keeps 3" in str(ei.value)
    bad = F.SparseTernaryTensor(1, 8, np.array([[0x71]], np.uint32), np.zeros((1, 1), np.uint32))
    with pytest.raises(_lib.SpbError):
        bad.validate()
    # argument checks that return before any CUDA call
    assert lib.spb_sparse_ternary_gemv(None, None, None, None, 0, 16, 1, 1, None) == 0  # rows == 0: silent
    assert lib.spb_sparse_ternary_gemv(None, None, None, None, 4, 6, 1, 1, None) == _lib.SPB_E_INVALID
    assert b"multiple of 4" in lib.spb_last_error_string()
    assert lib.spb_sparse_ternary_gemv(None, None, None, None, 4, 8, 1, 1, None) == _lib.SPB_E_INVALID
    assert lib.spb_rope(None, 2, 7, 0, 1e4, None) == _lib.SPB_E_INVALID
    assert lib.spb_engine_seq_len(None) == 0
