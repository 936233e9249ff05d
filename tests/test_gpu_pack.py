"""GPU pruning + packing against the reference's converter: the golden vectors made by importing
python/convert_model.py (tests/golden/format_py.npz) and a numpy restatement of its five steps."""
import numpy as np
import pytest
import torch

from spbitnet_b200 import kernels as K

pytestmark = pytest.mark.gpu


def converter_steps(wf):
    """python/convert_model.py:88-138, 270-283, 141-207 restated with the same numpy calls."""
    rows, cols = wf.shape
    g = cols // 4
    order = np.argsort(np.abs(wf).reshape(rows, g, 4), axis=-1, kind="stable")
    mask = np.zeros((rows, g, 4), bool)
    np.put_along_axis(mask, order[:, :, -2:], True, axis=-1)
    gamma = float(np.mean(np.abs(wf)))
    tern = np.zeros_like(wf, dtype=np.int8) if gamma < 1e-10 else np.clip(np.round(wf / gamma), -1, 1).astype(np.int8)
    sparse = tern.reshape(rows, g, 4) * mask
    w3 = wf.reshape(rows, g, 4)
    zero = mask & (sparse == 0)
    sparse[zero & (w3 >= 0)] = 1
    sparse[zero & (w3 < 0)] = -1
    bitmaps = np.zeros((rows, g), np.uint32)
    for i in range(4):
        bitmaps |= mask[:, :, i].astype(np.uint32) << i
    cs = np.cumsum(mask, axis=2)
    first = np.any(mask & (cs == 1) & (sparse == -1), axis=2).astype(np.uint32)
    second = np.any(mask & (cs == 2) & (sparse == -1), axis=2).astype(np.uint32)
    signs = first | (second << 1)
    ms, vs = (g + 7) // 8, (g + 15) // 16
    meta = np.zeros((rows, ms), np.uint32)
    values = np.zeros((rows, vs), np.uint32)
    for k in range(g):
        meta[:, k // 8] |= bitmaps[:, k] << np.uint32(4 * (k % 8))
        values[:, k // 16] |= signs[:, k] << np.uint32(2 * (k % 16))
    return meta, values, gamma


def run(wf):
    meta, values, gamma = K.prune_pack_gpu(torch.from_numpy(wf).cuda())
    torch.cuda.synchronize()
    return meta.cpu().numpy().view(np.uint32), values.cpu().numpy().view(np.uint32), gamma


def test_matches_the_converters_own_output(golden):
    g = golden("format_py.npz")  # ties, an all-zero group, ordinary weights: made by the reference's Python
    meta, values, gamma = run(g["weights_f32"])
    assert (meta == g["meta"]).all() and (values == g["values"]).all()
    assert abs(gamma - float(g["gamma"])) <= 1e-6 * float(g["gamma"])


@pytest.mark.parametrize("rows,cols", [(1, 4), (3, 60), (17, 132), (64, 256), (300, 2560), (128, 6912)])
def test_matches_the_restated_steps(rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    wf = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    wf[rng.random((rows, cols)) < 0.05] = 0.0                      # exact zeros, also negative zero
    wf[rng.random((rows, cols)) < 0.02] = -0.0
    q = rng.random((rows, cols)) < 0.1                               # many magnitude ties
    wf[q] = np.sign(wf[q]) * np.float32(0.0125)
    meta, values, gamma = run(wf)
    wm, wv, wg = converter_steps(wf)
    assert (meta == wm).all() and (values == wv).all()
    assert abs(gamma - wg) <= 1e-6 * max(wg, 1e-30)


def test_strided_input_and_bad_arguments():
    from spbitnet_b200 import _lib
    big = torch.randn(8, 300, device="cuda")
    view = big[:, 4:260]  # row stride 300, 16-byte aligned start
    meta, values, _ = K.prune_pack_gpu(view)
    wm, wv, _ = converter_steps(view.cpu().numpy().copy())
    assert (meta.cpu().numpy().view(np.uint32) == wm).all() and (values.cpu().numpy().view(np.uint32) == wv).all()
    odd = big[:, 1:257]   # unaligned rows take the scalar loads
    meta, values, _ = K.prune_pack_gpu(odd)
    wm, wv, _ = converter_steps(odd.cpu().numpy().copy())
    assert (meta.cpu().numpy().view(np.uint32) == wm).all() and (values.cpu().numpy().view(np.uint32) == wv).all()
    lib = _lib.load()
    assert lib.spb_prune_pack_gpu(big.data_ptr(), 8, 302, 302, big.data_ptr(), big.data_ptr(), 10, 5, None, None) != 0
    assert lib.spb_prune_pack_gpu(big.data_ptr(), 8, 256, 300, big.data_ptr(), big.data_ptr(), 7, 4, None, None) != 0
    assert lib.spb_prune_pack_gpu(big.data_ptr(), 0, 256, 300, None, None, 8, 4, None, None) == 0
