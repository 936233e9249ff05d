"""The drop-in claim, executed: code written against the reference's C++ API runs unchanged on this library.
  * a program that uses only the reference's SparseTernaryTensor header and spbitnet::sparse_ternary_gemv_gpu,
    compiled against include/spbitnet/*.h of this repository and linked with libspbitnet_b200.so, reproduces the
    reference's seeded exact-equality GEMV tests (tests/test_sparse_ternary.cu:252-402);
  * the reference's own InferenceEngine and Model::load (src/inference.cu, src/model.cu, unmodified) built the
    same way decode a model directory written by spbitnet_b200.model_io with the logits of the CPU oracle.
Both binaries are built by oracle/Makefile where the reference tree is present and travel in oracle/_ref."""
import subprocess

import numpy as np
import pytest

import oracle
from spbitnet_b200 import model_io, synth
from spbitnet_b200.engine import DeviceModel, InferenceEngine

pytestmark = pytest.mark.gpu


def test_reference_style_program_links_and_is_exact():
    if not oracle.DROPIN_GEMV_TEST.exists():
        pytest.skip("oracle/_ref/dropin_gemv_test not built")
    res = subprocess.run([str(oracle.DROPIN_GEMV_TEST)], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("exact") == 2


@pytest.mark.parametrize("cfg_name", ["tiny", "wide"])
def test_reference_engine_runs_on_these_kernels(tmp_path, cfg_name):
    if oracle.dropin() is None:
        pytest.skip("oracle/_ref/libspb_dropin.so not built")
    cfg = synth.TINY if cfg_name == "tiny" else dict(synth.BITNET_2B, num_hidden_layers=2, vocab_size=4096,
                                                     max_position_embeddings=64)
    # the wide model is drawn on the GPU (seconds with numpy) and brought back for the directory writer
    model = synth.random_model(cfg, seed=7) if cfg_name == "tiny" else synth.DeviceRandomModel(cfg, seed=7).to_host()
    ref_engine = oracle.DropInEngine(model_io.save_model_dir(model, tmp_path / "m"))
    ours = InferenceEngine(DeviceModel(model))
    cpu = oracle.Engine(model) if cfg_name == "tiny" else None
    tokens = [3, 99, 420, 17, 250, 8]
    for step, t in enumerate(tokens):
        a = ref_engine.forward(t)          # reference host code, this library's op-by-op kernels
        ours.forward(t)
        b = ours.logits()                  # this library's engine (fused kernels, CUDA graph)
        assert np.abs(a - b).max() < 1e-2, step
        assert int(np.argmax(a)) == int(np.argmax(b)), step
        if cpu is not None:
            c = cpu.forward(t)
            assert np.abs(a - c).max() < 1e-2 and int(np.argmax(a)) == int(np.argmax(c)), step
    assert ref_engine.seq_len == len(tokens)
