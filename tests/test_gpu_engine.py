"""End-to-end parity of the decode engine against the CPU oracle engine: logits within 1e-2
max-abs and identical greedy tokens, on random-init models (tiny, and a 2B-4T-width model with
few layers so the CPU side finishes in seconds)."""
import numpy as np
import pytest
import torch

import oracle
from spbitnet_b200 import synth
from spbitnet_b200.engine import DeviceModel, InferenceEngine

pytestmark = pytest.mark.gpu


def test_tiny_model_matches_oracle_and_reference_python(golden):
    g = golden("engine_py.npz")
    model = synth.random_model(synth.TINY, seed=int(g["seed"]))
    eng = InferenceEngine(DeviceModel(model))
    cpu = oracle.Engine(model)
    prompt = g["prompt"]
    # token-by-token forward(), the reference's call pattern (src/main.cpp:266-300)
    for t in prompt[:-1]:
        eng.forward(int(t))
        cpu.forward(int(t))
    tok = int(prompt[-1])
    for step in range(len(g["tokens"])):
        eng.forward(tok)
        lg = eng.logits()
        want = cpu.forward(tok)
        assert np.abs(lg - want).max() < 1e-2, step
        assert np.abs(lg - g["logits"][step]).max() < 1e-2, step  # baseline_pytorch.InferenceEngine
        tok = int(np.argmax(lg))
        assert tok == oracle.argmax(want) == int(g["tokens"][step])
    assert eng.seq_len == len(prompt) - 1 + len(g["tokens"])
    # the greedy loop with the device arg-max gives the same tokens
    eng.reset()
    assert eng.seq_len == 0
    assert (eng.generate(prompt, len(g["tokens"])) == g["tokens"]).all()
    # and again after a reset (KV cache cleared, graph reused)
    eng.reset()
    assert (eng.generate(prompt, len(g["tokens"])) == g["tokens"]).all()


def test_generate_stops_at_eos():
    model = synth.random_model(synth.TINY, seed=1)
    eng = InferenceEngine(DeviceModel(model))
    prompt = np.array([5, 17, 200], np.int32)
    full = eng.generate(prompt, 12)
    eng.reset()
    stop = eng.generate(prompt, 12, eos_token_id=int(full[4]))
    first = int(np.where(full == full[4])[0][0])
    assert (stop == full[: first + 1]).all()


def test_wide_model_few_layers():
    cfg = dict(synth.BITNET_2B, num_hidden_layers=2, vocab_size=8192, max_position_embeddings=64)
    model = synth.random_model(cfg, seed=3)
    eng = InferenceEngine(DeviceModel(model))
    cpu = oracle.Engine(model)
    prompt = np.random.default_rng(0).integers(0, cfg["vocab_size"], 4).astype(np.int32)
    want_tokens, want_logits = cpu.generate(prompt, 6)
    for t in prompt[:-1]:
        eng.forward(int(t))
    tok = int(prompt[-1])
    for step in range(6):
        eng.forward(tok)
        lg = eng.logits()
        assert np.abs(lg - want_logits[step]).max() < 1e-2, step
        tok = int(np.argmax(lg))
        assert tok == int(want_tokens[step]), step


def test_every_decode_mode_gives_the_same_tokens_and_logits():
    """Chain of fused kernels, one launch per vector-op group, the persistent kernel: the same bits."""
    model = synth.random_model(synth.TINY, seed=7)
    prompt = np.array([1, 2, 3, 400], np.int32)
    dm = DeviceModel(model)
    outs = []
    for mode in (InferenceEngine.DECODE_CHAIN, InferenceEngine.DECODE_UNFUSED, InferenceEngine.DECODE_PERSISTENT,
                 InferenceEngine.DECODE_AUTO):
        eng = InferenceEngine(dm)
        eng.set_decode_mode(mode)
        outs.append((eng.generate(prompt, 8), eng.logits()))
        assert eng.decode_is_persistent == (mode == InferenceEngine.DECODE_PERSISTENT)
    for tokens, logits in outs[1:]:
        assert (tokens == outs[0][0]).all() and (logits == outs[0][1]).all()
    want, _ = oracle.Engine(model).generate(prompt, 8)
    assert (outs[0][0] == want).all()


@pytest.mark.parametrize("cfg", [
    synth.TINY,
    dict(synth.TINY, hidden_size=384, intermediate_size=640),  # 384 columns: no prepared form, the packed kernels run
    dict(synth.BITNET_2B, num_hidden_layers=2, vocab_size=2048, max_position_embeddings=96),
    dict(synth.BITNET_2B, num_hidden_layers=1, vocab_size=2048, max_position_embeddings=64, num_attention_heads=16,
         num_key_value_heads=16, head_dim=160, intermediate_size=8192),  # no grouping, a vector of 8192
], ids=["tiny", "no-prepared-form", "2b4t-width", "wide-ffn"])
def test_chain_on_prepared_weights_matches_the_packed_format(cfg):
    """The default decode chain multiplies on the engine's prepared copies of the matrices (all of a warp's weights
    in registers before the launch's dependency resolves); with the copies switched off it runs the packed-format
    kernels.  Same tokens, same logits bit for bit at every step, also after switching on a live engine."""
    dm = synth.DeviceRandomModel(cfg, seed=31)
    prompt = np.random.default_rng(8).integers(0, cfg["vocab_size"], 7).astype(np.int32)
    prepared, packed = InferenceEngine(dm), InferenceEngine(dm)
    packed.set_prepared_weights(False)
    for t in prompt[:-1]:
        prepared.forward(int(t))
        packed.forward(int(t))
    tok = int(prompt[-1])
    for step in range(40):
        prepared.forward(tok)
        packed.forward(tok)
        a, b = prepared.logits(), packed.logits()
        assert (a == b).all(), (step, np.abs(a - b).max())
        tok = int(np.argmax(a))
    packed.reset()
    want = packed.generate(prompt, 24)
    prepared.reset()
    assert (prepared.generate(prompt, 24) == want).all()
    prepared.reset()
    prepared.set_prepared_weights(False)
    assert (prepared.generate(prompt, 24) == want).all()
    prepared.reset()
    prepared.set_prepared_weights(True)
    assert (prepared.generate(prompt, 24) == want).all()


def test_full_2b4t_shape_against_the_reference_cuda_kernels():
    """The 30-layer 2B-4T-shape model, 16-token prompt + 64 greedy steps, against the reference's
    own kernels on the same GPU: logits within 1e-2 max-abs, identical tokens."""
    from oracle import ref_cuda_engine
    if not ref_cuda_engine.available():
        pytest.skip("oracle/_ref/libspb_refcuda.so not built")
    cfg = dict(synth.BITNET_2B, max_position_embeddings=128)
    dm = synth.DeviceRandomModel(cfg, seed=2)  # all 210 matrices distinct, generated on the GPU
    ours, ref = InferenceEngine(dm), ref_cuda_engine.RefCudaEngine(dm)
    prompt = np.random.default_rng(4).integers(0, cfg["vocab_size"], 16).astype(np.int32)
    for t in prompt[:-1]:
        ours.forward(int(t))
        ref.forward(int(t))
    tok, worst, margins = int(prompt[-1]), 0.0, []
    for step in range(64):
        ours.forward(tok)
        a = ours.logits()
        b = ref.forward(tok).cpu().numpy()
        worst = max(worst, float(np.abs(a - b).max()))
        top2 = np.sort(b)[-2:]
        margins.append(float(top2[1] - top2[0]))
        assert int(np.argmax(a)) == int(np.argmax(b)), (step, margins[-1], worst)
        tok = int(np.argmax(b))
    assert worst < 1e-2, worst
    # and the device-side greedy loop reproduces the same 64 tokens
    ours.reset()
    ref_tokens = []
    ref.__init__(dm)
    for t in prompt[:-1]:
        ref.forward(int(t))
    tok = int(prompt[-1])
    for _ in range(64):
        tok = int(torch.argmax(ref.forward(tok)).item())
        ref_tokens.append(tok)
    assert (ours.generate(prompt, 64) == np.array(ref_tokens, np.int32)).all()


def test_model_directory_round_trip_gives_the_same_tokens(tmp_path):
    # a model written in the reference's directory format and read back decodes like the in-memory one,
    # with an untied head as well
    from spbitnet_b200 import model_io
    model = synth.random_model(synth.TINY, seed=11)
    prompt = np.array([3, 17, 200, 45], np.int32)
    want = InferenceEngine(DeviceModel(model)).generate(prompt, 12)
    back = model_io.load_model_dir(model_io.save_model_dir(model, tmp_path / "m"))
    assert list(InferenceEngine(DeviceModel(back)).generate(prompt, 12)) == list(want)
    model["lm_head"] = model["embed"].copy()  # same values, separate tensor: the untied path must agree
    back = model_io.load_model_dir(model_io.save_model_dir(model, tmp_path / "u"))
    assert list(InferenceEngine(DeviceModel(back)).generate(prompt, 12)) == list(want)
