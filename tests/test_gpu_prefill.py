"""Batched prefill against the token-serial path and the CPU oracle: the prompt fed as one or several batches
(BitLinear layers as the batched product) must give the logits of forward() token by token within 1e-2 and the
same greedy tokens, on tiny models (general layouts) and at the 2B-4T width (tensor-core product)."""
import numpy as np
import pytest

import oracle
from spbitnet_b200 import synth
from spbitnet_b200 import kernels as K
from spbitnet_b200.engine import DeviceModel, InferenceEngine

pytestmark = pytest.mark.gpu


def _serial_logits(eng, tokens):
    eng.reset()
    for t in tokens:
        eng.forward(int(t))
    return eng.logits()


@pytest.mark.parametrize("n", [1, 2, 7, 33])
def test_prefill_matches_token_serial_and_oracle(n):
    model = synth.random_model(synth.TINY, seed=11)
    eng = InferenceEngine(DeviceModel(model))
    tokens = np.random.default_rng(n).integers(0, synth.TINY["vocab_size"], n).astype(np.int32)
    want = _serial_logits(eng, tokens)
    eng.reset()
    eng.prefill(tokens)
    got = eng.logits()
    assert eng.seq_len == n
    assert np.abs(got - want).max() < 1e-2
    assert int(np.argmax(got)) == int(np.argmax(want))
    cpu = oracle.Engine(model)
    for t in tokens:
        ref = cpu.forward(int(t))
    assert np.abs(got - ref).max() < 1e-2
    # decoding continues from the prefilled cache exactly as from the token-serial one
    nxt = int(np.argmax(got))
    eng.forward(nxt)
    after = eng.logits()
    assert np.abs(after - cpu.forward(nxt)).max() < 1e-2


def test_prefill_in_two_calls_equals_one_call():
    model = synth.random_model(synth.TINY, seed=12)
    eng = InferenceEngine(DeviceModel(model))
    tokens = np.random.default_rng(5).integers(0, synth.TINY["vocab_size"], 20).astype(np.int32)
    eng.prefill(tokens)
    one = eng.logits()
    eng.reset()
    eng.prefill(tokens[:9])
    eng.prefill(tokens[9:])
    two = eng.logits()
    assert eng.seq_len == 20
    # the second call's tokens attend to the first call's cache entries; the arithmetic per token is the same
    assert (one == two).all()


@pytest.mark.parametrize("chunk", [3, 8, 256])
def test_generate_with_batched_prompt_gives_the_same_tokens(chunk):
    model = synth.random_model(synth.TINY, seed=13)
    eng = InferenceEngine(DeviceModel(model))
    prompt = np.random.default_rng(9).integers(0, synth.TINY["vocab_size"], 13).astype(np.int32)
    serial = eng.generate(prompt, 10)
    assert eng.seq_len == len(prompt) - 1 + 10
    eng.reset()
    assert eng.set_prefill_chunk(chunk) == 0
    batched = eng.generate(prompt, 10)
    assert eng.seq_len == len(prompt) - 1 + 10
    assert (serial == batched).all()
    want, _ = oracle.Engine(model).generate(prompt, 10)
    assert (batched == want).all()
    # a second turn on top of the first (positions continue), batched against serial
    more = np.array([3, 1, 4], np.int32)
    b2 = eng.generate(more, 5)
    eng.set_prefill_chunk(0)
    eng.reset()
    eng.generate(prompt, 10)
    s2 = eng.generate(more, 5)
    assert (b2 == s2).all()


def test_generate_with_batched_prompt_stops_at_eos_and_handles_zero_tokens():
    model = synth.random_model(synth.TINY, seed=1)
    eng = InferenceEngine(DeviceModel(model))
    prompt = np.array([5, 17, 200], np.int32)
    full = eng.generate(prompt, 12)
    eng.reset()
    eng.set_prefill_chunk(64)
    stop = eng.generate(prompt, 12, eos_token_id=int(full[4]))
    first = int(np.where(full == full[4])[0][0])
    assert (stop == full[: first + 1]).all()
    eng.reset()
    assert len(eng.generate(prompt, 0)) == 0
    assert eng.seq_len == len(prompt) - 1


def test_prefill_rejects_bad_arguments():
    model = synth.random_model(synth.TINY, seed=2)
    eng = InferenceEngine(DeviceModel(model))
    with pytest.raises(Exception):
        eng.prefill(np.array([synth.TINY["vocab_size"]], np.int32))
    with pytest.raises(Exception):
        eng.prefill(np.zeros(synth.TINY["max_position_embeddings"] + 1, np.int32))
    assert eng.seq_len == 0


def test_prefill_at_the_2b4t_width():
    cfg = dict(synth.BITNET_2B, num_hidden_layers=2, vocab_size=8192, max_position_embeddings=512)
    model = synth.random_model(cfg, seed=3)
    eng = InferenceEngine(DeviceModel(model))
    tokens = np.random.default_rng(0).integers(0, cfg["vocab_size"], 300).astype(np.int32)  # two chunks: 256 + 44
    want = _serial_logits(eng, tokens)
    eng.reset()
    eng.prefill(tokens)
    got = eng.logits()
    assert np.abs(got - want).max() < 1e-2
    assert int(np.argmax(got)) == int(np.argmax(want))
    assert K.gemm_tc_timeouts() == 0
    # greedy continuation identical
    eng.reset()
    serial = eng.generate(tokens[:40], 16)
    eng.reset()
    eng.set_prefill_chunk(256)
    assert (eng.generate(tokens[:40], 16) == serial).all()
