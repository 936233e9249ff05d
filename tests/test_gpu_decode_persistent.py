"""The persistent decode-step kernel (one cooperative launch per token) against the chain of kernels: identical
tokens and bit-identical logits, on shapes that exercise ragged tile counts, several chunks of positions per KV
head and every GQA group size the kernel is built for; its bounded grid barrier; what it refuses."""
import numpy as np
import pytest

import oracle
from spbitnet_b200 import _lib, kernels as K, synth
from spbitnet_b200.engine import DeviceModel, InferenceEngine

pytestmark = pytest.mark.gpu

CHAIN, PERSISTENT = InferenceEngine.DECODE_CHAIN, InferenceEngine.DECODE_PERSISTENT
TAGGED = InferenceEngine.DECODE_PERSISTENT_TAGGED


def both_modes(dm, prompt, n_new, check_every=1, persistent_mode=PERSISTENT):
    """Runs the same greedy generation in both modes, comparing the logits of every check_every-th step."""
    engines = []
    for mode in (CHAIN, persistent_mode):
        eng = InferenceEngine(dm)
        eng.set_decode_mode(mode)
        engines.append(eng)
    chain, pers = engines
    for t in prompt[:-1]:
        chain.forward(int(t))
        pers.forward(int(t))
    assert pers.decode_is_persistent and not chain.decode_is_persistent
    tok = int(prompt[-1])
    tokens = []
    for step in range(n_new):
        chain.forward(tok)
        pers.forward(tok)
        if step % check_every == 0 or step == n_new - 1:
            a, b = chain.logits(), pers.logits()
            assert (a == b).all(), (step, np.abs(a - b).max())
            tok = int(np.argmax(a))
        else:
            tok = int(np.argmax(chain.logits()))
        tokens.append(tok)
    return np.array(tokens, np.int32), chain, pers


@pytest.mark.parametrize("heads,kv_heads,head_dim", [(4, 4, 64), (4, 2, 64), (8, 2, 32), (16, 2, 16), (2, 1, 128)])
def test_small_models_every_group_size(heads, kv_heads, head_dim):
    cfg = dict(synth.TINY, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
               num_hidden_layers=3, max_position_embeddings=160)
    model = synth.random_model(cfg, seed=heads + kv_heads)
    prompt = np.random.default_rng(1).integers(0, cfg["vocab_size"], 6).astype(np.int32)
    tokens, _, pers = both_modes(DeviceModel(model), prompt, 140, check_every=7)  # crosses two chunk boundaries
    # the greedy loop with the device arg-max, the graph replayed per token
    pers.reset()
    assert (pers.generate(prompt, 40) == tokens[:40]).all()
    want, _ = oracle.Engine(model).generate(prompt, 12)
    assert (tokens[:12] == want).all()


def test_2b4t_width_two_layers():
    cfg = dict(synth.BITNET_2B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=256)
    dm = synth.DeviceRandomModel(cfg, seed=5)
    prompt = np.random.default_rng(2).integers(0, cfg["vocab_size"], 8).astype(np.int32)
    both_modes(dm, prompt, 72, check_every=9)


@pytest.mark.parametrize("cfg_over", [
    dict(num_hidden_layers=3),                                                       # the 2B-4T layer shape
    dict(num_hidden_layers=2, num_attention_heads=20, num_key_value_heads=20, intermediate_size=4096),  # no grouping
    dict(num_hidden_layers=2, hidden_size=3072, num_attention_heads=16, num_key_value_heads=2, head_dim=128,
         intermediate_size=8192),                                                    # groups of eight, long vectors
])
def test_barrier_free_form_matches_the_chain(cfg_over):
    """Stage outputs as tagged words, the residual stream in every block's shared memory: same logits, bit for bit,
    across chunk boundaries of the attention, after a reset, and with the graph replayed per token."""
    cfg = dict(synth.BITNET_2B, vocab_size=4096, max_position_embeddings=256, **cfg_over)
    dm = synth.DeviceRandomModel(cfg, seed=21)
    prompt = np.random.default_rng(7).integers(0, cfg["vocab_size"], 9).astype(np.int32)
    tokens, chain, tagged = both_modes(dm, prompt, 60, check_every=6, persistent_mode=TAGGED)
    before = K.gemm_tc_timeouts()
    for eng in (chain, tagged):
        eng.reset()
    want = chain.generate(prompt, 48)
    assert (tagged.generate(prompt, 48) == want).all()
    tagged.reset()
    assert (tagged.generate(prompt, 48) == want).all()
    assert (want == tokens[:48]).all()
    assert K.gemm_tc_timeouts() == before


def test_barrier_free_form_refuses_narrow_models():
    dm = DeviceModel(synth.random_model(synth.TINY, seed=3))  # fewer row tiles than blocks
    eng = InferenceEngine(dm)
    eng.set_decode_mode(TAGGED)
    with pytest.raises(_lib.SpbError) as err:
        eng.generate(np.array([1, 2, 3], np.int32), 4)
    assert err.value.code == _lib.SPB_E_UNSUPPORTED
    eng.set_decode_mode(PERSISTENT)
    assert len(eng.generate(np.array([1, 2, 3], np.int32), 4)) == 4


def test_more_tiles_than_blocks_and_fewer():
    # hidden 512 / ffn 1024: 32 + 2 x 16 q/k/v tiles and 64 gate/up pairs on 148 blocks (most blocks idle in a stage);
    # hidden 2560 / ffn 8192: 512 gate/up pairs (four per block on some), a vector of 8192 elements
    for cfg in (dict(synth.TINY, hidden_size=512, num_attention_heads=8, num_key_value_heads=4, intermediate_size=1024),
                dict(synth.BITNET_2B, num_hidden_layers=1, intermediate_size=8192, vocab_size=2048,
                     max_position_embeddings=128)):
        dm = synth.DeviceRandomModel(cfg, seed=9)
        prompt = np.random.default_rng(3).integers(0, cfg["vocab_size"], 5).astype(np.int32)
        both_modes(dm, prompt, 12)


def test_generate_with_a_prompt_in_the_graph():
    model = synth.random_model(synth.TINY, seed=11)
    dm = DeviceModel(model)
    prompt = np.random.default_rng(5).integers(0, 512, 20).astype(np.int32)
    outs = []
    for mode in (CHAIN, PERSISTENT):
        eng = InferenceEngine(dm)
        eng.set_decode_mode(mode)
        outs.append(eng.generate(prompt, 30))
        eng.reset()
        assert (eng.generate(prompt, 30) == outs[-1]).all()
    assert (outs[0] == outs[1]).all()


def test_refuses_what_it_cannot_take():
    cfg = dict(synth.TINY, hidden_size=128, num_attention_heads=2, num_key_value_heads=1)  # 128 columns: not whole sign rows
    dm = DeviceModel(synth.random_model(cfg, seed=2))
    prompt = np.array([3, 4, 5], np.int32)
    auto = InferenceEngine(dm)
    want = auto.generate(prompt, 6)  # automatic mode falls back to the chain
    assert not auto.decode_is_persistent
    eng = InferenceEngine(dm)
    eng.set_decode_mode(PERSISTENT)
    with pytest.raises(_lib.SpbError) as err:
        eng.generate(prompt, 6)
    assert err.value.code == _lib.SPB_E_UNSUPPORTED
    eng.set_decode_mode(CHAIN)
    assert (eng.generate(prompt, 6) == want).all()


def test_grid_barrier_wait_is_bounded():
    """Two blocks at a barrier that expects three arrivals: both waits run out, the run-out is counted once, the
    kernel returns; an engine sees SPB_E_TIMEOUT at its next synchronisation and works again after a reset."""
    model = synth.random_model(synth.TINY, seed=4)
    eng = InferenceEngine(DeviceModel(model))
    eng.set_decode_mode(PERSISTENT)
    prompt = np.array([5, 17, 300, 41], np.int32)
    first = eng.generate(prompt, 4)
    before = K.gemm_tc_timeouts()
    assert K.debug_grid_barrier_selftest(200000) == _lib.SPB_E_TIMEOUT, _lib.load().spb_last_error_string()
    assert K.gemm_tc_timeouts() == before + 1
    eng.reset()
    with pytest.raises(_lib.SpbError) as err:
        eng.generate(prompt, 4)
    assert err.value.code == _lib.SPB_E_TIMEOUT
    eng.reset()
    assert (eng.generate(prompt, 4) == first).all()
