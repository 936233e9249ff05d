"""The row-sharded engine (spb_shard_engine_*) on one GPU: with one rank it is the whole model and must reproduce
the single-GPU engine bit for bit (same kernels on "slices" that are the whole matrices) and the CPU oracle's
tokens; with a batch it decodes independent sequences in lock step, each equal to the same sequence decoded
alone; and a rank whose peer never answers must come back with SPB_E_TIMEOUT instead of hanging.  The multi-rank
runs are in tests/test_gpu_sharded.py (two GPUs) and in bench.py --gpus N, which checks the sharded logits against
one rank before it times anything."""
import numpy as np
import pytest
import torch

import oracle
from spbitnet_b200 import _lib, synth
from spbitnet_b200.engine import DeviceModel, InferenceEngine
from spbitnet_b200.shard_engine import ShardEngine

pytestmark = pytest.mark.gpu

ODD = dict(hidden_size=640, num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=5, head_dim=64,
           intermediate_size=1280, vocab_size=1001, max_position_embeddings=48, rms_norm_eps=1e-5, rope_theta=10000.0)


@pytest.mark.parametrize("cfg", [synth.TINY, ODD], ids=["tiny", "odd"])
def test_one_rank_is_the_single_gpu_engine(cfg):
    model = synth.random_model(cfg, seed=41)
    dm = DeviceModel(model)
    sharded, single = ShardEngine(dm), InferenceEngine(dm)
    prompt = np.random.default_rng(1).integers(0, cfg["vocab_size"], 6).astype(np.int32)
    for t in prompt:
        sharded.step([int(t)])
        single.forward(int(t))
        a, b = sharded.logits()[0], single.logits()
        assert (a.view(np.uint32) == b.view(np.uint32)).all()
    sharded.reset()
    want, _ = oracle.Engine(model).generate(prompt, 10)
    assert (sharded.generate(prompt, 10)[:, 0] == want).all()
    assert sharded.seq_len == len(prompt) - 1 + 10


@pytest.mark.parametrize("cfg,batch", [(synth.TINY, 3), (ODD, 5), (synth.TINY, 17)], ids=["tiny-3", "odd-5", "tiny-17"])
def test_batched_decode_equals_each_sequence_alone(cfg, batch):
    model = synth.random_model(cfg, seed=43)
    dm = DeviceModel(model)
    together = ShardEngine(dm, batch=batch)
    n_prompt, n_gen = 4, 8
    prompts = np.random.default_rng(2).integers(0, cfg["vocab_size"], (n_prompt, batch)).astype(np.int32)
    got = together.generate(prompts, n_gen)  # [n_gen, batch]
    cpu = oracle.Engine(model)
    for b in range(batch):
        cpu.reset()
        want, _ = cpu.generate(prompts[:, b], n_gen)
        assert (got[:, b] == want).all(), b
    # the logits of the last step against the oracle's, sequence by sequence
    lg = together.logits()
    for b in (0, batch - 1):
        cpu.reset()
        seq = list(prompts[:, b]) + list(got[:-1, b])
        for t in seq:
            ref = cpu.forward(int(t))
        assert np.abs(lg[b] - ref).max() < 1e-2


def test_batched_decode_at_the_2b4t_width():
    # the tensor-core product (tcgen05 above 32 activation rows) and the batched LM head inside the step
    cfg = dict(synth.BITNET_2B, num_hidden_layers=2, vocab_size=4096, max_position_embeddings=64)
    dm = synth.DeviceRandomModel(cfg, seed=3)
    batch = 40
    together, alone = ShardEngine(dm, batch=batch), InferenceEngine(dm)
    prompts = np.random.default_rng(3).integers(0, cfg["vocab_size"], (3, batch)).astype(np.int32)
    got = together.generate(prompts, 6)
    lg = together.logits()
    for b in (0, 17, batch - 1):
        alone.reset()
        want = alone.generate(prompts[:, b], 6)
        assert (got[:, b] == want).all(), b
        assert np.abs(lg[b] - alone.logits()).max() < 1e-2


WIDE = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
            intermediate_size=16640, vocab_size=2048, max_position_embeddings=32, rms_norm_eps=1e-5, rope_theta=500000.0)


@pytest.mark.parametrize("wide,form", [(False, 0), (True, 0), (True, 1), (True, 2)],
                         ids=["narrow", "wide-launch", "wide-consumer", "wide-direct"])
def test_a_silent_peer_ends_in_a_timeout_not_a_hang(wide, form):
    """Rank 0 of a two-rank group whose "peer" is a zero-filled buffer that nobody writes: every exchange stores
    the rank's slices there, the first wait for the peer's flag runs out after the (short) bound, the kernel raises
    the status word and returns, later exchanges skip their waits, and the host call answers SPB_E_TIMEOUT.
    (wide: the three forms of the exchange of the single-sequence step of a wide model.)"""
    model = synth.random_model(synth.TINY, seed=44)
    dm = synth.DeviceRandomModel(WIDE, seed=44) if wide else DeviceModel(model)
    eng = ShardEngine(dm, rank=0, world=2, timeout_ms=20, connect=False)
    eng.set_exchange_fold(form)
    fake_peer = torch.zeros(eng.exchange_bytes, dtype=torch.uint8, device="cuda")
    eng.set_peer_pointers([0, fake_peer.data_ptr()])
    with pytest.raises(_lib.SpbError) as err:
        eng.step([5])
    assert err.value.code == _lib.SPB_E_TIMEOUT
    torch.cuda.synchronize()
    # the context is healthy: an ordinary engine on the same device still decodes correctly
    ok = InferenceEngine(DeviceModel(model))
    want, _ = oracle.Engine(model).generate(np.array([5, 9], np.int32), 4)
    assert (ok.generate(np.array([5, 9], np.int32), 4) == want).all()
    # rank 0 pushed its slices into the stand-in peer before it gave up
    assert fake_peer.any().item()


@pytest.mark.parametrize("batch", [1, 3])
def test_wide_model_path(batch):
    """hidden >= 4096 switches the engine to its throughput form (one vector kernel per activation, every matrix through
    the tensor-core GEMV, the down projection's 16640-column rows in chunks): against the single-GPU engine, which
    runs the fused SIMT form."""
    cfg = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=16640, vocab_size=2048, max_position_embeddings=32, rms_norm_eps=1e-5, rope_theta=500000.0)
    dm = synth.DeviceRandomModel(cfg, seed=12)
    wide, ref = ShardEngine(dm, batch=batch), InferenceEngine(dm)
    prompts = np.random.default_rng(5).integers(0, cfg["vocab_size"], (3, batch)).astype(np.int32)
    got = wide.generate(prompts, 6)
    lg = wide.logits()
    for b in range(batch):
        ref.reset()
        want = ref.generate(prompts[:, b], 6)
        assert (got[:, b] == want).all(), b
        assert np.abs(lg[b] - ref.logits()).max() < 1e-2


def test_prepared_weights_do_not_change_a_bit():
    """The wide single-sequence step on prepared copies of the slices (the large ones by default, all, none): the
    same tokens and the same logits bit for bit."""
    cfg = dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=16640, vocab_size=2048, max_position_embeddings=32, rms_norm_eps=1e-5, rope_theta=500000.0)
    dm = synth.DeviceRandomModel(cfg, seed=21)
    prompt = np.random.default_rng(6).integers(0, cfg["vocab_size"], (4, 1)).astype(np.int32)
    outs = []
    for level in (1, 0, 2, 1):
        eng = ShardEngine(dm, batch=1)
        eng.set_prepared_weights(level)
        outs.append((eng.generate(prompt, 8), eng.logits()))
        eng.close()
    for tokens, logits in outs[1:]:
        assert (tokens == outs[0][0]).all() and (logits == outs[0][1]).all()
    # switching on a live engine
    eng = ShardEngine(dm, batch=1)
    a = eng.generate(prompt, 8)
    eng.set_prepared_weights(0)
    eng.reset()
    assert (eng.generate(prompt, 8) == a).all()
    eng.set_prepared_weights(2)
    eng.reset()
    assert (eng.generate(prompt, 8) == a).all() and (a == outs[0][0]).all()
