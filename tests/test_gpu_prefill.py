"""Batched prefill against the token-serial path and the CPU oracle: the prompt fed as one or several batches
(BitLinear layers as the batched product) must give the logits of forward() token by token within 1e-2 and the
same greedy tokens, on tiny models (general layouts) and at the 2B-4T width (tensor-core product)."""
import numpy as np
import pytest

import oracle
from spbitnet_b200 import synth
from spbitnet_b200 import kernels as K
from spbitnet_b200.engine import DeviceModel, InferenceEngine
from gpu_util import Guarded, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1, 3], ids=["auto", "simt", "tcgen05sp"])
def gemm_variant(request):
    old = K.set_gemm_variant(request.param)
    yield request.param
    K.set_gemm_variant(old)


@pytest.mark.parametrize("rows,cols,n", [(256, 256, 1), (640, 2560, 5), (2560, 2560, 40), (6912, 2560, 130),
                                          (2560, 6912, 64), (129, 384, 33), (100, 260, 7), (300, 1024, 257)])
def test_batched_bitlinear_is_gemm_then_dequantize(rows, cols, n, gemm_variant):
    # half outputs bit-identical to the oracle's dequantize of the oracle's integer product, row by row
    case = synth.gemm_case(rows, cols, n, seed=n)
    before = K.gemm_tc_timeouts()
    rng = np.random.default_rng(n)
    absmax = rng.uniform(0.5, 4.0, n).astype(np.float32)
    absmax[0] = 0.0  # an all-zero activation row: scale 0, outputs +0
    gamma = np.float32(0.0371)
    acc = oracle.sparse_gemm(case["meta"], case["values"], case["X"], rows, cols)
    want = np.stack([oracle.dequantize(acc[j], absmax[j], gamma) for j in range(n)])
    out = Guarded(n * rows * 2)
    ws = Guarded(n * rows * 4)
    K.sparse_bitlinear_gemm_gpu(dev(case["meta"]), dev(case["values"]), dev(case["X"]), out.ptr, dev(absmax), gamma,
                                rows, cols, n, case["meta_stride"], case["values_stride"], acc_workspace=ws.ptr)
    got = out.read(np.float16).reshape(n, rows)
    assert (got.view(np.uint16) == want.view(np.uint16)).all()
    assert K.gemm_tc_timeouts() == before


def test_batched_bitlinear_without_workspace():
    # the default forms need no workspace; a layout that falls to the SIMT form answers "unsupported" without one
    case = synth.gemm_case(2560, 2560, 48, seed=1)
    absmax = np.ones(48, np.float32)
    out = Guarded(48 * 2560 * 2)
    K.sparse_bitlinear_gemm_gpu(dev(case["meta"]), dev(case["values"]), dev(case["X"]), out.ptr, dev(absmax), 1.0,
                                2560, 2560, 48, case["meta_stride"], case["values_stride"])
    acc = oracle.sparse_gemm(case["meta"], case["values"], case["X"], 2560, 2560)
    want = np.stack([oracle.dequantize(acc[j], 1.0, 1.0) for j in range(48)])
    assert (out.read(np.float16).reshape(48, 2560).view(np.uint16) == want.view(np.uint16)).all()
    odd = synth.gemm_case(100, 260, 7, seed=2)
    out2 = Guarded(7 * 100 * 2)
    with pytest.raises(Exception):
        K.sparse_bitlinear_gemm_gpu(dev(odd["meta"]), dev(odd["values"]), dev(odd["X"]), out2.ptr, dev(absmax), 1.0,
                                    100, 260, 7, odd["meta_stride"], odd["values_stride"])


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


def test_repeated_prefill_replays_a_graph_with_the_same_result():
    # the first call launches kernel by kernel, the second captures a graph, the third replays it
    model = synth.random_model(synth.TINY, seed=14)
    eng = InferenceEngine(DeviceModel(model))
    tokens = np.random.default_rng(1).integers(0, synth.TINY["vocab_size"], 11).astype(np.int32)
    outs = []
    for _ in range(4):
        eng.reset()
        eng.prefill(tokens)
        outs.append(eng.logits())
    assert all((o == outs[0]).all() for o in outs[1:])
    # a replayed chunk at another start position (the position lives in device memory)
    eng.reset()
    eng.prefill(tokens[:5])
    eng.prefill(tokens)      # 11 tokens at positions 5..15, graph of T = 11
    a = eng.logits()
    eng.reset()
    for t in list(tokens[:5]) + list(tokens):
        eng.forward(int(t))
    assert np.abs(a - eng.logits()).max() < 1e-2


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
    eng.set_prefill_chunk(256)
    eng.prefill(tokens)
    got = eng.logits()
    assert np.abs(got - want).max() < 1e-2
    assert int(np.argmax(got)) == int(np.argmax(want))
    eng.reset()
    eng.set_prefill_chunk(0)
    eng.prefill(tokens)      # one chunk of 300
    one = eng.logits()
    assert np.abs(one - want).max() < 1e-2 and int(np.argmax(one)) == int(np.argmax(want))
    # (a tensor-core wait that ran out would have made prefill() raise SPB_E_TIMEOUT)
    # greedy continuation identical
    eng.reset()
    serial = eng.generate(tokens[:40], 16)
    eng.reset()
    eng.set_prefill_chunk(256)
    assert (eng.generate(tokens[:40], 16) == serial).all()
