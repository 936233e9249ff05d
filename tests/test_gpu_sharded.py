"""Row-sharded BitLinear over NCCL on two GPUs: every rank computes its slice of the output rows
with the ordinary kernel and an all-gather rebuilds the full vector, which must equal the oracle's
unsharded result bit for bit (no reduction is involved).  Skipped on boxes with one GPU."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import oracle
        from spbitnet_b200 import sharding, synth
        ok = True
        for rows, cols, mult in [(2560, 2560, 128), (640, 2560, 128), (6912, 2560, 1)]:
            case = synth.gemv_case(rows, cols, seed=rows)
            t = dict(case, gamma=np.float32(0.0231))
            x = (np.random.default_rng(5).standard_normal(cols) * 2).astype(np.float16)
            q, absmax = oracle.absmax_quantize(x)
            want = oracle.fused_bitlinear(case["meta"], case["values"], x, absmax, 0.0231, rows, cols)
            layer = sharding.ShardedBitLinear(t, multiple=mult)
            xq = torch.from_numpy(q).cuda()
            d_abs = torch.tensor([absmax], dtype=torch.float32, device="cuda")
            full = layer.forward(xq, d_abs)
            torch.cuda.synchronize()
            got = full.view(torch.int16).cpu().numpy().view(np.uint16)
            ok = ok and got.shape[0] == rows and bool((got == want.view(np.uint16)).all())
        out_q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_sharded_bitlinear_two_gpus():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in results)


def _engine_worker(rank, world, port, out_q):
    import time
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import oracle
        from spbitnet_b200 import sharding, synth
        from spbitnet_b200.engine import DeviceModel, InferenceEngine
        ok, notes = True, {}
        configs = [
            dict(synth.TINY),
            # five KV heads over two ranks (3 + 2), odd vocabulary (501 + 500 rows of the lm_head)
            dict(hidden_size=640, num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=5, head_dim=64,
                 intermediate_size=1280, vocab_size=1001, max_position_embeddings=32, rms_norm_eps=1e-5,
                 rope_theta=10000.0),
        ]
        for ci, cfg in enumerate(configs):
            model = synth.random_model(cfg, seed=21 + ci)
            sharded = sharding.ShardedEngine(model)
            single = sharding.ShardedEngine(model, single=True)
            fused = InferenceEngine(DeviceModel(model))
            prompt = np.random.default_rng(ci).integers(0, cfg["vocab_size"], 5).astype(np.int32)
            toks = [int(t) for t in prompt]
            gen = []
            for step in range(11):
                tok = toks[step] if step < len(toks) else gen[-1]
                a = sharded.forward(tok)
                b = single.forward(tok)
                fused.forward(tok)
                c = fused.logits()
                ah = a.cpu().numpy()
                # same ops on row slices, concatenated: bit-identical to one rank
                ok = ok and bool((ah.view(np.uint32) == b.cpu().numpy().view(np.uint32)).all())
                # against the production engine (fused kernels, split attention): the engine's logits tolerance
                ok = ok and float(np.abs(ah - c).max()) < 1e-2 and int(np.argmax(ah)) == int(np.argmax(c))
                if step >= len(toks) - 1:
                    gen.append(int(np.argmax(ah)))
            if rank == 0:
                want, _ = oracle.Engine(model).generate(prompt, 6)
                ok = ok and gen[:6] == [int(t) for t in want]
        # timing at the 2B-4T width (4 layers, small vocabulary): the sharded step against the same step on one rank
        cfg = dict(synth.BITNET_2B, num_hidden_layers=4, vocab_size=8192, max_position_embeddings=128)
        model = synth.random_model(cfg, seed=5, shared_layer=True)
        for name, eng in (("sharded", sharding.ShardedEngine(model)), ("one_rank", sharding.ShardedEngine(model, single=True))):
            for t in range(3):
                eng.forward(t)
            torch.cuda.synchronize()
            dist.barrier()
            t0 = time.perf_counter()
            for t in range(20):
                eng.forward(t)
            torch.cuda.synchronize()
            notes[name + "_ms_per_token"] = round((time.perf_counter() - t0) / 20 * 1e3, 3)
        out_q.put((rank, ok, notes))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_sharded_engine_two_gpus():
    """Whole decode step row-sharded over two GPUs (q/k/v by KV heads, the other matrices and the lm_head by rows,
    all-gathers only): logits bit-identical to the same step on one rank, within 1e-2 of the production engine,
    greedy tokens equal to the oracle's."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_engine_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    print("row-sharded engine timing:", [n for _, _, n in results])
    assert all(ok for _, ok, _ in results)


def test_sharded_engine_on_one_rank_matches_the_engine():
    """The op-by-op step the sharded engine is made of (single=True: no process group) against the production engine
    and the oracle; runs on any box."""
    import oracle
    from spbitnet_b200 import sharding, synth
    from spbitnet_b200.engine import DeviceModel, InferenceEngine
    model = synth.random_model(synth.TINY, seed=31)
    eng = sharding.ShardedEngine(model, single=True)
    fused = InferenceEngine(DeviceModel(model))
    cpu = oracle.Engine(model)
    for tok in [3, 400, 17, 99, 250, 1]:
        a = eng.forward(tok).cpu().numpy()
        fused.forward(tok)
        want = cpu.forward(tok)
        assert np.abs(a - want).max() < 1e-2
        assert np.abs(a - fused.logits()).max() < 1e-2
        assert int(np.argmax(a)) == oracle.argmax(want)
    prompt = np.array([5, 17, 200], np.int32)
    eng.reset()
    want_tokens, _ = cpu.__class__(model).generate(prompt, 6)
    assert (eng.generate(prompt, 6) == want_tokens).all()


def _shard_engine_worker(rank, world, port, out_q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import oracle
        from spbitnet_b200 import synth
        from spbitnet_b200.engine import DeviceModel
        from spbitnet_b200.shard_engine import ShardEngine
        ok, notes = True, []
        configs = [
            (dict(synth.TINY), 1),
            # five KV heads over two ranks (3 + 2), odd vocabulary (501 + 500 rows of the LM head)
            (dict(hidden_size=640, num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=5, head_dim=64,
                  intermediate_size=1280, vocab_size=1001, max_position_embeddings=32, rms_norm_eps=1e-5,
                  rope_theta=10000.0), 1),
            (dict(synth.TINY), 6),
            # wide model: the throughput form of the step
            (dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                  intermediate_size=16640, vocab_size=2048, max_position_embeddings=32, rms_norm_eps=1e-5,
                  rope_theta=500000.0), 1),
            1,  # the same model with the exchanges inside the kernels that consume the gathered vectors
            0,  # ... and as launches of their own
        ]
        for ci, entry in enumerate(configs):
            form = entry if isinstance(entry, int) else None  # None: the default (slices sent by the producers' epilogues)
            cfg, batch = configs[3] if form is not None else entry
            wide = cfg["hidden_size"] >= 4096
            if wide:
                model, dm = None, synth.DeviceRandomModel(cfg, seed=61)
            else:
                model = synth.random_model(cfg, seed=61 + ci)
                dm = DeviceModel(model)
            sharded = ShardEngine(dm, rank=rank, world=world, batch=batch)
            if form is not None:
                sharded.set_exchange_fold(form)
            one = ShardEngine(dm, batch=batch)  # the same step with every matrix whole, on this rank's GPU
            prompts = np.random.default_rng(ci).integers(0, cfg["vocab_size"], (5, batch)).astype(np.int32)
            for step in range(5):
                sharded.step(prompts[step])
                one.step(prompts[step])
                a, b = sharded.logits(), one.logits()
                same = bool((a.view(np.uint32) == b.view(np.uint32)).all())
                ok = ok and same
                if not same:
                    notes.append(("logits differ", ci, step, float(np.abs(a - b).max())))
            sharded.reset()
            one.reset()
            got, want = sharded.generate(prompts, 9), one.generate(prompts, 9)
            ok = ok and bool((got == want).all())
            if batch == 1 and rank == 0 and model is not None:
                cpu, _ = oracle.Engine(model).generate(prompts[:, 0], 9)
                ok = ok and bool((got[:, 0] == cpu).all())
            dist.barrier()
            sharded.close()
        out_q.put((rank, ok, notes))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_shard_engine_two_gpus():
    """The C++ row-sharded engine over two GPUs (slices exchanged by peer stores and flags, no library collective):
    logits bit-identical to the same engine with one rank, greedy tokens equal to the oracle's, with an uneven split
    and with a batch of sequences."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_shard_engine_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results), [n for _, _, n in results]
