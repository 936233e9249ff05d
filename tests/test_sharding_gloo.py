"""Host logic of the row-sharded path on CPU: shard plan, slice contents, and the gather order
over a world_size-2 (and 3) gloo group.  The per-rank arithmetic here is the oracle's; the GPU
kernels are exercised by the -m gpu tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from spbitnet_b200 import sharding, synth


def test_row_ranges_cover_and_keep_heads_whole():
    for rows, world, mult in [(2560, 8, 128), (640, 2, 128), (640, 4, 128), (6912, 8, 1), (28672, 8, 1), (7, 3, 1)]:
        spans = [sharding.row_range(rows, world, r, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((s1 - s0) % mult == 0 for s0, s1 in spans)
        sizes = [s1 - s0 for s0, s1 in spans]
        assert max(sizes) - min(sizes) <= mult
        assert sizes == sharding.gather_sizes(rows, world, mult)
    with pytest.raises(ValueError):
        sharding.row_range(100, 2, 0, 128)


def test_slices_reproduce_the_full_product():
    case = synth.gemv_case(640, 256, seed=3)
    t = dict(case)
    full = oracle.sparse_gemv(case["meta"], case["values"], case["x"], 640, 256)
    parts = []
    for r in range(5):
        s = sharding.shard_rows(t, 5, r, multiple=128)
        parts.append(oracle.sparse_gemv(s["meta"], s["values"], case["x"], s["rows"], 256))
    assert (np.concatenate(parts) == full).all()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, cols, mult, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = synth.gemv_case(rows, cols, seed=11)
        s = sharding.shard_rows(dict(case), world, rank, mult)
        local = oracle.sparse_gemv(s["meta"], s["values"], case["x"], s["rows"], cols) if s["rows"] else np.zeros(0, np.int32)
        full = sharding.all_gather_rows(torch.from_numpy(local), rows, mult)
        want = oracle.sparse_gemv(case["meta"], case["values"], case["x"], rows, cols)
        out_q.put((rank, bool((full.numpy() == want).all()), int(full.numel())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,rows,mult", [(2, 640, 128), (3, 640, 128), (2, 37, 1)])
def test_all_gather_of_row_slices_gloo(world, rows, mult):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, rows, 256, mult, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == list(range(world))
    assert all(ok and n == rows for _, ok, n in results)


def test_head_split_keeps_query_heads_with_their_kv_head():
    # the sharded engine splits q by (query heads per KV head) * head_dim rows and k/v by head_dim rows: on every
    # rank the query heads must be exactly those of the rank's KV heads, also when the KV heads do not divide evenly
    from spbitnet_b200 import sharding
    for nh, nkv, hd, world in [(20, 5, 128, 2), (20, 5, 128, 4), (64, 8, 128, 8), (4, 2, 64, 2), (10, 5, 64, 3)]:
        g = nh // nkv
        covered = 0
        for r in range(world):
            q0, q1 = sharding.row_range(nh * hd, world, r, g * hd)
            k0, k1 = sharding.row_range(nkv * hd, world, r, hd)
            kv0, kv1 = sharding.row_range(nkv, world, r)
            assert (k0, k1) == (kv0 * hd, kv1 * hd)
            assert (q0, q1) == (kv0 * g * hd, kv1 * g * hd)
            covered += kv1 - kv0
        assert covered == nkv


def _engine_worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cpu_kernels
        # five KV heads over the ranks (uneven), odd vocabulary
        cfg = dict(hidden_size=320, num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=5, head_dim=32,
                   intermediate_size=512, vocab_size=301, max_position_embeddings=16, rms_norm_eps=1e-5,
                   rope_theta=10000.0)
        model = synth.random_model(cfg, seed=7)
        eng = sharding.ShardedEngine(model, device="cpu", kernels=cpu_kernels)
        one = sharding.ShardedEngine(model, single=True, device="cpu", kernels=cpu_kernels)
        cpu = oracle.Engine(model)
        ok = True
        tok = 5
        for step in range(6):
            a = eng.forward(tok).numpy()
            b = one.forward(tok).numpy()
            want = cpu.forward(tok)
            ok = ok and a.shape == (cfg["vocab_size"],)
            ok = ok and bool((a.view(np.uint32) == b.view(np.uint32)).all())   # the split changes no bit
            ok = ok and float(np.abs(a - want).max()) < 1e-4 and int(np.argmax(a)) == oracle.argmax(want)
            tok = int(np.argmax(a))
        out_q.put((rank, ok, eng.nkv_loc))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_sharded_decode_step_gloo(world):
    """sharding.ShardedEngine (KV-head split of q/k/v, row split of the other matrices and of the lm_head, four
    all-gathers per layer) under gloo with oracle-backed stand-ins for the per-op kernels: logits bit-identical to the
    same step on one rank and equal to the oracle engine's."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_engine_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results)
    assert sum(n for _, _, n in results) == 5
