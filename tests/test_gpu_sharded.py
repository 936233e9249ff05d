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
