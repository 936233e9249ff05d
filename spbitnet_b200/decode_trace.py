"""Stage times of the persistent decode kernel: where a layer's microseconds go.

    python -m spbitnet_b200.decode_trace [--layers N] [--prompt 128] [--tokens 40]

Runs a random-init BitNet-2B-4T-shape model in the persistent decode mode with the kernel's stage marks switched on
(spb_debug_set_decode_trace) and prints, for the first and the last block of the grid, the mean time between
consecutive marks of the last generated token (layers 2 .. N-2).  Needs a GPU.
"""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np

MARKS = 20
NAMES = ["S1 q/k/v  wait for slab", "S1        produce x", "S1        rows + RoPE", "S1        barrier",
         "S2 attn   issue next slab", "S2        chunks + merge", "S2        barrier",
         "S3 o      wait for slab", "S3        produce x", "S3        rows", "S3        barrier",
         "S4 gate/up wait for slab", "S4        produce x", "S4        rows", "S4        barrier",
         "S5 down   wait for slab", "S5        produce x", "S5        rows", "S5        barrier"]


def main() -> None:
    import torch
    from . import _lib, synth
    from .engine import InferenceEngine
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=30)
    ap.add_argument("--prompt", type=int, default=128)
    ap.add_argument("--tokens", type=int, default=40)
    ap.add_argument("--tagged", action="store_true", help="the barrier-free form (stage outputs as tagged words)")
    args = ap.parse_args()
    cfg = dict(synth.BITNET_2B, num_hidden_layers=args.layers)
    lib = _lib.load()
    dm = synth.DeviceRandomModel(cfg, seed=0)
    trace = torch.zeros(2 * 4096, dtype=torch.int64, device="cuda")
    lib.spb_debug_set_decode_trace(C.c_void_p(trace.data_ptr()))
    try:
        eng = InferenceEngine(dm)
        eng.set_decode_mode(InferenceEngine.DECODE_PERSISTENT_TAGGED if args.tagged else InferenceEngine.DECODE_PERSISTENT)
        prompt = np.random.default_rng(0).integers(0, cfg["vocab_size"], args.prompt).astype(np.int32)
        eng.generate(prompt, args.tokens)
        torch.cuda.synchronize()
    finally:
        lib.spb_debug_set_decode_trace(C.c_void_p(0))
    t = trace.cpu().numpy().astype(np.float64)
    n = args.layers
    lo, hi = (2, n - 2) if n >= 6 else (0, n)
    for name, off in (("first block", 0), ("last block", 4096)):
        a = t[off:off + n * MARKS].reshape(n, MARKS)[:, :19]
        flat = a.reshape(-1)
        d = np.concatenate([[np.nan], np.diff(flat)]).reshape(n, 19)
        d[:, 0] = a[:, 0] - np.concatenate([[np.nan], a[:-1, 18]])  # from the previous layer's last mark
        layer_us = np.nanmean(np.diff(a[:, 0])[lo:hi]) / 1e3 if n > 1 else float("nan")
        print(f"{name}: {layer_us:.2f} us per layer at position {args.prompt + args.tokens - 1}")
        for k, label in enumerate(NAMES):
            print(f"  {label:28s} {np.nanmean(d[lo:hi, k]) / 1e3:6.2f} us")


if __name__ == "__main__":
    main()
