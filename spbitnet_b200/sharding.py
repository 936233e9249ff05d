"""Output-row sharding of sparse-ternary matrices over the ranks of one node.

The reference is single-GPU; this is the one way its hot path partitions without a
reduction: rank r owns a contiguous slice of the output rows of every matrix (a contiguous
slice of `meta` and `values`, which are row-major), computes its slice with the ordinary
kernels on the full activation vector, and the slices are concatenated by an all-gather.
Integer accumulators and half outputs are therefore bit-identical to the unsharded result.
q/k/v are split by whole heads so that attention and the KV cache stay local.
"""
from __future__ import annotations

import numpy as np


def row_range(rows: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Contiguous, balanced slice [start, stop) of `rows`, in units of `multiple` rows
    (multiple = head_dim keeps heads whole).  The first `extra` ranks get one unit more."""
    if rows % multiple:
        raise ValueError(f"{rows} rows are not a multiple of {multiple}")
    units = rows // multiple
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return start * multiple, stop * multiple


def shard_rows(t: dict, world: int, rank: int, multiple: int = 1) -> dict:
    """Row slice of one matrix in the synth / converter layout (dict with meta, values, rows, ...)."""
    r0, r1 = row_range(t["rows"], world, rank, multiple)
    out = dict(t)
    out.update(meta=np.ascontiguousarray(t["meta"][r0:r1]), values=np.ascontiguousarray(t["values"][r0:r1]),
               rows=r1 - r0, row_start=r0)
    return out


def gather_sizes(rows: int, world: int, multiple: int = 1) -> list[int]:
    return [row_range(rows, world, r, multiple)[1] - row_range(rows, world, r, multiple)[0] for r in range(world)]


def all_gather_rows(local, rows: int, multiple: int = 1, group=None):
    """Concatenates the per-rank output slices (1-D tensors) into the full `rows` vector on every
    rank.  Slices may differ by one unit; they are padded to the largest for the collective."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = gather_sizes(rows, world, multiple)
    pad = max(sizes)
    buf = torch.zeros(pad, dtype=local.dtype, device=local.device)
    buf[: local.numel()] = local
    out = torch.empty(world * pad, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, buf, group=group)
    return torch.cat([out[r * pad: r * pad + sizes[r]] for r in range(world)])


class ShardedBitLinear:
    """One BitLinear layer row-sharded over the default process group: local slice through
    sparse_bitlinear_q8_gpu, then an all-gather (NCCL over NVLink on GPUs)."""

    def __init__(self, t: dict, multiple: int = 1, group=None):
        import torch
        import torch.distributed as dist
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.cols, self.multiple = t["rows"], t["cols"], multiple
        s = shard_rows(t, self.world, self.rank, multiple)
        self.local_rows = s["rows"]
        self.meta = torch.from_numpy(s["meta"].view(np.int32)).cuda()
        self.values = torch.from_numpy(s["values"].view(np.int32)).cuda()
        self.ms, self.vs, self.gamma = t["meta_stride"], t["values_stride"], float(t["gamma"])
        self.local = torch.empty(max(self.local_rows, 1), dtype=torch.float16, device="cuda")

    def forward(self, xq, d_absmax):
        from . import kernels as K
        K.sparse_bitlinear_q8_gpu(self.meta, self.values, xq, self.local, d_absmax, self.gamma, self.local_rows,
                                  self.cols, self.ms, self.vs)
        return all_gather_rows(self.local[: self.local_rows], self.rows, self.multiple, self.group)
