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


class ShardedEngine:
    """The decode step of spbitnet::InferenceEngine::forward (src/inference.cu:123-283) with every matrix
    row-sharded over the ranks of a process group and no reduction anywhere:

      * q/k/v by whole KV heads (a rank owns some KV heads, their query heads and their KV cache), so RoPE,
        the cache scatter and attention are local; the attention output is all-gathered (half);
      * o_proj, gate/up, down by output rows; their outputs are all-gathered (half; the relu2 * up product as
        fp32, because ffn_sub_norm needs the sum of squares over the whole vector);
      * lm_head by vocabulary rows; the logits are all-gathered (fp32);
      * the vector ops (norms, quantisation, residual adds) are replicated: every rank holds the full
        activation, which is what lets the integer path stay bit-exact.

    Four all-gathers per layer plus one for the logits.  The ops are the library's per-op entry points, called
    in the reference's order, so the logits are bit-identical to the same engine on one rank (single=True).
    The reference itself is single-GPU; this class has no counterpart there."""

    def __init__(self, model: dict, group=None, single: bool = False, device=None, kernels=None):
        """device: where the tensors live (default: the current CUDA device).  kernels: the module providing the
        per-op entry points (default: spbitnet_b200.kernels, i.e. the CUDA library; the CPU tests pass an
        oracle-backed stand-in together with device="cpu" to exercise the split and the collectives under gloo)."""
        import torch
        import torch.distributed as dist
        if kernels is None:
            from . import kernels
        self.K = kernels
        self.group = group
        self.world = 1 if single else dist.get_world_size(group)
        self.rank = 0 if single else dist.get_rank(group)
        c = self.cfg = dict(model["config"])
        self.H, self.hd = c["hidden_size"], c["head_dim"]
        self.nh, self.nkv, self.inter = c["num_attention_heads"], c["num_key_value_heads"], c["intermediate_size"]
        self.vocab, self.max_seq = c["vocab_size"], c["max_position_embeddings"]
        if self.nh % self.nkv:
            raise ValueError("query heads must be a multiple of KV heads")
        if self.world > self.nkv:
            raise ValueError(f"{self.world} ranks but only {self.nkv} KV heads to split")
        self.group_heads = self.nh // self.nkv
        kv0, kv1 = row_range(self.nkv, self.world, self.rank)
        self.nkv_loc, self.nh_loc = kv1 - kv0, (kv1 - kv0) * self.group_heads
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dev = dev

        def up(a):
            t = torch.from_numpy(np.ascontiguousarray(a).view(np.int16) if a.dtype == np.float16 else np.ascontiguousarray(a))
            t = t.to(dev)
            return t.view(torch.float16) if a.dtype == np.float16 else t

        # per matrix: row multiple that keeps the split aligned with the KV heads
        mult = [self.group_heads * self.hd, self.hd, self.hd, 1, 1, 1, 1]
        self.mult = mult
        self.layers = []
        for layer in model["layers"]:
            lin = []
            for i, t in enumerate(layer["linear"]):
                s = shard_rows(t, self.world, self.rank, mult[i])
                lin.append(dict(rows=t["rows"], cols=t["cols"], local_rows=s["rows"], ms=t["meta_stride"],
                                vs=t["values_stride"], gamma=float(t["gamma"]),
                                meta=up(s["meta"].view(np.int32)), values=up(s["values"].view(np.int32))))
            norms = [None if n is None else up(n) for n in layer["norm"]]
            kc = torch.zeros((max(self.nkv_loc, 1), self.max_seq, self.hd), dtype=torch.float16, device=dev)
            self.layers.append(dict(lin=lin, norm=norms, kcache=kc, vcache=torch.zeros_like(kc)))
        self.embed = up(model["embed"])
        head = model.get("lm_head")
        head = model["embed"] if head is None else head
        v0, v1 = row_range(self.vocab, self.world, self.rank)
        self.head_loc = up(head[v0:v1])
        self.final_norm = up(model["final_norm"])
        f16 = dict(dtype=torch.float16, device=dev)
        self.x = torch.zeros(self.H, **f16)
        self.xn = torch.zeros(max(self.H, self.inter, self.nh * self.hd), **f16)
        self.xq = torch.zeros(max(self.H, self.inter, self.nh * self.hd), dtype=torch.int8, device=dev)
        self.absmax = torch.zeros(1, dtype=torch.float32, device=dev)
        self.seq_len = 0
        self.logits = None

    def reset(self):
        for L in self.layers:
            L["kcache"].zero_()
            L["vcache"].zero_()
        self.seq_len = 0

    def _gather(self, local, rows, multiple=1):
        if self.world == 1:
            return local
        return all_gather_rows(local, rows, multiple, self.group)

    def _bitlinear(self, lin):
        """Local rows of BitLinear(lin) on the quantised activation in self.xq / self.absmax."""
        import torch
        K = self.K
        out = torch.empty(max(lin["local_rows"], 1), dtype=torch.float16, device=self.dev)
        if lin["local_rows"]:
            K.sparse_bitlinear_q8_gpu(lin["meta"], lin["values"], self.xq, out, self.absmax, lin["gamma"],
                                      lin["local_rows"], lin["cols"], lin["ms"], lin["vs"])
        return out[: lin["local_rows"]]

    def forward(self, token_id: int):
        """One token; returns the full logits (vocab_size float32, device tensor) on every rank."""
        import torch
        K = self.K
        if self.seq_len >= self.max_seq:
            raise ValueError("KV cache full")
        c, H, hd = self.cfg, self.H, self.hd
        eps, theta, pos = float(c["rms_norm_eps"]), float(c["rope_theta"]), self.seq_len
        scale = 1.0 / float(np.sqrt(hd))
        x = self.x
        x.copy_(self.embed[int(token_id)])
        for L in self.layers:
            lin, norm = L["lin"], L["norm"]
            K.rms_norm_gpu(x, norm[0], self.xn, H, eps)
            K.absmax_quantize_gpu(self.xn, self.xq, self.absmax, H)
            q, k, v = (self._bitlinear(lin[i]) for i in range(3))
            attn_loc = torch.empty(max(self.nh_loc * hd, 1), dtype=torch.float16, device=self.dev)
            if self.nkv_loc:
                K.rope_gpu(q, self.nh_loc, hd, pos, theta)
                K.rope_gpu(k, self.nkv_loc, hd, pos, theta)
                K.scatter_kv_gpu(k, L["kcache"], self.nkv_loc, hd, self.max_seq, pos)
                K.scatter_kv_gpu(v, L["vcache"], self.nkv_loc, hd, self.max_seq, pos)
                K.decode_attention_gpu(q, L["kcache"], L["vcache"], attn_loc, self.nh_loc, self.nkv_loc, hd,
                                       self.max_seq, pos + 1, scale)
            attn = self._gather(attn_loc[: self.nh_loc * hd], self.nh * hd, self.mult[0])
            K.absmax_quantize_gpu(attn, self.xq, self.absmax, self.nh * hd)
            o = self._gather(self._bitlinear(lin[3]), H).contiguous()
            if norm[2] is not None:
                K.rms_norm_gpu(o, norm[2], o, H, eps)
            K.residual_add_gpu(o, x, x, H)
            K.rms_norm_gpu(x, norm[1], self.xn, H, eps)
            K.absmax_quantize_gpu(self.xn, self.xq, self.absmax, H)
            gate, upv = self._bitlinear(lin[4]), self._bitlinear(lin[5])
            n_loc = lin[4]["local_rows"]
            m_loc = torch.empty(max(n_loc, 1), dtype=torch.float32, device=self.dev)
            if n_loc:
                K.relu2_mul_f32_gpu(gate, upv, m_loc, n_loc)
            m = self._gather(m_loc[:n_loc], self.inter).contiguous()
            if norm[3] is not None:
                K.rms_norm_f32in_gpu(m, norm[3], self.xn, self.inter, eps)
            else:
                K.float_to_half_gpu(m, self.xn, self.inter)
            K.absmax_quantize_gpu(self.xn, self.xq, self.absmax, self.inter)
            down = self._gather(self._bitlinear(lin[6]), H).contiguous()
            K.residual_add_gpu(down, x, x, H)
        K.rms_norm_gpu(x, self.final_norm, self.xn, H, eps)
        loc = torch.empty(max(self.head_loc.shape[0], 1), dtype=torch.float32, device=self.dev)
        if self.head_loc.shape[0]:
            K.half_gemv_gpu(self.head_loc, self.xn, loc, self.head_loc.shape[0], H)
        self.logits = self._gather(loc[: self.head_loc.shape[0]], self.vocab)
        self.seq_len += 1
        return self.logits

    def generate(self, prompt, max_tokens: int):
        """Greedy loop of src/main.cpp:266-300 (first maximum wins); returns the generated ids."""
        import torch
        out = []
        tok = None
        for t in prompt:
            lg = self.forward(int(t))
        for _ in range(max_tokens):
            tok = int(torch.argmax(lg).item())  # torch.argmax returns the first maximum on ties for 1-D input
            out.append(tok)
            if len(out) == max_tokens:
                break
            lg = self.forward(tok)
        return np.asarray(out, np.int32)
