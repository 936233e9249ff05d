"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (they stand in for the reference's own bench inputs, which are uniform
ternary weights with a random 2-of-4 mask and x in [-5, 5], benchmarks/bench_kernels.cu:165-194).

Weights: every element ternary with P(0)=0.42, P(+1)=P(-1)=0.29; in each group of four keep
at most two non-zeros chosen uniformly among those present; groups with fewer than two
non-zeros additionally mark zero positions in ascending index until two are marked (the
format stores a marked zero as +1, sparse_ternary_tensor.h:86-91).  The effective matrix is
whatever the packed bits unpack to.  numpy only; deterministic for a given seed.
"""
from __future__ import annotations

import numpy as np

from .format import meta_words_per_row, values_words_per_row

GEMV_SHAPES = [(2560, 2560), (640, 2560), (6912, 2560), (2560, 6912), (2048, 2048),
               (5632, 2048), (2048, 5632), (4096, 4096), (8192, 2560)]
METRIC_SHAPE = (6912, 2560)
GEMM_SHAPES = [(6912, 2560), (2560, 6912)]
GEMM_BATCHES = [1, 4, 16, 64, 256, 1024]


def ternary_weights_and_mask(rows: int, cols: int, rng: np.random.Generator):
    """Returns (weights int8 {-1,0,1}, mask bool with exactly two per group)."""
    u = rng.random((rows, cols))
    w = np.where(u < 0.42, 0, np.where(u < 0.71, 1, -1)).astype(np.int8)
    keys = rng.random((rows, cols))
    g = cols // 4
    wg = w.reshape(rows, g, 4)
    nz = wg != 0
    # non-zeros first (by random key), then zeros by ascending index
    order_key = np.where(nz, keys.reshape(rows, g, 4), 2.0 + np.arange(4)[None, None, :])
    order = np.argsort(order_key, axis=-1, kind="stable")
    keep = np.zeros((rows, g, 4), bool)
    np.put_along_axis(keep, order[:, :, :2], True, axis=-1)
    return w, keep.reshape(rows, cols)


def pack_numpy(w: np.ndarray, mask: np.ndarray):
    """Vectorised packer (numpy): the same bits as pack_from_dense.  Used to build large
    synthetic matrices quickly; tests check it against the C packers."""
    rows, cols = w.shape
    g = cols // 4
    ms, vs = meta_words_per_row(cols), values_words_per_row(cols)
    mg = mask.reshape(rows, g, 4)
    bitmap = (mg.astype(np.uint32) << np.arange(4, dtype=np.uint32)[None, None, :]).sum(-1, dtype=np.uint32)
    rank = np.cumsum(mg, axis=-1) - 1  # 0 for the first kept, 1 for the second
    neg = (w.reshape(rows, g, 4) < 0) & mg
    signs = (neg.astype(np.uint32) << np.where(mg, rank, 0).astype(np.uint32)).sum(-1, dtype=np.uint32)
    bm = np.zeros((rows, ms * 8), np.uint32)
    bm[:, :g] = bitmap
    sg = np.zeros((rows, vs * 16), np.uint32)
    sg[:, :g] = signs
    meta = (bm.reshape(rows, ms, 8) << (4 * np.arange(8, dtype=np.uint32))[None, None, :]).sum(-1, dtype=np.uint32)
    values = (sg.reshape(rows, vs, 16) << (2 * np.arange(16, dtype=np.uint32))[None, None, :]).sum(-1, dtype=np.uint32)
    return np.ascontiguousarray(meta), np.ascontiguousarray(values)


def sparse_matrix(rows: int, cols: int, seed: int = 0):
    """(meta, values, meta_stride, values_stride) of one synthetic matrix."""
    rng = np.random.default_rng(seed)
    w, mask = ternary_weights_and_mask(rows, cols, rng)
    meta, values = pack_numpy(w, mask)
    return meta, values, meta.shape[1], values.shape[1]


def gemv_case(rows: int, cols: int, seed: int = 0):
    """Weights as above plus x ~ U{-127..127} int8; activation scale 1/127 (absmax 1.0),
    weight scale gamma = 1.0."""
    rng = np.random.default_rng(seed)
    w, mask = ternary_weights_and_mask(rows, cols, rng)
    meta, values = pack_numpy(w, mask)
    x = rng.integers(-127, 128, cols, dtype=np.int8)
    return {"meta": meta, "values": values, "x": x, "rows": rows, "cols": cols,
            "meta_stride": meta.shape[1], "values_stride": values.shape[1],
            "absmax": np.float32(1.0), "gamma": np.float32(1.0)}


def gemm_case(rows: int, cols: int, n: int, seed: int = 0):
    rng = np.random.default_rng(seed)
    w, mask = ternary_weights_and_mask(rows, cols, rng)
    meta, values = pack_numpy(w, mask)
    X = rng.integers(-127, 128, (n, cols), dtype=np.int8)
    absmax = rng.uniform(0.5, 4.0, n).astype(np.float32)
    return {"meta": meta, "values": values, "X": X, "absmax": absmax, "rows": rows, "cols": cols, "n": n,
            "meta_stride": meta.shape[1], "values_stride": values.shape[1]}


def gemv_algorithmic_bytes(rows: int, cols: int) -> int:
    """The reference's byte count for one GEMV (benchmarks/bench_kernels.cu:248):
    both weight streams + int8 x + int32 y."""
    return rows * 4 * (meta_words_per_row(cols) + values_words_per_row(cols)) + cols + 4 * rows


# ---- models -------------------------------------------------------------------------

BITNET_2B = dict(hidden_size=2560, num_hidden_layers=30, num_attention_heads=20, num_key_value_heads=5,
                 head_dim=128, intermediate_size=6912, vocab_size=128256, max_position_embeddings=4096,
                 rms_norm_eps=1e-5, rope_theta=500000.0)
LLAMA_70B_SHAPE = dict(hidden_size=8192, num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
                       head_dim=128, intermediate_size=28672, vocab_size=128256, max_position_embeddings=4096,
                       rms_norm_eps=1e-5, rope_theta=500000.0)
TINY = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
            intermediate_size=512, vocab_size=512, max_position_embeddings=64, rms_norm_eps=1e-5,
            rope_theta=10000.0)

LINEAR_NAMES = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
NORM_NAMES = ["input_layernorm", "post_attention_layernorm", "attn_sub_norm", "ffn_sub_norm"]


def linear_shapes(cfg: dict):
    H, qd = cfg["hidden_size"], cfg["num_attention_heads"] * cfg["head_dim"]
    kvd, I = cfg["num_key_value_heads"] * cfg["head_dim"], cfg["intermediate_size"]
    return [(qd, H), (kvd, H), (kvd, H), (H, qd), (I, H), (I, H), (H, I)]


def random_model(cfg: dict, seed: int = 0, layers: int | None = None, shared_layer: bool = False):
    """Random-init model of the given architecture as host numpy arrays.

    Per matrix the ternary 2:4 distribution above; gamma ~ U(0.5, 2)/sqrt(cols) so that
    activations stay inside the fp16 range; norm gains N(1, 0.02) fp32; embedding fp16
    N(0, 0.02), tied LM head.  With shared_layer=True all layers alias layer 0's arrays
    (saves host time when only throughput matters; byte counts on the device are still one
    copy per layer because each layer is uploaded separately).
    """
    L = cfg["num_hidden_layers"] if layers is None else layers
    rng = np.random.default_rng(seed)
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    model = {"config": dict(cfg, num_hidden_layers=L), "layers": []}
    model["embed"] = (rng.standard_normal((cfg["vocab_size"], H), dtype=np.float32) * 0.02).astype(np.float16)
    model["final_norm"] = (1.0 + 0.02 * rng.standard_normal(H)).astype(np.float32)
    for l in range(L):
        if shared_layer and l > 0:
            model["layers"].append(model["layers"][0])
            continue
        layer = {"linear": [], "norm": []}
        for i, (r, c) in enumerate(linear_shapes(cfg)):
            lrng = np.random.default_rng([seed, l, i])
            w, mask = ternary_weights_and_mask(r, c, lrng)
            meta, values = pack_numpy(w, mask)
            gamma = np.float32(lrng.uniform(0.5, 2.0) / np.sqrt(c))
            layer["linear"].append({"meta": meta, "values": values, "gamma": gamma, "rows": r, "cols": c,
                                    "meta_stride": meta.shape[1], "values_stride": values.shape[1]})
        for n in (H, H, H, I):
            layer["norm"].append((1.0 + 0.02 * rng.standard_normal(n)).astype(np.float32))
        model["layers"].append(layer)
    return model


# ---- the same distributions generated on the GPU (torch) ------------------------------------------
# A 2B-4T-shape model has 210 distinct matrices and a 70B-shape layer 1.2e9 weights; numpy needs seconds per
# matrix, the GPU milliseconds.  Same draw rules as ternary_weights_and_mask / pack_numpy, with torch's
# generator (so the bits differ from the numpy ones for the same seed, the distribution does not).

def device_sparse_matrix(rows: int, cols: int, seed, device=None, chunk_rows: int = 2048):
    """(meta, values) int32 CUDA tensors [rows, cols/32] and [rows, cols/64] of one synthetic matrix.
    cols must be a multiple of 64.  Generated `chunk_rows` rows at a time to bound temporaries."""
    import torch
    if cols % 64:
        raise ValueError("device_sparse_matrix: cols must be a multiple of 64")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(np.random.SeedSequence(seed).generate_state(1, np.uint64)[0] >> 1))
    g = cols // 4
    meta = torch.empty((rows, cols // 32), dtype=torch.int32, device=dev)
    values = torch.empty((rows, cols // 64), dtype=torch.int32, device=dev)
    idx = torch.arange(4, device=dev, dtype=torch.float32)
    sh4 = torch.arange(4, device=dev, dtype=torch.int64)
    for r0 in range(0, rows, chunk_rows):
        n = min(chunk_rows, rows - r0)
        u = torch.rand((n, g, 4), generator=gen, device=dev)
        neg = u >= 0.71
        nz = u >= 0.42
        keys = torch.rand((n, g, 4), generator=gen, device=dev)
        order_key = torch.where(nz, keys, 2.0 + idx)           # non-zeros first (random), then zeros by index
        kept = torch.argsort(order_key, dim=-1, stable=True)[..., :2]
        mask = torch.zeros((n, g, 4), dtype=torch.bool, device=dev)
        mask.scatter_(-1, kept, True)
        bitmap = (mask.to(torch.int64) << sh4).sum(-1)                       # [n, g], 4 bits
        rank = torch.cumsum(mask.to(torch.int64), -1) - 1
        sneg = (neg & mask).to(torch.int64) << torch.where(mask, rank, torch.zeros_like(rank))
        signs = sneg.sum(-1)                                                  # [n, g], 2 bits
        m = (bitmap.view(n, g // 8, 8) << (4 * torch.arange(8, device=dev, dtype=torch.int64))).sum(-1)
        v = (signs.view(n, g // 16, 16) << (2 * torch.arange(16, device=dev, dtype=torch.int64))).sum(-1)
        meta[r0:r0 + n] = m.to(torch.int32)      # int64 -> int32 keeps the low 32 bits
        values[r0:r0 + n] = v.to(torch.int32)
    return meta, values


class DeviceRandomModel:
    """Random-init model generated on the current CUDA device, in the attribute layout of
    spbitnet_b200.engine.DeviceModel (config, device, embed, final_norm, lm_head, layers).  Every matrix of
    every layer has its own seed (seed, layer, matrix); with repeat_layer=True layer 0 is generated once and
    every further layer is a separate device COPY of it (for shapes where only throughput matters: the HBM
    traffic is still one distinct copy per layer).  Distributions as in random_model()."""

    def __init__(self, cfg: dict, seed: int = 0, repeat_layer: bool = False, device=None):
        import torch
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.config, self.device = dict(cfg), dev
        H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
        gen = torch.Generator(device=dev)
        gen.manual_seed(1000003 * seed + 17)
        self.embed = (torch.randn((cfg["vocab_size"], H), generator=gen, device=dev) * 0.02).to(torch.float16)
        self.final_norm = 1.0 + 0.02 * torch.randn(H, generator=gen, device=dev)
        self.lm_head = None
        self.layers = []
        host = np.random.default_rng([seed, 99])
        for l in range(L):
            if repeat_layer and l > 0:
                first = self.layers[0]
                lin = [dict(t, d_meta=t["d_meta"].clone(), d_values=t["d_values"].clone()) for t in first["linear"]]
                self.layers.append({"linear": lin, "norm": [n.clone() for n in first["norm"]]})
                continue
            lin = []
            for i, (r, c) in enumerate(linear_shapes(cfg)):
                meta, values = device_sparse_matrix(r, c, [seed, l, i], dev)
                gamma = np.float32(host.uniform(0.5, 2.0) / np.sqrt(c))
                lin.append({"d_meta": meta, "d_values": values, "gamma": gamma, "rows": r, "cols": c,
                            "meta_stride": meta.shape[1], "values_stride": values.shape[1]})
            norms = [1.0 + 0.02 * torch.randn(n, generator=gen, device=dev) for n in (H, H, H, I)]
            self.layers.append({"linear": lin, "norm": norms})

    def sparse_bytes(self) -> int:
        return sum(t["d_meta"].numel() * 4 + t["d_values"].numel() * 4 for L in self.layers for t in L["linear"])

    def to_host(self) -> dict:
        """The model as host numpy arrays in the random_model() layout (what the CPU oracle takes)."""
        def u32(t):
            return np.ascontiguousarray(t.cpu().numpy()).view(np.uint32)
        layers = []
        for L in self.layers:
            lin = [{"meta": u32(t["d_meta"]), "values": u32(t["d_values"]), "gamma": t["gamma"], "rows": t["rows"],
                    "cols": t["cols"], "meta_stride": t["meta_stride"], "values_stride": t["values_stride"]}
                   for t in L["linear"]]
            layers.append({"linear": lin, "norm": [n.cpu().numpy() for n in L["norm"]]})
        return {"config": dict(self.config), "layers": layers, "final_norm": self.final_norm.cpu().numpy(),
                "embed": self.embed.view(self.embed.dtype).cpu().numpy()}
