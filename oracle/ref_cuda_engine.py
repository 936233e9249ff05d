"""The reference's forward pass (src/inference.cu:123-283) replayed with the reference's OWN CUDA
kernels, recompiled for sm_100a into oracle/_ref/libspb_refcuda.so.  Test infrastructure: the
second checker beside the CPU oracle, fast enough for the full 2B-4T shape."""
import ctypes as C

import numpy as np
import torch

import oracle


def available() -> bool:
    return oracle.refcuda() is not None


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


class RefCudaEngine:
    def __init__(self, device_model):
        self.lib = oracle.refcuda()
        self.m = device_model
        c = device_model.config
        self.c = c
        H, hd, nh, nkv = c["hidden_size"], c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"]
        I, V, mx, L = c["intermediate_size"], c["vocab_size"], c["max_position_embeddings"], c["num_hidden_layers"]
        f16 = dict(dtype=torch.float16, device="cuda")
        self.kc = [torch.zeros(nkv, mx, hd, **f16) for _ in range(L)]
        self.vc = [torch.zeros(nkv, mx, hd, **f16) for _ in range(L)]
        self.x, self.res, self.q = torch.zeros(H, **f16), torch.zeros(H, **f16), torch.zeros(max(H, nh * hd), **f16)
        self.kv, self.gate, self.up = torch.zeros(nkv * hd, **f16), torch.zeros(I, **f16), torch.zeros(I, **f16)
        self.mlp = torch.zeros(I, dtype=torch.float32, device="cuda")
        self.absmax = torch.zeros(1, dtype=torch.float32, device="cuda")
        self.logits = torch.zeros(V, dtype=torch.float32, device="cuda")
        self.scores = torch.zeros(nh, mx, dtype=torch.float32, device="cuda")
        self.seq_len = 0

    def _bitlinear(self, x, n, t, out):  # src/inference.cu:106-117
        self.lib.refcuda_absmax_reduce(_p(x), _p(self.absmax), n, None)
        self.lib.refcuda_fused_bitlinear(_p(t["d_meta"]), _p(t["d_values"]), _p(x), _p(out), _p(self.absmax),
                                         C.c_float(float(t["gamma"])), t["rows"], t["cols"], t["meta_stride"],
                                         t["values_stride"], None)

    def forward(self, token: int) -> torch.Tensor:
        c, lib = self.c, self.lib
        H, hd, nh, nkv = c["hidden_size"], c["head_dim"], c["num_attention_heads"], c["num_key_value_heads"]
        I, mx = c["intermediate_size"], c["max_position_embeddings"]
        eps, theta = C.c_float(c["rms_norm_eps"]), C.c_float(c["rope_theta"])
        pos, seq_len = self.seq_len, self.seq_len + 1
        with torch.cuda.stream(torch.cuda.default_stream()):
            self.x.copy_(self.m.embed[token])
            for l, layer in enumerate(self.m.layers):
                lin, norm = layer["linear"], layer["norm"]
                self.res.copy_(self.x)
                lib.refcuda_rms_norm(_p(self.res), _p(norm[0]), _p(self.x), H, eps, None)
                self._bitlinear(self.x, H, lin[0], self.q)
                self._bitlinear(self.x, H, lin[1], self.kv)
                lib.refcuda_rope(_p(self.q), nh, hd, pos, theta, None)
                lib.refcuda_rope(_p(self.kv), nkv, hd, pos, theta, None)
                lib.refcuda_scatter_kv(_p(self.kv), _p(self.kc[l]), nkv, hd, mx, pos, None)
                self._bitlinear(self.x, H, lin[2], self.kv)
                lib.refcuda_scatter_kv(_p(self.kv), _p(self.vc[l]), nkv, hd, mx, pos, None)
                lib.refcuda_attention_scores(_p(self.q), _p(self.kc[l]), _p(self.scores), nh, nkv, hd, mx, seq_len,
                                             C.c_float(1.0 / np.sqrt(np.float32(hd))), None)
                lib.refcuda_softmax(_p(self.scores), nh, mx, seq_len, None)
                lib.refcuda_attention_output(_p(self.scores), _p(self.vc[l]), _p(self.x), nh, nkv, hd, mx, seq_len, None)
                self._bitlinear(self.x, nh * hd, lin[3], self.q)
                lib.refcuda_rms_norm(_p(self.q), _p(norm[2]), _p(self.q), H, eps, None)
                lib.refcuda_residual_add(_p(self.q), _p(self.res), _p(self.x), H, None)
                self.res.copy_(self.x)
                lib.refcuda_rms_norm(_p(self.res), _p(norm[1]), _p(self.x), H, eps, None)
                self._bitlinear(self.x, H, lin[4], self.gate)
                self._bitlinear(self.x, H, lin[5], self.up)
                lib.refcuda_relu2_mul_f32(_p(self.gate), _p(self.up), _p(self.mlp), I, None)
                lib.refcuda_rms_norm_f32in(_p(self.mlp), _p(norm[3]), _p(self.gate), I, eps, None)
                self._bitlinear(self.gate, I, lin[6], self.q)
                lib.refcuda_residual_add(_p(self.q), _p(self.res), _p(self.x), H, None)
            lib.refcuda_rms_norm(_p(self.x), _p(self.m.final_norm), _p(self.res), H, eps, None)
            lib.refcuda_half_gemv(_p(self.m.embed), _p(self.res), _p(self.logits), c["vocab_size"], H, None)
        self.seq_len += 1
        torch.cuda.synchronize()
        return self.logits
