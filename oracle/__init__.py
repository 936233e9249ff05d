"""CPU oracle for the sparse-ternary hot path -- TEST INFRASTRUCTURE ONLY.

ctypes bindings of oracle/libspb_oracle.so (the C restatement, spb_oracle.c), of
oracle/_ref/libspb_ref.so (the reference's own header behind a shim, when built) and of
oracle/_ref/libspb_refcuda.so (the reference's CUDA kernels recompiled for sm_100a, when
built).  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference legs
may import this package; the product (spbitnet_b200/) never does.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_ORACLE = HERE / "libspb_oracle.so"
_TESTGEN = HERE / "libspb_testgen.so"
_REF = HERE / "_ref" / "libspb_ref.so"
_REFCUDA = HERE / "_ref" / "libspb_refcuda.so"
_CSLT = HERE / "libspb_cslt.so"


def build(quiet: bool = True) -> None:
    """make -C oracle: always the restatement; the _ref targets only where the reference tree exists."""
    subprocess.run(["make", "-f", str(HERE / "Makefile")], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


_libs: dict = {}


def _load(path: Path):
    key = str(path)
    if key not in _libs:
        if not path.exists():
            if path in (_ORACLE, _TESTGEN):
                build()
            if not path.exists():
                return None
        _libs[key] = C.CDLL(key)
    return _libs[key]


def lib():
    l = _load(_ORACLE)
    if l is None:
        raise ImportError("oracle/libspb_oracle.so missing and could not be built (gcc + make needed)")
    return l


def ref():
    """The reference-header shim, or None when oracle/_ref was not built."""
    return _load(_REF)


def refcuda():
    """The reference CUDA kernels for sm_100a, or None."""
    return _load(_REFCUDA)


def cslt():
    """The cuSPARSELt comparison shim (cslt_shim.cpp), or None when it was not built."""
    try:
        return _load(_CSLT)
    except OSError:  # the shim is there but libcusparseLt is not
        return None


def _p(a):
    if a is None:
        return C.c_void_p(0)
    return C.c_void_p(a.ctypes.data)


def meta_words_per_row(cols):
    return lib().spbo_meta_words_per_row(int(cols))


def values_words_per_row(cols):
    return lib().spbo_values_words_per_row(int(cols))


def pack_from_dense(w, mask):
    w = np.ascontiguousarray(w, np.int8)
    m = np.ascontiguousarray(mask).astype(np.uint8)
    rows, cols = w.shape
    meta = np.zeros((rows, meta_words_per_row(cols)), np.uint32)
    values = np.zeros((rows, values_words_per_row(cols)), np.uint32)
    f = lib().spbo_pack_from_dense
    f.restype = C.c_long
    rc = f(_p(w), _p(m), rows, cols, _p(meta), _p(values))
    if rc != 0:
        raise ValueError(f"group {-rc - 1} does not keep exactly two entries")
    return meta, values


def pack_with_pruning(latent):
    x = np.ascontiguousarray(latent, np.float32)
    rows, cols = x.shape
    meta = np.zeros((rows, meta_words_per_row(cols)), np.uint32)
    values = np.zeros((rows, values_words_per_row(cols)), np.uint32)
    lib().spbo_pack_with_pruning(_p(x), rows, cols, _p(meta), _p(values))
    return meta, values


def unpack_to_int8(meta, values, rows, cols):
    meta = np.ascontiguousarray(meta, np.uint32)
    values = np.ascontiguousarray(values, np.uint32)
    out = np.empty((rows, cols), np.int8)
    lib().spbo_unpack_to_int8(_p(meta), _p(values), rows, cols, meta.shape[1], values.shape[1], _p(out))
    return out


def validate(meta, rows, cols):
    meta = np.ascontiguousarray(meta, np.uint32)
    f = lib().spbo_validate
    f.restype = C.c_long
    return int(f(_p(meta), rows, cols, meta.shape[1]))


def sparse_gemv(meta, values, x, rows, cols, threads: int = 1):
    meta = np.ascontiguousarray(meta, np.uint32)
    values = np.ascontiguousarray(values, np.uint32)
    x = np.ascontiguousarray(x, np.int8)
    y = np.empty(rows, np.int32)
    if threads <= 1:
        lib().spbo_sparse_gemv(_p(meta), _p(values), _p(x), _p(y), rows, cols, meta.shape[1], values.shape[1])
    else:
        lib().spbo_sparse_gemv_mt(_p(meta), _p(values), _p(x), _p(y), rows, cols, meta.shape[1],
                                  values.shape[1], int(threads))
    return y


def sparse_gemm(meta, values, X, rows, cols):
    meta = np.ascontiguousarray(meta, np.uint32)
    values = np.ascontiguousarray(values, np.uint32)
    X = np.ascontiguousarray(X, np.int8)
    n = X.shape[0]
    Y = np.empty((n, rows), np.int32)
    lib().spbo_sparse_gemm(_p(meta), _p(values), _p(X), _p(Y), rows, cols, n, meta.shape[1], values.shape[1])
    return Y


def int8_gemm(A, B):
    A = np.ascontiguousarray(A, np.int8)
    B = np.ascontiguousarray(B, np.int8)
    m, k = A.shape
    n = B.shape[1]
    D = np.empty((m, n), np.int32)
    lib().spbo_int8_gemm(_p(A), _p(B), _p(D), m, k, n)
    return D


def _h(a):
    """float16 array -> contiguous uint16 view."""
    return np.ascontiguousarray(a, np.float16).view(np.uint16)


def absmax_reduce(x):
    f = lib().spbo_absmax_reduce
    f.restype = C.c_float
    xh = _h(x)
    return np.float32(f(_p(xh), xh.size))


def absmax_quantize(x):
    f = lib().spbo_absmax_quantize
    f.restype = C.c_float
    xh = _h(x)
    q = np.empty(xh.size, np.int8)
    a = f(_p(xh), _p(q), xh.size)
    return q, np.float32(a)


def dequantize(acc, absmax, gamma):
    acc = np.ascontiguousarray(acc, np.int32)
    out = np.empty(acc.size, np.uint16)
    lib().spbo_dequantize(_p(acc), _p(out), C.c_float(absmax), C.c_float(gamma), acc.size)
    return out.view(np.float16)


def dequantize_f32(acc, absmax, gamma):
    acc = np.ascontiguousarray(acc, np.int32)
    out = np.empty(acc.size, np.float32)
    lib().spbo_dequantize_f32(_p(acc), _p(out), C.c_float(absmax), C.c_float(gamma), acc.size)
    return out


def fused_bitlinear(meta, values, x, absmax, gamma, rows, cols):
    meta = np.ascontiguousarray(meta, np.uint32)
    values = np.ascontiguousarray(values, np.uint32)
    xh = _h(x)
    out = np.empty(rows, np.uint16)
    lib().spbo_fused_bitlinear(_p(meta), _p(values), _p(xh), _p(out), C.c_float(absmax), C.c_float(gamma),
                               rows, cols, meta.shape[1], values.shape[1])
    return out.view(np.float16)


def rms_norm(x, w, eps):
    xh = _h(x)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty(xh.size, np.uint16)
    lib().spbo_rms_norm(_p(xh), _p(w), _p(out), xh.size, C.c_float(eps))
    return out.view(np.float16)


def rms_norm_f32in(x, w, eps):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    out = np.empty(x.size, np.uint16)
    lib().spbo_rms_norm_f32in(_p(x), _p(w), _p(out), x.size, C.c_float(eps))
    return out.view(np.float16)


def rope(vec, num_heads, head_dim, pos, theta):
    v = _h(vec).copy()
    lib().spbo_rope(_p(v), num_heads, head_dim, pos, C.c_float(theta))
    return v.view(np.float16)


def scatter_kv(src, cache, num_kv_heads, head_dim, max_seq_len, pos):
    c = _h(cache).copy()
    lib().spbo_scatter_kv(_p(_h(src)), _p(c), num_kv_heads, head_dim, max_seq_len, pos)
    return c.view(np.float16)


def attention_scores(Q, K, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len, scale):
    s = np.zeros((num_heads, max_seq_len), np.float32)
    lib().spbo_attention_scores(_p(_h(Q)), _p(_h(K)), _p(s), num_heads, num_kv_heads, head_dim, max_seq_len,
                                seq_len, C.c_float(scale))
    return s


def softmax(scores, seq_len):
    s = np.ascontiguousarray(scores, np.float32).copy()
    lib().spbo_softmax(_p(s), s.shape[0], s.shape[1], seq_len)
    return s


def attention_output(scores, V, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len):
    s = np.ascontiguousarray(scores, np.float32)
    out = np.empty(num_heads * head_dim, np.uint16)
    lib().spbo_attention_output(_p(s), _p(_h(V)), _p(out), num_heads, num_kv_heads, head_dim, max_seq_len, seq_len)
    return out.view(np.float16)


def attention(Q, K, V, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len, scale):
    s = attention_scores(Q, K, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len, scale)
    s = softmax(s, seq_len)
    return attention_output(s, V, num_heads, num_kv_heads, head_dim, max_seq_len, seq_len)


def relu2_mul(gate, up):
    g, u = _h(gate), _h(up)
    out = np.empty(g.size, np.uint16)
    lib().spbo_relu2_mul(_p(g), _p(u), _p(out), g.size)
    return out.view(np.float16)


def relu2_mul_f32(gate, up):
    g, u = _h(gate), _h(up)
    out = np.empty(g.size, np.float32)
    lib().spbo_relu2_mul_f32(_p(g), _p(u), _p(out), g.size)
    return out


def float_to_half(x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.size, np.uint16)
    lib().spbo_float_to_half(_p(x), _p(out), x.size)
    return out.view(np.float16)


def residual_add(a, b):
    a, b = _h(a), _h(b)
    out = np.empty(a.size, np.uint16)
    lib().spbo_residual_add(_p(a), _p(b), _p(out), a.size)
    return out.view(np.float16)


def half_gemv(W, x):
    Wh, xh = _h(W), _h(x)
    rows, cols = Wh.shape
    y = np.empty(rows, np.float32)
    lib().spbo_half_gemv(_p(Wh), _p(xh), _p(y), rows, cols)
    return y


def argmax(v):
    v = np.ascontiguousarray(v, np.float32)
    return int(lib().spbo_argmax(_p(v), v.size))


class Engine:
    """spbo_engine: the reference forward pass (src/inference.cu:123-283) on the CPU, for a
    host model in the spbitnet_b200.synth.random_model layout."""

    def __init__(self, model: dict, use_sub_norm: bool = True):
        L = lib()
        L.spbo_engine_create.restype = C.c_void_p
        L.spbo_engine_forward.restype = C.POINTER(C.c_float)
        cfg = model["config"]
        self.cfg = cfg
        self._keep = model
        self._h = C.c_void_p(L.spbo_engine_create(
            cfg["hidden_size"], cfg["num_hidden_layers"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
            cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"], cfg["max_position_embeddings"],
            C.c_float(cfg["rms_norm_eps"]), C.c_float(cfg["rope_theta"])))
        for l, layer in enumerate(model["layers"]):
            for i, t in enumerate(layer["linear"]):
                L.spbo_engine_set_linear(self._h, l, i, _p(t["meta"]), _p(t["values"]), C.c_float(t["gamma"]),
                                         t["rows"], t["cols"], t["meta_stride"], t["values_stride"])
            for i, n in enumerate(layer["norm"]):
                if i >= 2 and not use_sub_norm:
                    continue
                L.spbo_engine_set_norm(self._h, l, i, _p(n))
        self._embed = np.ascontiguousarray(model["embed"]).view(np.uint16)
        L.spbo_engine_set_globals(self._h, _p(self._embed), C.c_void_p(0), _p(model["final_norm"]))

    def forward(self, token: int) -> np.ndarray:
        ptr = lib().spbo_engine_forward(self._h, int(token))
        return np.ctypeslib.as_array(ptr, shape=(self.cfg["vocab_size"],)).copy()

    def reset(self):
        lib().spbo_engine_reset(self._h)

    @property
    def seq_len(self):
        return lib().spbo_engine_seq_len(self._h)

    def generate(self, prompt, max_tokens):
        """src/main.cpp:266-300 without the EOS stop."""
        for t in prompt[:-1]:
            self.forward(int(t))
        tok, out, logits = int(prompt[-1]), [], []
        for _ in range(max_tokens):
            lg = self.forward(tok)
            tok = argmax(lg)
            out.append(tok)
            logits.append(lg)
        return np.array(out, np.int32), logits

    def __del__(self):
        try:
            lib().spbo_engine_destroy(self._h)
        except Exception:
            pass


def testgen_gemv_case(seed, rows, cols, xlo, xhi):
    """Inputs of the reference's seeded GEMV tests (tests/test_sparse_ternary.cu:252-402)."""
    l = _load(_TESTGEN)
    w = np.empty((rows, cols), np.int8)
    m = np.empty((rows, cols), np.uint8)
    x = np.empty(cols, np.int8)
    l.testgen_gemv_case(C.c_uint(seed), rows, cols, xlo, xhi, _p(w), _p(m), _p(x))
    return w, m, x


# ---- the reference's own code (oracle/_ref), when built -------------------------------

def ref_pack_from_dense(w, mask):
    r = ref()
    w = np.ascontiguousarray(w, np.int8)
    m = np.ascontiguousarray(mask).astype(np.uint8)
    rows, cols = w.shape
    meta = np.zeros((rows, r.ref_meta_stride(cols)), np.uint32)
    values = np.zeros((rows, r.ref_values_stride(cols)), np.uint32)
    r.ref_pack_from_dense(_p(w), _p(m), rows, cols, _p(meta), _p(values))
    return meta, values


def ref_pack_with_pruning(latent):
    r = ref()
    x = np.ascontiguousarray(latent, np.float32)
    rows, cols = x.shape
    meta = np.zeros((rows, r.ref_meta_stride(cols)), np.uint32)
    values = np.zeros((rows, r.ref_values_stride(cols)), np.uint32)
    r.ref_pack_with_pruning(_p(x), rows, cols, _p(meta), _p(values))
    return meta, values


def ref_roundtrip(w, mask):
    r = ref()
    w = np.ascontiguousarray(w, np.int8)
    m = np.ascontiguousarray(mask).astype(np.uint8)
    out = np.empty_like(w)
    r.ref_roundtrip(_p(w), _p(m), w.shape[0], w.shape[1], _p(out))
    return out


def ref_cpu_sparse_gemv(w, mask, x, threads: int = 1, repeats: int = 1):
    r = ref()
    w = np.ascontiguousarray(w, np.int8)
    m = np.ascontiguousarray(mask).astype(np.uint8)
    x = np.ascontiguousarray(x, np.int8)
    y = np.empty(w.shape[0], np.int32)
    r.ref_cpu_sparse_gemv(_p(w), _p(m), w.shape[0], w.shape[1], _p(x), _p(y), int(threads), int(repeats))
    return y


class RefCpuGemv:
    """The reference's CPU GEMV (tests/test_sparse_ternary.cu:17-33) over `slices` row slices, one thread each,
    packed once.  run(x, repeats, dot_only): dot_only=False unpacks and multiplies every repeat (the reference's
    cpu_sparse_gemv), dot_only=True multiplies pre-unpacked rows."""

    def __init__(self, w, mask, slices: int = 1):
        self._r = ref()
        if self._r is None:
            raise RuntimeError("oracle/_ref/libspb_ref.so is not built")
        self._r.ref_gemv_ctx_create.restype = C.c_void_p
        self._r.ref_gemv_ctx_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        self._r.ref_gemv_ctx_destroy.argtypes = [C.c_void_p]
        w = np.ascontiguousarray(w, np.int8)
        m = np.ascontiguousarray(mask).astype(np.uint8)
        self.rows, self.cols = w.shape
        self._h = C.c_void_p(self._r.ref_gemv_ctx_create(_p(w), _p(m), self.rows, self.cols, int(slices)))

    def run(self, x, repeats: int = 1, dot_only: bool = False):
        x = np.ascontiguousarray(x, np.int8)
        y = np.empty(self.rows, np.int32)
        self._r.ref_gemv_ctx_run(self._h, _p(x), _p(y), int(repeats), 1 if dot_only else 0)
        return y

    def __del__(self):
        try:
            if self._h:
                self._r.ref_gemv_ctx_destroy(self._h)
                self._h = None
        except Exception:
            pass


class CusparseLtGemm:
    """spbitnet::CuSparseLtGemm (include/spbitnet/cusparselt_backend.h:28-77) through cslt_shim.cpp: plan at
    construction, prepare(dense int8 [m, k] device pointer) once, execute(B, D) per call.  Pointers are device
    addresses (ints); stream is a CUDA stream handle (int) or None."""

    def __init__(self, m: int, k: int, n: int):
        self._l = cslt()
        if self._l is None:
            raise RuntimeError("oracle/libspb_cslt.so is not built or cuSPARSELt is missing")
        l = self._l
        l.cslt_last_error.restype = C.c_char_p
        l.cslt_create.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        l.cslt_destroy.argtypes = [C.c_void_p]
        l.cslt_prepare.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        l.cslt_execute.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        l.cslt_pruned.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        self.m, self.k, self.n = m, k, n
        self._h = C.c_void_p()
        self._check(l.cslt_create(m, k, n, C.byref(self._h)))

    def _check(self, rc):
        if rc:
            raise RuntimeError(f"cuSPARSELt shim error {rc}: {self._l.cslt_last_error().decode()}")

    def prepare(self, d_weights: int, stream=None):
        self._check(self._l.cslt_prepare(self._h, C.c_void_p(d_weights), C.c_void_p(stream or 0)))

    def execute(self, d_B: int, d_D: int, stream=None):
        self._check(self._l.cslt_execute(self._h, C.c_void_p(d_B), C.c_void_p(d_D), C.c_void_p(stream or 0)))

    def pruned(self, d_out: int, stream=None):
        self._check(self._l.cslt_pruned(self._h, C.c_void_p(d_out), C.c_void_p(stream or 0)))

    def close(self):
        if self._h:
            self._l.cslt_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_DROPIN = HERE / "_ref" / "libspb_dropin.so"
DROPIN_GEMV_TEST = HERE / "_ref" / "dropin_gemv_test"


def dropin():
    """The reference's own engine + loader built over this repository's kernels (ref_dropin_shim.cu), or None."""
    try:
        return _load(_DROPIN)
    except OSError:
        return None


class DropInEngine:
    """spbitnet::Model::load + spbitnet::InferenceEngine (the reference's unmodified host code) running on the
    sm_100a library through the drop-in headers.  forward(token) returns the logits as a host array."""

    def __init__(self, model_dir):
        self._l = dropin()
        if self._l is None:
            raise RuntimeError("oracle/_ref/libspb_dropin.so is not built")
        l = self._l
        l.dropin_create.restype = C.c_void_p
        l.dropin_create.argtypes = [C.c_char_p]
        l.dropin_last_error.restype = C.c_char_p
        for name in ("dropin_destroy", "dropin_reset"):
            getattr(l, name).argtypes = [C.c_void_p]
        l.dropin_vocab.argtypes = [C.c_void_p]
        l.dropin_seq_len.argtypes = [C.c_void_p]
        l.dropin_forward.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        h = l.dropin_create(str(model_dir).encode())
        if not h:
            raise RuntimeError(l.dropin_last_error().decode())
        self._h = C.c_void_p(h)
        self.vocab = l.dropin_vocab(self._h)

    def forward(self, token: int) -> np.ndarray:
        out = np.empty(self.vocab, np.float32)
        if self._l.dropin_forward(self._h, int(token), _p(out)):
            raise RuntimeError(self._l.dropin_last_error().decode())
        return out

    def reset(self):
        self._l.dropin_reset(self._h)

    @property
    def seq_len(self):
        return self._l.dropin_seq_len(self._h)

    def close(self):
        if self._h:
            self._l.dropin_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_REFTOK = HERE / "_ref" / "libspb_reftok.so"


class RefTokenizer:
    """The reference's own spbitnet::Tokenizer (src/tokenizer.cpp, unmodified) through ref_tokenizer_shim.cpp."""

    def __init__(self, path):
        self._l = _load(_REFTOK)
        if self._l is None:
            raise RuntimeError("oracle/_ref/libspb_reftok.so is not built")
        l = self._l
        l.reftok_load.restype = C.c_void_p
        l.reftok_load.argtypes = [C.c_char_p]
        l.reftok_destroy.argtypes = [C.c_void_p]
        l.reftok_vocab_size.argtypes = [C.c_void_p]
        l.reftok_encode.argtypes = [C.c_void_p, C.c_char_p, C.c_size_t, C.c_void_p, C.c_int]
        l.reftok_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
        h = l.reftok_load(str(path).encode())
        if not h:
            raise RuntimeError(f"reference tokenizer could not load {path}")
        self._h = C.c_void_p(h)

    @staticmethod
    def available() -> bool:
        return _REFTOK.exists()

    @property
    def vocab_size(self):
        return self._l.reftok_vocab_size(self._h)

    def encode(self, raw: bytes):
        n = self._l.reftok_encode(self._h, raw, len(raw), None, 0)
        ids = np.zeros(max(n, 1), np.int32)
        self._l.reftok_encode(self._h, raw, len(raw), _p(ids), n)
        return [int(i) for i in ids[:n]]

    def decode(self, ids) -> bytes:
        a = np.ascontiguousarray(ids, np.int32)
        n = self._l.reftok_decode(self._h, _p(a), a.size, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._l.reftok_decode(self._h, _p(a), a.size, buf, n + 1)
        return buf.raw[:n]

    def __del__(self):
        try:
            if self._h:
                self._l.reftok_destroy(self._h)
                self._h = None
        except Exception:
            pass
