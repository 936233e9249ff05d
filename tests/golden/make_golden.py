#!/usr/bin/env python3
"""Generates the golden vectors under tests/golden/ from the reference itself.

Run where the reference checkout is present (pass its location with --ref) and oracle/_ref is built:
    python tests/golden/make_golden.py [--ref <reference checkout>]

Sources of truth used here:
  * python/convert_model.py   generate_24_mask, quantize_ternary_absmean, pack_sparse_ternary
  * python/generate_sparse_mask.py  export_sparse_ternary / import_sparse_ternary (loop packer)
  * python/baseline_pytorch.py  SparseBitLinear.forward, rms_norm, rope_inplace, attention,
                                relu2_mul, half_gemv, InferenceEngine.forward
  * include/spbitnet/sparse_ternary_tensor.h through oracle/_ref/libspb_ref.so
    (pack_from_dense, pack_with_pruning, unpack_to_int8, and the test-style CPU GEMV)
  * src/tokenizer.cpp through oracle/_ref/libspb_reftok.so (encode / decode on the synthetic tokenizer.json of
    tests/tokenizer_fixture.py) -> tokenizer_golden.json
The tests read only the files written here; nothing at test time touches the reference.
"""
import argparse
import hashlib
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default="/root/reference")
    args = ap.parse_args()
    sys.path.insert(0, str(Path(args.ref) / "python"))
    import torch
    import convert_model as cm
    import generate_sparse_mask as gsm
    import baseline_pytorch as bp
    import oracle
    from spbitnet_b200 import synth

    assert oracle.ref() is not None, "build oracle/_ref first (make -f oracle/Makefile)"

    # ---- 1. Python packers on a float matrix (convert_model.py:88-207) ------------------
    rng = np.random.default_rng(42)
    wf = (rng.standard_normal((32, 128)) * 0.05).astype(np.float32)
    wf[3, 8:12] = [0.1, 0.1, 0.1, 0.1]        # magnitude ties: lower index must lose to the stable top-2 rule
    wf[5, 0:4] = [0.0, 0.0, 0.0, 0.0]         # all-zero group: kept zeros pack as +1
    mask = cm.generate_24_mask(wf)
    ternary, gamma = cm.quantize_ternary_absmean(wf)
    sparse = ternary * mask.astype(np.int8)
    zero_at_mask = mask & (sparse == 0)
    sparse[zero_at_mask & (wf >= 0)] = 1
    sparse[zero_at_mask & (wf < 0)] = -1
    meta, values, ms, vs = cm.pack_sparse_ternary(sparse, mask)
    np.savez_compressed(HERE / "format_py.npz", weights_f32=wf, mask=mask, ternary=ternary,
                        gamma=np.float64(gamma), sparse=sparse, meta=meta, values=values,
                        meta_stride=ms, values_stride=vs)

    # ---- 2. the reference header: packers, unpack, the tests' seeded GEMV cases ----------
    w42, m42, x42 = oracle.testgen_gemv_case(42, 64, 256, -5, 5)
    meta42, values42 = oracle.ref_pack_from_dense(w42, m42)
    y42 = oracle.ref_cpu_sparse_gemv(w42, m42, x42)
    dense42 = oracle.ref_roundtrip(w42, m42)
    w77, m77, x77 = oracle.testgen_gemv_case(77, 2048, 2048, -5, 5)
    y77 = oracle.ref_cpu_sparse_gemv(w77, m77, x77)
    h77 = hashlib.sha256(w77.tobytes() + m77.tobytes() + x77.tobytes()).hexdigest()
    lat = (np.random.default_rng(7).standard_normal((16, 64)) * 0.8).astype(np.float32)
    lat[0, 0:4] = [0.7, -0.7, 0.7, -0.7]      # four-way tie
    lat[1, 4:8] = [0.2, -0.6, 0.5, -0.5]      # tie for second place, and the +-0.5 threshold
    pmeta, pvalues = oracle.ref_pack_with_pruning(lat)
    np.savez_compressed(HERE / "format_ref.npz", w42=w42, m42=m42, x42=x42, meta42=meta42, values42=values42,
                        y42=y42, dense42=dense42, y77=y77, sha77=np.array(h77), latent=lat, pmeta=pmeta,
                        pvalues=pvalues)

    # ---- 3. baseline_pytorch ops (baseline_pytorch.py:89-207) -----------------------------
    r = np.random.default_rng(3)
    out = {}
    x = (r.standard_normal(2560) * 1.7).astype(np.float16)
    wn = (1 + 0.02 * r.standard_normal(2560)).astype(np.float32)
    out["norm_x"], out["norm_w"] = x, wn
    out["norm_y"] = bp.rms_norm(torch.from_numpy(x), torch.from_numpy(wn), 1e-5).numpy()
    xf = (r.standard_normal(1024) * 300).astype(np.float32)
    wf2 = (1 + 0.02 * r.standard_normal(1024)).astype(np.float32)
    out["normf_x"], out["normf_w"] = xf, wf2
    out["normf_y"] = bp.rms_norm(torch.from_numpy(xf), torch.from_numpy(wf2), 1e-5).numpy()
    v = (r.standard_normal(4 * 128)).astype(np.float16)
    out["rope_x"] = v.copy()
    t = torch.from_numpy(v.copy())
    bp.rope_inplace(t, 4, 128, 37, 500000.0)
    out["rope_y"] = t.numpy()
    nh, nkv, hd, mx, sl = 4, 2, 64, 32, 19
    Q = r.standard_normal(nh * hd).astype(np.float16)
    K = np.zeros((nkv, mx, hd), np.float16)
    V = np.zeros((nkv, mx, hd), np.float16)
    K[:, :sl] = r.standard_normal((nkv, sl, hd)).astype(np.float16)
    V[:, :sl] = r.standard_normal((nkv, sl, hd)).astype(np.float16)
    out["attn_q"], out["attn_k"], out["attn_v"] = Q, K, V
    out["attn_y"] = bp.attention(torch.from_numpy(Q), torch.from_numpy(K), torch.from_numpy(V), nh, nkv, hd, sl,
                                 1.0 / hd ** 0.5).numpy()
    g = (r.standard_normal(768) * 3).astype(np.float16)
    u = (r.standard_normal(768) * 3).astype(np.float16)
    out["relu_g"], out["relu_u"] = g, u
    out["relu_y"] = bp.relu2_mul(torch.from_numpy(g), torch.from_numpy(u)).numpy()
    W = (r.standard_normal((48, 200)) * 0.1).astype(np.float16)
    hx = r.standard_normal(200).astype(np.float16)
    out["hg_w"], out["hg_x"] = W, hx
    out["hg_y"] = bp.half_gemv(torch.from_numpy(W), torch.from_numpy(hx)).numpy()
    # SparseBitLinear.forward on packed synthetic weights (ctor bypassed: it re-derives masks)
    case = synth.gemv_case(64, 256, seed=11)
    dense = oracle.unpack_to_int8(case["meta"], case["values"], 64, 256)
    lin = object.__new__(bp.SparseBitLinear)
    lin.weight = torch.from_numpy(dense.astype(np.float32))
    lin.gamma, lin.rows, lin.cols = 0.0371, 64, 256
    bx = (r.standard_normal(256) * 2).astype(np.float16)
    out["bl_x"], out["bl_gamma"] = bx, np.float32(0.0371)
    out["bl_y"] = lin.forward(torch.from_numpy(bx)).numpy()
    np.savez_compressed(HERE / "ops_py.npz", **out)

    # ---- 4. baseline_pytorch.InferenceEngine.forward on a tiny random model ---------------
    model = synth.random_model(synth.TINY, seed=5)
    cfg = model["config"]
    m = object.__new__(bp.BitNetModel)
    m.hidden_size, m.num_layers = cfg["hidden_size"], cfg["num_hidden_layers"]
    m.num_heads, m.num_kv_heads, m.head_dim = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    m.intermediate_size, m.vocab_size, m.max_seq = cfg["intermediate_size"], cfg["vocab_size"], cfg["max_position_embeddings"]
    m.rms_norm_eps, m.rope_theta = cfg["rms_norm_eps"], cfg["rope_theta"]
    m.tie_embeddings, m.bos_token_id, m.eos_token_id = True, 1, -1
    m.embed_tokens = torch.from_numpy(model["embed"])
    m.lm_head = m.embed_tokens
    m.final_norm = torch.from_numpy(model["final_norm"])
    names = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
             "mlp.up_proj", "mlp.down_proj"]
    m.layers = []
    for layer in model["layers"]:
        d = {}
        for name, tns in zip(names, layer["linear"]):
            lin = object.__new__(bp.SparseBitLinear)
            lin.weight = torch.from_numpy(oracle.unpack_to_int8(tns["meta"], tns["values"], tns["rows"],
                                                                tns["cols"]).astype(np.float32))
            lin.gamma, lin.rows, lin.cols = float(tns["gamma"]), tns["rows"], tns["cols"]
            d[name] = lin
        d["input_ln"], d["post_attn_ln"] = torch.from_numpy(layer["norm"][0]), torch.from_numpy(layer["norm"][1])
        d["attn_sub_norm"], d["ffn_sub_norm"] = torch.from_numpy(layer["norm"][2]), torch.from_numpy(layer["norm"][3])
        m.layers.append(d)
    eng = bp.InferenceEngine(m)
    prompt = np.random.default_rng(9).integers(0, cfg["vocab_size"], 6)
    logits, tokens = [], []
    for tkn in prompt[:-1]:
        eng.forward(int(tkn))
    tok = int(prompt[-1])
    for _ in range(10):
        lg = eng.forward(tok)
        tok = int(torch.argmax(lg).item())
        logits.append(lg.numpy())
        tokens.append(tok)
    np.savez_compressed(HERE / "engine_py.npz", prompt=prompt.astype(np.int32), tokens=np.array(tokens, np.int32),
                        logits=np.stack(logits), seed=np.int32(5))
    # ---- tokenizer: ids and decoded bytes from the reference's own src/tokenizer.cpp ----------------
    import json
    import tempfile
    sys.path.insert(0, str(ROOT / "tests"))
    import tokenizer_fixture as tf
    with tempfile.TemporaryDirectory() as d:
        path = Path(d) / "tokenizer.json"
        tf.write(path)
        ref = oracle.RefTokenizer(path)
        cases = []
        for text in tf.TEXTS:
            raw = text.encode("utf-8")
            ids = ref.encode(raw)
            cases.append({"text_hex": raw.hex(), "ids": ids, "decoded_hex": ref.decode(ids).hex()})
        (HERE / "tokenizer_golden.json").write_text(json.dumps({"vocab_size": ref.vocab_size, "cases": cases}, indent=0))
    for f in sorted(HERE.glob("*.npz")) + [HERE / "tokenizer_golden.json"]:
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
