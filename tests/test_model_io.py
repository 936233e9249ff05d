"""Model directory I/O (the reference's on-disk format, docs/compression_format.md section 4;
fixture modelled on tests/test_model_loader.cu:52-191): what is written is what Model::load reads."""
import json

import numpy as np
import pytest

from spbitnet_b200 import model_io, synth


@pytest.fixture()
def tiny(tmp_path):
    model = synth.random_model(synth.TINY, seed=5)
    return model, model_io.save_model_dir(model, tmp_path / "m", stats=True)


def test_directory_layout_and_manifest(tiny):
    model, root = tiny
    cfg = json.loads((root / "config.json").read_text())
    assert cfg["model_type"] == "bitnet" and cfg["hidden_act"] == "relu2" and cfg["tie_word_embeddings"] is True
    for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "intermediate_size",
                "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta", "head_dim"):
        assert key in cfg
    man = json.loads((root / "manifest.json").read_text())
    assert man["format_version"] == 1
    w = man["weights"]
    assert w["lm_head"] == {"tied_to": "embed_tokens", "dtype": "tied"}
    assert w["embed_tokens"]["dtype"] == "float16" and w["norm"]["dtype"] == "float32"
    # names that src/model.cu:245-303 looks up
    for name in ("layers.0.input_layernorm", "layers.0.post_attention_layernorm", "layers.0.self_attn.attn_sub_norm",
                 "layers.0.mlp.ffn_sub_norm"):
        assert w[name]["dtype"] == "float32" and (root / w[name]["file"]).stat().st_size == w[name]["nbytes"]
    for proj in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
                 "mlp.up_proj", "mlp.down_proj"):
        e = w[f"layers.0.{proj}"]
        rows, cols = e["shape"]
        assert e["dtype"] == "sparse_ternary"
        assert e["meta_stride"] == (cols // 4 + 7) // 8 and e["values_stride"] == (cols // 4 + 15) // 16
        assert e["meta_nbytes"] == rows * e["meta_stride"] * 4 == (root / e["meta_file"]).stat().st_size
        assert e["values_nbytes"] == rows * e["values_stride"] * 4 == (root / e["values_file"]).stat().st_size
        assert e["meta_file"] == f"weights/layers.0.{proj}.meta"  # flat names with dots, no sub-directories


def test_round_trip_is_exact(tiny):
    model, root = tiny
    back = model_io.load_model_dir(root)
    assert back["config"]["num_hidden_layers"] == model["config"]["num_hidden_layers"]
    assert (back["embed"].view(np.uint16) == model["embed"].view(np.uint16)).all()
    assert (back["final_norm"] == model["final_norm"]).all()
    for a, b in zip(back["layers"], model["layers"]):
        for ta, tb in zip(a["linear"], b["linear"]):
            assert (ta["meta"] == tb["meta"]).all() and (ta["values"] == tb["values"]).all()
            assert ta["gamma"] == np.float32(tb["gamma"]) and (ta["rows"], ta["cols"]) == (tb["rows"], tb["cols"])
        for na, nb in zip(a["norm"], b["norm"]):
            assert (na == nb).all()
    assert len(model_io.load_model_dir(root, layers=1)["layers"]) == 1


def test_reference_fixture_pattern_loads(tmp_path):
    # the fixture of tests/test_model_loader.cu: every group is {+1, -1, 0, 0}: bitmap 0b0011, signs 0b10
    cfg = dict(hidden_size=8, num_hidden_layers=1, num_attention_heads=1, num_key_value_heads=1, head_dim=8,
               intermediate_size=16, vocab_size=32, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0)
    layer = {"linear": [], "norm": [np.ones(8, np.float32), np.ones(8, np.float32), None, None]}
    for rows, cols in synth.linear_shapes(cfg):
        g = cols // 4
        meta = np.zeros((rows, (g + 7) // 8), np.uint32)
        values = np.zeros((rows, (g + 15) // 16), np.uint32)
        for k in range(g):
            meta[:, k // 8] |= np.uint32(0x3 << ((k % 8) * 4))
            values[:, k // 16] |= np.uint32(0x2 << ((k % 16) * 2))
        layer["linear"].append(dict(meta=meta, values=values, gamma=0.5, rows=rows, cols=cols,
                                    meta_stride=meta.shape[1], values_stride=values.shape[1]))
    model = {"config": cfg, "layers": [layer], "embed": np.zeros((32, 8), np.float16), "final_norm": np.ones(8, np.float32)}
    root = model_io.save_model_dir(model, tmp_path / "test_model")
    back = model_io.load_model_dir(root)
    assert back["layers"][0]["norm"][2] is None and back["layers"][0]["norm"][3] is None  # sub-norms are optional
    q = back["layers"][0]["linear"][0]
    assert q["meta"][0, 0] == 0x33 and q["values"][0, 0] == 0xA and q["gamma"] == np.float32(0.5)


def test_untied_head(tmp_path):
    model = synth.random_model(synth.TINY, seed=1, layers=1)
    model["lm_head"] = (model["embed"].astype(np.float32) * 2).astype(np.float16)
    root = model_io.save_model_dir(model, tmp_path / "u")
    assert json.loads((root / "config.json").read_text())["tie_word_embeddings"] is False
    back = model_io.load_model_dir(root)
    assert (back["lm_head"].view(np.uint16) == model["lm_head"].view(np.uint16)).all()


def test_rejects_what_the_kernels_cannot_take(tiny):
    model, root = tiny
    man = json.loads((root / "manifest.json").read_text())
    name = "layers.0.self_attn.q_proj"
    f = root / man["weights"][name]["meta_file"]
    raw = np.fromfile(f, np.uint32)
    bad = raw.copy()
    bad[3] = (bad[3] & ~np.uint32(0xF)) | np.uint32(0x7)  # three bits in one bitmap
    bad.tofile(f)
    with pytest.raises(model_io.ModelFormatError, match=name):
        model_io.load_model_dir(root)
    model_io.load_model_dir(root, validate=False)  # the caller may skip the check
    raw[:-1].tofile(f)  # truncated file
    with pytest.raises(model_io.ModelFormatError, match="bytes"):
        model_io.load_model_dir(root)
    raw.tofile(f)
    man["format_version"] = 2
    (root / "manifest.json").write_text(json.dumps(man))
    with pytest.raises(model_io.ModelFormatError, match="format_version"):
        model_io.load_model_dir(root)
