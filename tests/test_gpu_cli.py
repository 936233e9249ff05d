"""The C++ side of the directory format and the command line: spb_model_load against the Python loader, and the
spbitnet_infer binary (the reference's src/main.cpp flags and --dump-tokens JSON, src/main.cpp:43-68,315-340)
against the engine driven from Python on the same directory and tokenizer."""
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

import oracle
from spbitnet_b200 import build, model_io, synth
from spbitnet_b200.engine import DeviceModel, InferenceEngine
from spbitnet_b200.tokenizer import LoadedModel, Tokenizer
from tokenizer_fixture import write as write_tokenizer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    root = tmp_path_factory.mktemp("cli") / "model"
    cfg = dict(synth.TINY, bos_token_id=456, eos_token_id=457)
    model = synth.random_model(cfg, seed=77)
    model_io.save_model_dir(model, root)
    data = write_tokenizer(root / "tokenizer.json", n_merges=200)
    assert len(data["model"]["vocab"]) == 456 and cfg["vocab_size"] >= 459
    return root, model


def test_cxx_loader_decodes_like_the_python_loader(model_dir):
    root, model = model_dir
    loaded = LoadedModel(root)
    assert loaded.config["hidden_size"] == synth.TINY["hidden_size"] and loaded.bos_token_id == 456
    a = InferenceEngine.from_loaded(loaded)
    b = InferenceEngine(DeviceModel(model_io.load_model_dir(root)))
    prompt = np.array([456, 17, 300, 5], np.int32)
    ta, tb = a.generate(prompt, 12), b.generate(prompt, 12)
    assert (ta == tb).all()
    assert (a.logits().view(np.uint32) == b.logits().view(np.uint32)).all()
    want, _ = oracle.Engine(model).generate(prompt, 12)
    assert (ta == want).all()


def test_cxx_loader_rejects_a_broken_directory(model_dir, tmp_path):
    import shutil
    root, _ = model_dir
    bad = tmp_path / "bad"
    shutil.copytree(root, bad)
    f = next((bad / "weights").glob("layers.0.self_attn.q_proj.meta"))
    raw = bytearray(f.read_bytes())
    raw[0] = 0xFF  # two bitmaps with four bits each
    f.write_bytes(bytes(raw))
    with pytest.raises(Exception) as err:
        LoadedModel(bad)
    assert "bitmap" in str(err.value)
    f.write_bytes(bytes(raw[:-4]))
    with pytest.raises(Exception):
        LoadedModel(bad)


def test_command_line_dump_tokens(model_dir, tmp_path):
    root, model = model_dir
    assert build.CLI.exists(), "spbitnet_infer was not built"
    out = tmp_path / "tokens.json"
    prompt = "Hello world, it\'s 42"
    # generated pieces of a random model need not be valid UTF-8: read the output as bytes
    res = subprocess.run([str(build.CLI), "--model", str(root), "--prompt", prompt, "--max-tokens", "10", "--dump-tokens", str(out)],
                         capture_output=True, timeout=300)
    stdout = res.stdout.decode("utf-8", "replace")
    assert res.returncode == 0, stdout + res.stderr.decode("utf-8", "replace")
    dump = json.loads(out.read_text())
    tok = Tokenizer(root / "tokenizer.json")
    assert dump["prompt"] == prompt
    assert dump["prompt_ids"] == tok.encode(prompt)
    assert dump["input_ids"] == [456] + dump["prompt_ids"]
    eng = InferenceEngine(DeviceModel(model))
    want = eng.generate(np.array(dump["input_ids"], np.int32), 10, eos_token_id=457)
    assert dump["generated_ids"] == [int(t) for t in want]
    assert "--- Generation ---" in stdout and f"{len(want)} tokens generated" in stdout
    # --benchmark runs and reports a rate
    res = subprocess.run([str(build.CLI), "--model", str(root), "--benchmark", "16", "--max-tokens", "1"], capture_output=True,
                         timeout=300)
    assert res.returncode == 0 and b"tok/s" in res.stdout
