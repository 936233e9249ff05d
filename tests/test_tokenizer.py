"""The tokenizer (spb_tokenizer_*) against the reference's own spbitnet::Tokenizer compiled from src/tokenizer.cpp
(when oracle/_ref is built) and against golden ids generated from it (tests/golden/tokenizer_golden.json, always):
encode must give the same ids, decode the same bytes, on a synthetic byte-level BPE file.  Also the behaviours the
reference's tests/test_tokenizer.cpp:123-180 checks: vocabulary size, round trip, special tokens skipped on
decode, bytes outside the merges fall back to byte tokens.  Host only."""
import json
import random

import numpy as np
import pytest

import oracle
from spbitnet_b200.tokenizer import Tokenizer
from conftest import GOLDEN
from tokenizer_fixture import TEXTS, write


@pytest.fixture(scope="module")
def tok_path(tmp_path_factory):
    p = tmp_path_factory.mktemp("tok") / "tokenizer.json"
    write(p)
    return p


def _random_texts(n=300, seed=5):
    rng = random.Random(seed)
    alphabet = list("abcdefghijklmnopqrstuvwxyzABCDEFG 0123456789   \n\t\r'.,!?-_(){}[]<>|:;\"") + ["'s", "'re", " the", "é", "世", "\U0001F600", "\n\n"]
    out = []
    for _ in range(n):
        out.append("".join(rng.choice(alphabet) for _ in range(rng.randint(0, 60))))
    for _ in range(50):  # arbitrary bytes, not necessarily valid UTF-8
        out.append(bytes(rng.randrange(256) for _ in range(rng.randint(1, 40))))
    return out


def test_matches_the_golden_ids(tok_path):
    gold = json.loads((GOLDEN / "tokenizer_golden.json").read_text())
    tok = Tokenizer(tok_path)
    assert tok.vocab_size == gold["vocab_size"]
    for case in gold["cases"]:
        raw = bytes.fromhex(case["text_hex"])
        ids = tok.encode(raw)
        assert ids == case["ids"], raw
        assert tok.decode_bytes(ids).hex() == case["decoded_hex"], raw


@pytest.mark.skipif(not oracle.RefTokenizer.available(), reason="oracle/_ref/libspb_reftok.so not built")
def test_matches_the_reference_tokenizer_live(tok_path):
    tok, ref = Tokenizer(tok_path), oracle.RefTokenizer(tok_path)
    assert tok.vocab_size == ref.vocab_size
    for text in TEXTS + _random_texts():
        raw = text.encode("utf-8") if isinstance(text, str) else text
        ids = tok.encode(raw)
        assert ids == ref.encode(raw), raw
        assert tok.decode_bytes(ids) == ref.decode(ids), raw
    rng = np.random.default_rng(0)
    for _ in range(50):  # decode of arbitrary id sequences, specials and out-of-range ids included
        ids = rng.integers(-3, tok.vocab_size + 3, rng.integers(0, 30)).astype(np.int32)
        assert tok.decode_bytes(ids) == ref.decode(ids)


def test_behaviours_the_reference_tests_pin(tok_path):
    data = json.loads(tok_path.read_text())
    tok = Tokenizer(tok_path)
    n_vocab = len(data["model"]["vocab"])
    assert tok.vocab_size == n_vocab + 3
    bos = n_vocab
    for text in ("Hello world", "The quick brown fox", "hello hello world"):
        ids = tok.encode(text)
        assert ids and all(0 <= i < n_vocab for i in ids)
        assert tok.decode(ids) == text                      # round trip
        assert tok.decode([bos] + ids + [bos + 1]) == text  # special tokens are skipped
    assert tok.decode_token(bos) == ""
    # a frequent word is fewer tokens than its bytes; bytes the merges never saw fall back to one token per byte
    assert len(tok.encode(" world")) < len(" world")
    rare = "你"
    assert len(tok.encode(rare)) == len(rare.encode("utf-8"))
    assert tok.encode("") == [] and tok.decode([]) == ""
    with pytest.raises(Exception):
        Tokenizer(tok_path.parent / "missing.json")
