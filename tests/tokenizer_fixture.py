"""A small synthetic tokenizer.json for the tokenizer tests: the 256 byte tokens of GPT-2's stand-in alphabet, a
few hundred merges learnt greedily from a fixed text, and added special tokens -- the schema of a HuggingFace
byte-level BPE file (what the reference's tests/test_tokenizer.cpp:12-100 builds by hand, larger)."""
import json
from collections import Counter

CORPUS = (
    "The quick brown fox jumps over the lazy dog. It's the dog's day, isn't it? We're here; they've gone, I'll stay. "
    "Numbers: 1 22 333 4444 55555 3.14159 2024-11-25 10:30.\n\nNew paragraph\twith tabs   and   spaces.\r\nWindows line. "
    "Sparse ternary weights keep two of four values; the other two are zero. hello hello world world world!!! ??? ... "
    "def f(x): return x*x + 1  # comment\n    indent_level = 4\n"
) * 3


def bytes_to_unicode():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


def build(n_merges: int = 300) -> dict:
    enc = bytes_to_unicode()
    words = Counter()
    for w in CORPUS.replace("\n", " \n ").split(" "):
        if w:
            words[tuple(enc[b] for b in (" " + w).encode("utf-8"))] += 1
    vocab = {enc[b]: i for i, b in enumerate(range(256))}
    merges = []
    for _ in range(n_merges):
        pairs = Counter()
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += c
        if not pairs:
            break
        best = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))[0]
        merges.append(f"{best[0]} {best[1]}")
        if best[0] + best[1] not in vocab:
            vocab[best[0] + best[1]] = len(vocab)
        new_words = Counter()
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and (w[i], w[i + 1]) == best:
                    out.append(w[i] + w[i + 1])
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            new_words[tuple(out)] += c
        words = new_words
    n = len(vocab)
    added = [{"id": n, "content": "<|begin_of_text|>", "special": True},
             {"id": n + 1, "content": "<|end_of_text|>", "special": True},
             {"id": n + 2, "content": "<|plain added|>", "special": False}]
    return {"version": "1.0", "added_tokens": added,
            "model": {"type": "BPE", "vocab": vocab, "merges": merges}}


def write(path, n_merges: int = 300):
    data = build(n_merges)
    with open(path, "w", encoding="utf-8") as f:
        json.dump(data, f, ensure_ascii=True)  # exercises the \\uXXXX escapes of the readers
    return data


TEXTS = [
    "Hello", " Hello", "Hello world", "The quick brown fox", "It's we're THEY'VE i'll don't 'd 'M 'x ''s",
    "1 22 333 4444 55555 1234567", "3.14159, 2024-11-25", "a  b   c    d", "  leading and trailing  ", "tabs\tand\nnewlines\r\n\r\nmixed \n \n",
    "!!! ??? ... ;;; :-) (x) [y] {z} <|begin_of_text|>", "café naïve über", "你好，世界", "emoji \U0001F600 done",
    "", " ", "\n", "   ", "x", "'", "''", "a'", "'re", "'r", "9", "99'99", "word1word22word333", "snake_case_name = 42",
    "def f(x): return x*x + 1  # comment\n    indent_level = 4\n", "trailing space ", "trailing spaces   ", "\t\tdouble tab start",
    "A B non-breaking", "mixed separator", "end with newline\n", "\r\n\r\n", "a\r\nb", " '", "' s", "hello hello world world world!!!",
]
