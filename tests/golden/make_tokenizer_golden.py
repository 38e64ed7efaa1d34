"""Writes tests/golden/tokenizer.json: ids the REFERENCE's llama_vocabulary::tokenize (llama_cu.cu:1344-1437) produces on a
seeded synthetic vocabulary, through oracle/_ref/libllama_cu_ref.so (ref_tokenize in oracle/ref_shim.cu).  Host-only code:
runs wherever the reference library has been built (no GPU needed).

    python tests/golden/make_tokenizer_golden.py

The vocabulary builder and the texts are imported by tests/test_tokenizer_cpu.py, so fixture and test cannot drift."""
import ctypes as C
import json
import os
import random
import struct
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))

TEXTS = ["abc def ghij", " a b c", "日本 eé xyz", "", "aaaaaaaaaaaaaaaa bbbbbb", "jjihgfedcba abcabcabc", "hi\tthere\n", "  two  spaces",
         "é decomposed", "\U0001f600 four-byte", "abcabcabcabcabcabcabcabc" * 4]


def build_vocab(path, seed=7):
    """extract.py:44-61 layout: int32 count, count x {int32 offset, float score}, zero-terminated pieces.  Ids 0-2 are
    control tokens, 3-258 the byte tokens, the rest seeded pieces over a small alphabet with many score ties."""
    rnd = random.Random(seed)
    base = ["<unk>", "<s>", "</s>"] + [f"<0x{i:02X}>" for i in range(256)]
    letters = "abcdefghij eé日本"
    pieces = set(letters)
    while len(pieces) < 420:
        pieces.add("".join(rnd.choice(letters) for _ in range(rnd.randint(2, 5))))
    pieces = sorted(pieces)
    scores = [0.0] * 259 + [-float(rnd.randint(1, 60)) for _ in pieces]
    enc = [p.encode() for p in base + pieces]
    with open(path, "wb") as f:
        off = 4 + 8 * len(enc)
        f.write(struct.pack("<i", len(enc)))
        for e, s in zip(enc, scores):
            f.write(struct.pack("<if", off, s))
            off += len(e) + 1
        for e in enc:
            f.write(e + b"\0")
    return len(enc)


def reference_ids(vocab_path, text, bos=1):
    lib = C.CDLL(os.path.join(HERE, "..", "..", "oracle", "_ref", "libllama_cu_ref.so"))
    lib.ref_tokenize.restype = C.c_int
    lib.ref_tokenize.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.POINTER(C.c_int16), C.c_int]
    out = (C.c_int16 * 4096)()
    n = lib.ref_tokenize(vocab_path.encode(), text.encode(), bos, out, 4096)
    assert 0 <= n <= 4096
    return [int(x) for x in out[:n]]


if __name__ == "__main__":
    with tempfile.TemporaryDirectory() as d:
        vp = os.path.join(d, "vocab")
        n = build_vocab(vp)
        gold = {"vocab_entries": n, "cases": [{"text": t, "bos": b, "ids": reference_ids(vp, t, b)} for t in TEXTS for b in (1, 0)]}
    json.dump(gold, open(os.path.join(HERE, "tokenizer.json"), "w"))
    print(f"wrote {len(gold['cases'])} cases")
