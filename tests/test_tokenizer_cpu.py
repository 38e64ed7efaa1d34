"""llama_vocabulary::tokenize of the new library (lcu_tokenize in the C ABI; the C++ class of include/llama_cu.h) against
the ids the reference's tokenizer produced on the same seeded vocabulary (tests/golden/tokenizer.json, written by
tests/golden/make_tokenizer_golden.py through the reference itself), and live against the reference where its library
or the drop-in binaries are present.  Host-only code: no GPU involved."""
import ctypes as C
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, load_package

sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
import make_tokenizer_golden as G  # noqa: E402

GOLD = json.load(open(os.path.join(ROOT, "tests", "golden", "tokenizer.json")))


def mine(lcu, vocab, text, bos):
    out = np.zeros(4096, np.int16)
    n = lcu.lib.lcu_tokenize(vocab.encode(), text.encode(), bos, out.ctypes.data_as(C.c_void_p), out.size)
    assert 0 <= n <= out.size
    return out[:n].tolist()


def test_tokenizer_matches_reference_golden(tmp_path):
    lcu = load_package()
    vocab = str(tmp_path / "vocab")
    assert G.build_vocab(vocab) == GOLD["vocab_entries"]
    for case in GOLD["cases"]:
        assert mine(lcu, vocab, case["text"], case["bos"]) == case["ids"], case["text"]
    # capacity smaller than the result: the count comes back, only `capacity` ids are written
    out = np.full(4, -1, np.int16)
    n = lcu.lib.lcu_tokenize(vocab.encode(), b"abc def ghij", 1, out.ctypes.data_as(C.c_void_p), 3)
    assert n > 3 and out[3] == -1 and out[0] == 1
    assert lcu.lib.lcu_tokenize(b"/nonexistent/vocab", b"x", 1, out.ctypes.data_as(C.c_void_p), 4) == -1
    assert b"vocabulary" in lcu.lib.lcu_last_error()


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libllama_cu_ref.so")), reason="reference library not built")
def test_tokenizer_matches_reference_live(tmp_path):
    lcu = load_package()
    vocab = str(tmp_path / "vocab")
    G.build_vocab(vocab, seed=11)  # another vocabulary than the fixture's
    rng = np.random.default_rng(3)
    alphabet = list("abcdefghij eé日本z ")
    for _ in range(40):
        text = "".join(rng.choice(alphabet, size=int(rng.integers(0, 60))))
        assert mine(lcu, vocab, text, 1) == G.reference_ids(vocab, text, 1), text
    # the same through the C++ classes: one client source built against each header
    ref_bin, new_bin = (os.path.join(ROOT, "oracle", "_ref", n) for n in ("dropin_ref", "dropin_new"))
    if os.path.exists(ref_bin) and os.path.exists(new_bin):
        for text in G.TEXTS:
            a = subprocess.run([ref_bin, "tokenize", vocab, text], capture_output=True, text=True)
            b = subprocess.run([new_bin, "tokenize", vocab, text], capture_output=True, text=True)
            assert a.returncode == 0 and b.returncode == 0 and a.stdout == b.stdout, text
