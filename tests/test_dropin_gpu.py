"""Drop-in proof on a GPU.  ONE client source (oracle/dropin_driver.cu), written against the reference's C++ interface
- llama_params / llama_partition / llama_model::load / llama_context::next_token, tensor4d, generic_tensor and both
overloads of the matmul_nt operator seam (llama_cu.cu:738-747) - is built twice by oracle/Makefile: against the
reference's header + the reference compiled for sm_100a, and against include/llama_cu.h + libllama_cu_b200.so.  Both
binaries run on the same saved weight directory; their matmul outputs and tokens are compared.  The reference's own
quantizer tool (transform.cu, unmodified) is built against the new header and library too and must write the same bytes
as the library's quantizer."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu
REFDIR = os.path.join(ROOT, "oracle", "_ref")
BIN_REF, BIN_NEW, TRANSFORM_NEW = (os.path.join(REFDIR, n) for n in ("dropin_ref", "dropin_new", "transform_new"))
CFG = dict(dim=512, n_heads=4, n_layers=4, n_vocab=2000)


def parse(path):
    out = {"matmul": {}}
    for line in open(path):
        f = line.split()
        if f[0] == "matmul":
            out["matmul"][f[1]] = np.array(f[4:], np.uint16).reshape(int(f[2]), int(f[3])).view(np.float16).astype(np.float32)
        elif f[0] == "tokens":
            out["tokens"] = [int(t) for t in f[1:]]
        else:
            out[f[0]] = int(f[1])
    return out


def run(binary, *args):
    r = subprocess.run([binary, *args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (binary, r.stdout[-1000:], r.stderr[-2000:])
    return r.stdout


@pytest.mark.skipif(not (os.path.exists(BIN_REF) and os.path.exists(BIN_NEW)), reason="drop-in binaries not built (oracle/Makefile)")
@pytest.mark.parametrize("bs", [0, 128])
def test_one_client_source_against_reference_and_new_library(lcu, tmp_path, bs):
    model = lcu.Model.synthetic(block_size=bs, seed=1234, scale=0.06, **CFG)
    d = str(tmp_path / "model")
    model.save(d)
    model.close()
    rep_ref, rep_new, rep_forced = (str(tmp_path / n) for n in ("ref.txt", "new.txt", "new_forced.txt"))
    run(BIN_REF, "run", d, rep_ref)
    ref = parse(rep_ref)
    assert "Device name" in run(BIN_NEW, "run", d, rep_new)  # initialize() prints the device properties like the reference's
    new = parse(rep_new)
    # teacher-forced on the reference's tokens: what the reference produced at step i is fed at step i
    forced_file = str(tmp_path / "forced.txt")
    open(forced_file, "w").write(" ".join(str(t) for t in ref["tokens"][:-1]))
    run(BIN_NEW, "run", d, rep_forced, forced_file)
    forced = parse(rep_forced)
    # the operator seam: same inputs, outputs within the matmul tolerance (2e-3 of the largest output)
    assert sorted(ref["matmul"]) == sorted(new["matmul"]) and len(ref["matmul"]) == 8
    for name, want in ref["matmul"].items():
        got = new["matmul"][name]
        scale = max(1.0, float(np.abs(want).max()))
        assert np.abs(got - want).max() <= 2e-3 * scale, name
    # the forward pass: the prompt's token equals, teacher-forced top-1 agreement is high, bookkeeping is the reference's
    agree = np.mean(np.array(forced["tokens"]) == np.array(ref["tokens"]))
    print(f"drop-in bs={bs}: free-run tokens equal for {int(np.argmax(np.array(new['tokens']) != np.array(ref['tokens']))) if new['tokens'] != ref['tokens'] else len(ref['tokens'])}"
          f" of {len(ref['tokens'])} steps, teacher-forced agreement {agree:.3f}")
    assert agree >= 0.9, (forced["tokens"], ref["tokens"])
    assert new["tokens_left"] == ref["tokens_left"] == 128 - 16 - 24
    assert new["tokens_left_after_clear"] == ref["tokens_left_after_clear"] == 128
    assert new["context_bytes"] > 0


@pytest.mark.skipif(not os.path.exists(TRANSFORM_NEW), reason="transform_new not built (oracle/Makefile)")
def test_reference_quantizer_tool_on_the_new_library(lcu, tmp_path):
    """`transform quantize <in> <out> 128` - the reference's tool, its own kernels and tensor4d / gpu_buffer / mapped_buffer
    use - linked against the new library: every file it writes must equal what lcu_quantize_model_dir writes."""
    models = tmp_path / "models"
    models.mkdir()
    fp = lcu.Model.synthetic(block_size=0, seed=5, scale=0.08, dim=256, n_heads=2, n_layers=2, n_vocab=1000)
    fp.save(str(models / "in"))
    fp.close()
    (models / "tool").mkdir()
    r = subprocess.run([TRANSFORM_NEW, "quantize", "in", "tool", "128"], cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lcu.check(lcu.lib.lcu_quantize_model_dir(str(models / "in").encode(), str(models / "lib").encode(), 128))
    names = sorted(os.listdir(models / "lib"))
    assert names == sorted(os.listdir(models / "tool")) and len(names) == 38  # params, 2 x (weight + scale), norm, 2 layers x (2 norms + 7 x (weight + scale))
    for n in names:
        assert open(models / "lib" / n, "rb").read() == open(models / "tool" / n, "rb").read(), n
