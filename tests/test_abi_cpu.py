"""The C-ABI library loads without a GPU, exports every declared symbol, and refuses to compute
without a device (no silent CPU path).  Host-side model/partition logic is checked as well."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import ROOT, load_package


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "llama_cu_c.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lcu_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lcu = load_package()
    names = declared_symbols()
    assert len(names) >= 45
    for n in names:
        assert hasattr(lcu.lib, n), f"{n} declared in include/llama_cu_c.h but not exported"
    assert set(lcu.EXPORTS) == set(names), set(lcu.EXPORTS) ^ set(names)


def test_no_cpu_fallback_without_a_device():
    lcu = load_package()
    if lcu.lib.lcu_device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(lcu.LcuError, match="no CUDA device"):
        lcu.quantize(np.zeros((2, 128), np.uint16), 128)
    with pytest.raises(lcu.LcuError, match="no CUDA device"):
        lcu.matmul_nt(np.zeros((1, 256), np.uint16), np.zeros((2, 256), np.uint16))
    with pytest.raises(lcu.LcuError, match="no CUDA device"):
        lcu.Model.synthetic(256, 2, 1, 1000)


def test_host_side_shapes_and_partitions():
    lcu = load_package()
    assert lcu.lib.lcu_ffn_dim(4096, 256) == 11008
    assert lcu.lib.lcu_ffn_dim(5120, 256) == 13824
    assert lcu.lib.lcu_ffn_dim(8192, 256) == 22016
    lg = np.zeros(80, np.int32)
    assert lcu.lib.lcu_partition_even(80, 8, lg.ctypes.data_as(C.c_void_p)) == 0
    assert (np.bincount(lg) == 10).all() and (np.diff(lg) >= 0).all()
    assert lcu.lib.lcu_partition_even(40, 2, lg.ctypes.data_as(C.c_void_p)) == 0
    assert lg[:40].tolist() == [0] * 20 + [1] * 20
    assert lcu.lib.lcu_partition_even(2, 4, lg.ctypes.data_as(C.c_void_p)) != 0
    assert b"partition" in lcu.lib.lcu_last_error()
    assert len(lcu.pack_params(4096, 256, 32, 32, 32000)) == 40
    assert lcu.lib.lcu_set_matmul_type(3) != 0 and lcu.lib.lcu_set_matmul_type(4) == 0


def test_oracle_is_not_linked_into_the_product():
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(ROOT, "llama.cu_b200", "libllama_cu_b200.so")],
                         capture_output=True, text=True).stdout
    assert "orc_" not in out and "ref_" not in out
    for root, _, files in os.walk(os.path.join(ROOT, "llama.cu_b200")):
        for f in files:
            if f.endswith((".cu", ".cuh", ".py", ".h")):
                src = open(os.path.join(root, f)).read()
                assert "oracle" not in src.lower().replace("oracle/liboracle", "") or f == "__init__.py" and "oracle" not in src, f


@pytest.mark.skipif(not os.path.exists("/root/reference/main.cpp"), reason="reference sources not present")
def test_reference_main_compiles_against_the_new_header(tmp_path):
    """Drop-in proof at the source level: the reference's own client builds against include/llama_cu.h."""
    exe = tmp_path / "llama_cu_main"
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    r = subprocess.run([cxx, "-std=c++17", "-I", os.path.join(ROOT, "include"), "/root/reference/main.cpp", "-o", str(exe),
                        "-L", os.path.join(ROOT, "llama.cu_b200"), "-lllama_cu_b200",
                        "-Wl,-rpath," + os.path.join(ROOT, "llama.cu_b200")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
