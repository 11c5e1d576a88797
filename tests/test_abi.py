"""CPU tests of the drop-in boundary: the C-ABI library builds for sm_100a, loads, and exports
exactly the symbols include/tie_cuda.h declares.  No compute call is made here."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


@pytest.fixture(scope="module")
def lib():
    from tie_b200 import build, moe
    build.build_cuda()
    return moe.load_library()


def _declared():
    src = open(os.path.join(ROOT, "include", "tie_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tie_cuda_[a-z0-9_]+)\s*\(", src)))


def test_header_and_python_binding_agree():
    from tie_b200 import moe
    assert _declared() == sorted(moe.EXPORTS)


def test_library_exports_every_declared_symbol(lib):
    for name in _declared():
        assert hasattr(lib, name), name
    out = subprocess.run(["nm", "-D", "--defined-only", os.path.join(ROOT, "tie_b200", "libtie_cuda.so")],
                         capture_output=True, text=True).stdout
    exported = sorted(set(re.findall(r" T (tie_cuda_[a-z0-9_]+)", out)))
    assert exported == _declared()


def test_header_compiles_as_plain_c(tmp_path):
    c = tmp_path / "t.c"
    c.write_text('#include "tie_cuda.h"\nint main(void){ tie_cuda_config c; (void)c; return TIE_CUDA_OK; }\n')
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(c), "-o", str(tmp_path / "t.o")])


def test_strerror_and_version(lib):
    assert lib.tie_cuda_strerror(0) == b"ok"
    for code in range(-7, 0):
        assert lib.tie_cuda_strerror(code) not in (b"", b"unknown error")
    assert lib.tie_cuda_strerror(-99) == b"unknown error"
    assert b"sm_100a" in lib.tie_cuda_version()


def test_default_silu_table_is_host_side_and_matches_the_restatement(lib, ref_silu_table):
    from oracle import port
    from tie_b200 import moe
    t = moe.silu_table_default()
    assert np.array_equal(t.view(np.uint32), port.silu_table().view(np.uint32))
    assert np.abs(t - ref_silu_table).max() <= 2e-6


def test_init_rejects_bad_configs_without_a_gpu(lib):
    from tie_b200 import moe
    h = ctypes.c_void_p()
    bad = moe.Config(0, 2000, 128, 8, 768, 1, 16, 1e-6, None, 0, 1)  # hidden not a multiple of 256
    assert lib.tie_cuda_init(ctypes.byref(h), ctypes.byref(bad)) == moe.EINVAL
    bad = moe.Config(0, 2048, 128, 9, 768, 1, 16, 1e-6, None, 0, 1)  # top_k > 8
    assert lib.tie_cuda_init(ctypes.byref(h), ctypes.byref(bad)) == moe.EINVAL
    bad = moe.Config(0, 2048, 128, 8, 768, 1, 16, 1e-6, None, 3, 2)  # ep_rank >= ep_size
    assert lib.tie_cuda_init(ctypes.byref(h), ctypes.byref(bad)) == moe.EINVAL
    assert lib.tie_cuda_init(None, None) == moe.EINVAL
    import torch
    if not torch.cuda.is_available():
        ok = moe.Config(0, 2048, 128, 8, 768, 1, 16, 1e-6, None, 0, 1)
        assert lib.tie_cuda_init(ctypes.byref(h), ctypes.byref(ok)) == moe.ENODEV  # fails loudly, no CPU path
        assert not h.value


def test_product_never_imports_the_oracle():
    """Nothing under tie_b200/ (the product) or include/ may reference oracle/."""
    for base, _, files in os.walk(os.path.join(ROOT, "tie_b200")):
        if "build" in base.split(os.sep)[-1:]:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".c", ".h")):
                txt = open(os.path.join(base, f)).read()
                assert "oracle" not in txt.replace("moe_oracle", "").lower(), (base, f)


def test_reference_side_glue_compiles_against_the_reference_headers(tmp_path):
    """tie_b200/dropin/tie_cuda_qwen3.c is written against the reference's own structures
    (struct TIEContext, Model, LayerWeights, MemType): where the reference tree is present it must
    compile as plain C with the reference's flags.  (Elsewhere the prebuilt
    oracle/_ref/libtie_ref_dropin.so is what travels.)"""
    import oracle
    ref_dir = oracle.reference_dir()
    if not ref_dir:
        pytest.skip("reference tree not present")
    src = os.path.join(ROOT, "tie_b200", "dropin", "tie_cuda_qwen3.c")
    obj = tmp_path / "glue.o"
    subprocess.check_call(["gcc", "-std=gnu11", "-Wall", "-Werror", "-Wno-pointer-sign", "-funsigned-char", "-c", src,
                           "-I", ref_dir, "-I", os.path.join(ROOT, "include"), "-I", os.path.dirname(src), "-o", str(obj)])
    syms = subprocess.check_output(["nm", "--defined-only", str(obj)], text=True)
    assert "tie_cuda_qwen3_load" in syms and "tie_cuda_qwen3_moe_ffn" in syms
