"""The C-ABI library loads and exports what include/shainet_attn.h declares.
No compute calls here: these run without a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from shainet_b200 import build, _lib
    build.build()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "shainet_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(shainet_attn_\w+|kv_cache_append_f32|attention_kv_f32|gemm_q8_f32)\s*\(", text)
    return sorted(set(names))


def test_header_symbols_are_exported(lib):
    from shainet_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 26
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_matches_header(lib):
    text = open(os.path.join(ROOT, "include", "shainet_attn.h")).read()
    v = int(re.search(r"#define SHAINET_ATTN_VERSION (\d+)", text).group(1))
    assert lib.shainet_attn_version() == v


def test_library_is_sm100a_only_and_torch_free():
    import subprocess
    from shainet_b200 import _lib
    out = subprocess.run(["ldd", _lib.LIB_PATH], capture_output=True, text=True).stdout
    assert "torch" not in out and "c10" not in out
    assert "liboracle" not in out


def test_null_arguments_are_rejected_without_a_device(lib):
    from shainet_b200 import _lib
    assert lib.shainet_attn_ctx_create(None, 0) == _lib.E_INVALID
    assert b"null" in lib.shainet_attn_last_error()
    assert lib.shainet_attn_kv_len(None) == _lib.E_INVALID
    assert lib.shainet_attn_kv_reset(None) == _lib.E_INVALID
    assert lib.shainet_attn_ctx_sync(None) == _lib.E_INVALID
    assert lib.shainet_attn_ctx_destroy(None) == _lib.OK
    assert lib.shainet_attn_kv_destroy(None) == _lib.OK


def test_no_cpu_fallback_without_a_device(lib):
    import shainet_b200 as S
    if S.device_count() > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(S.ShainetAttnError) as e:
        S.AttnContext(0)
    assert "no CUDA device" in str(e.value)


def test_product_does_not_touch_the_oracle():
    """The shipped package must never import, link or execute the CPU oracle."""
    pkg = os.path.join(ROOT, "shainet_b200")
    for base, _, files in os.walk(pkg):
        if os.sep + "build" in base or os.sep + "lib" in base:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cr")):
                text = open(os.path.join(base, f), errors="replace").read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def test_crystal_binding_declares_every_entry_point():
    """The Crystal `lib` block (unexecuted here: no compiler) names every shainet_attn_*
    function the header declares."""
    import re
    hdr = open(os.path.join(ROOT, "include", "shainet_attn.h")).read()
    cr = open(os.path.join(ROOT, "shainet_b200", "crystal", "shainet_attn.cr")).read()
    declared = set(re.findall(r"\b(shainet_attn_[a-z_0-9]+)\s*\(", hdr))
    bound = set(re.findall(r"=\s*(shainet_attn_[a-z_0-9]+)", cr))
    assert declared - bound == set(), sorted(declared - bound)
