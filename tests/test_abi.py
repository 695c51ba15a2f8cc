"""CPU tests (no GPU): the shared library loads, exports every symbol the headers declare,
and refuses to compute without a device instead of falling back to anything."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"LK_API[^;(]*?\b(lkx?_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from loki_b200 import _lib
    names = _declared("lokiscan.h") + _declared("lokiscan_index.h")
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(_lib.lib, n)]
    assert not missing, f"declared but not exported: {missing}"
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    exported = set(re.findall(r" T (lkx?_[a-z0-9_]+)", out))
    assert exported == set(names), f"exported but undeclared: {sorted(exported - set(names))}"


def test_no_cpu_fallback_without_a_device():
    from loki_b200 import _lib
    if _lib.device_count() > 0:
        pytest.skip("a CUDA device is present")
    h = C.c_void_p()
    st = _lib.lib.lk_index_create(8, _lib.LK_F32, 0, 0, C.byref(h))
    assert st == _lib.LK_ECUDA and not h
    assert b"no CPU path" in _lib.lib.lk_last_error()
    with pytest.raises(_lib.LokiError):
        _lib.DeviceIndex(8)
    from loki_b200 import embedindex
    with pytest.raises(_lib.LokiError):
        embedindex.New()
    cnt = C.c_int64(0)
    hs = np.arange(4, dtype=np.uint64)
    out = np.zeros(8, np.uint32)
    assert _lib.lib.lk_hamming_pairs(_lib.ptr(hs), 4, 1, 0, 1, 0, _lib.ptr(out), 4, C.byref(cnt)) == _lib.LK_ECUDA


def test_argument_validation_needs_no_device():
    from loki_b200 import _lib
    h = C.c_void_p()
    assert _lib.lib.lk_index_create(0, _lib.LK_F32, 0, 0, C.byref(h)) == _lib.LK_EDIM
    assert _lib.lib.lk_index_create(8, 9, 0, 0, C.byref(h)) == _lib.LK_EINVAL
    assert _lib.lib.lk_index_create(8, _lib.LK_I8, 1, 0, C.byref(h)) == _lib.LK_EINVAL  # centering needs f32
    assert _lib.lib.lk_version().decode().count(".") == 2


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "loki_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, f


def test_embedvec_codec():
    from loki_b200 import embedvec
    v = np.array([0.5, -0.25, 1.0, 0.0], np.float32)
    assert np.array_equal(embedvec.Decode(embedvec.Encode(v)), v)
    with pytest.raises(ValueError):
        embedvec.Decode(b"\x01\x02\x03")
    rows = embedvec.decode_rows([embedvec.Encode(v), b"\x00" * 8], 4)
    assert np.array_equal(rows[0], v) and np.all(rows[1] == 0)
