"""CPU-side checks of the C ABI: the library loads, exports every declared symbol, and the
argument validation (which runs before any CUDA call) returns the reference's messages."""
import ctypes as C

import pytest

from kaio_b200 import _lib


@pytest.fixture(scope="module")
def lib():
    from kaio_b200 import build
    build.build()
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    names = _lib.declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), name
    for name in _lib.SIGNATURES:
        assert name in names


def test_version(lib):
    assert lib.kaio_b200_version() == 1001


def err(lib):
    return lib.kaio_b200_last_error().decode()


def test_matmul_tc_validation_messages(lib):
    """validate_dims_tc, kaio-ops/src/matmul_tc_kernel.rs:123-164."""
    for f in (lib.kaio_b200_matmul_tc, lib.kaio_b200_matmul_tc_async):
        assert f(None, 0, None, 0, None, 0, 0, 8, 16, None) == 1
        assert err(lib) == "matmul_tc dimensions must be non-zero"
        assert f(None, 0, None, 0, None, 0, 16, 8, 24, None) == 1
        assert err(lib).startswith("matmul_tc: K must be a multiple of 16 (got 24).")
        assert f(None, 5, None, 0, None, 0, 16, 8, 16, None) == 1
        assert err(lib) == "matmul_tc: A buffer too small: need 256 f16 (16×16), got 5"
        assert f(None, 256, None, 7, None, 0, 16, 8, 16, None) == 1
        assert err(lib) == "matmul_tc: B buffer too small: need 128 f16 (16×8), got 7"
        assert f(None, 256, None, 128, None, 3, 16, 8, 16, None) == 1
        assert err(lib) == "matmul_tc: C buffer too small: need 128 f32 (16×8), got 3"


def test_int8_validation_messages(lib):
    assert lib.kaio_b200_matmul_int8(None, 0, None, 0, None, 0, 1.0, 16, 8, 31, None) == 1
    assert "K must be a multiple of 32 (got 31)" in err(lib)
    assert lib.kaio_b200_matmul_int8(None, 0, None, 0, None, 0, 1.0, 0, 8, 32, None) == 1
    assert err(lib) == "matmul_int8 dimensions must be non-zero"
    assert lib.kaio_b200_matmul_int8(None, 5, None, 0, None, 0, 1.0, 16, 8, 32, None) == 1
    assert err(lib) == "matmul_int8: A buffer too small: need 512 i8 (16×32), got 5"


def test_int4_validation_messages(lib):
    f = lib.kaio_b200_matmul_int4
    assert f(None, 0, None, 0, None, 0, None, 0, 16, 8, 127, 128, None) == 1
    assert "K must be a multiple of group_size=128 (got 127)" in err(lib)
    assert f(None, 0, None, 0, None, 0, None, 0, 16, 8, 128, 64, None) == 1
    assert "group_size must be 128 (got 64)" in err(lib)
    assert f(None, 0, None, 0, None, 0, None, 0, 0, 8, 128, 128, None) == 1
    assert "dimensions must be non-zero" in err(lib)
    assert f(None, 16 * 128, None, 3, None, 0, None, 0, 16, 8, 128, 128, None) == 1
    assert "B packed buffer too small: need 128 u32 (8 cols × 16 K-words), got 3" in err(lib)


def test_qkv_validation_messages(lib):
    f8 = lib.kaio_b200_qkv_project_int8
    args = [None, 0] * 4 + [1.0, 1.0, 1.0] + [None, 0] * 3
    assert f8(*args, 64, 16, 24, None) == 1
    assert "K must be a multiple of K_TILE_SHARED=16 (got 24)" in err(lib)
    assert f8(*args, 64, 15, 16, None) == 1
    assert "N must be even (got 15)" in err(lib)
    f4 = lib.kaio_b200_qkv_project_int4
    args4 = [None, 0] * 10
    assert f4(*args4, 64, 16, 128, 64, None) == 1
    assert "group_size must be 128" in err(lib)
    assert f4(*args4, 64, 16, 192, 128, None) == 1
    assert "K must be a multiple of group_size=128" in err(lib)


def test_attention_validation_messages(lib):
    f = lib.kaio_b200_attention_tc
    base = [None, 0] * 4
    assert f(*base, 17, 16, 16, 8, 0, None) == 1
    assert "seq_q must be a multiple of 16 (got 17)" in err(lib)
    assert f(*base, 16, 400, 16, 8, 0, None) == 1
    assert "seq_k must be ≤ 384 (got 400)" in err(lib)
    assert f(*base, 16, 16, 16, 12, 0, None) == 1
    assert "d_v must be a multiple of 8" in err(lib)
    assert f(*base, 16, 16, 16, 8, 0, None) == 1
    assert "Q buffer too small: need 256 f16 (16×16), got 0" in err(lib)


def test_no_cpu_fallback_without_gpu(lib):
    """With valid arguments but no CUDA device the call must fail, not compute on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    a = (C.c_int8 * (16 * 32))()
    b = (C.c_int8 * (32 * 16))()
    c = (C.c_float * (16 * 16))()
    rc = lib.kaio_b200_matmul_int8(a, 16 * 32, b, 32 * 16, c, 16 * 16, 1.0, 16, 16, 32, None)
    assert rc in (2, 3), err(lib)
    assert all(v == 0.0 for v in c)


def test_cpp_mirror_header_compiles_and_reports_reference_errors(lib, tmp_path):
    """include/kaio_ops.hpp (C++ mirror of the kaio-ops signatures) compiles against the header,
    links against the library and surfaces validation errors as KaioError with the reference text."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "t.cpp"
    src.write_text(r'''
#include <cstdio>
#include <cstring>
#include "kaio_ops.hpp"
int main() {
    kaio_ops::KaioDevice dev(0);
    kaio_ops::GpuBuffer<const int8_t> a(nullptr, 0), b(nullptr, 0);
    kaio_ops::GpuBuffer<float> c(nullptr, 0);
    try { kaio_ops::matmul_int8(dev, a, b, c, 1.0f, 16, 8, 31); }
    catch (const kaio_ops::KaioError& e) {
        if (e.is_invalid_config() && std::strstr(e.what(), "K must be a multiple of 32")) { std::puts("ok"); return 0; }
    }
    return 1;
}
''')
    exe = tmp_path / "t"
    libdir = os.path.join(root, "kaio_b200", "lib")
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(root, "include"), str(src), "-o", str(exe),
                    "-L", libdir, "-lkaio_b200", f"-Wl,-rpath,{libdir}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok"
