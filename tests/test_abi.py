"""The C-ABI shared library loads on a machine without a GPU and exports every symbol that
include/winograd2x2_b200.h declares; argument validation answers before any CUDA call."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "winograd2x2_b200.h")
LIB = os.path.join(ROOT, "sparse-winograd-cnn_b200", "libwinograd2x2_b200.so")


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        import importlib.util
        spec = importlib.util.spec_from_file_location("wg_build", os.path.join(ROOT, "sparse-winograd-cnn_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return ctypes.CDLL(LIB)


def _declared():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r"\b(wg2x2_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), n


def test_python_binding_covers_header():
    import wg2x2._lib as b
    assert sorted(b.EXPORTS) == [n for n in _declared()]


def test_reference_launcher_symbols(lib):
    out = subprocess.check_output(["nm", "-D", "--defined-only", LIB], text=True)
    for mangled in ("_Z33Winograd2x2ImTransComputeLauncherPKfPfiiiiii",
                    "_Z37Winograd2x2ImTransGradComputeLauncherPKfPfiiiiii",
                    "_Z30Winograd2x2ConvComputeLauncherPKfS0_PfS1_PKxiiiiiii",
                    "_Z34Winograd2x2ConvGradComputeLauncherPKfS0_S0_PfS1_S1_Pxiiiiiii"):
        assert mangled in out


def test_argument_validation_without_gpu(lib):
    lib.wg2x2_status_string.restype = ctypes.c_char_p
    assert lib.wg2x2_abi_version() >= 1
    assert lib.wg2x2_imtrans_fwd(None, None, 1, 4, 4, 4, 0, 0, None) == -1
    assert lib.wg2x2_imtrans_bwd(None, None, None, 1, 4, 4, 4, 0, None) == -1
    one = ctypes.c_void_p(256)
    assert lib.wg2x2_imtrans_fwd(one, one, 0, 4, 4, 4, 0, 0, None) == -1      # B = 0
    assert lib.wg2x2_imtrans_fwd(one, one, 1, 4, 4, 4, 7, 0, None) == -1      # unknown layout
    f = lib.wg2x2_conv_fwd
    f.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 9 + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    assert f(None, one, one, 1, 2, 2, 4, 4, 4, 4, 0, 0, None, 0, None) == -1
    assert f(one, one, one, 1, 2, 2, 4, 4, 5, 4, 0, 0, None, 0, None) == -1   # out_h not in {2nH-1, 2nH}
    assert f(one, one, one, 1, 2, 2, 4, 4, 4, 4, 0, 9, None, 0, None) == -1   # unknown math mode
    assert b"workspace" in lib.wg2x2_status_string(-2)


def test_misaligned_operands_are_refused_before_any_launch(lib):
    """The tensor-core backward pass and the wide forward path use TMA and 16-byte accesses on every operand:
    a pointer off a 16-byte boundary must come back as BAD_ARG, not reach a kernel.  The pointers here are
    fake; the checks run before the first CUDA call, so this needs no GPU."""
    P = ctypes.c_void_p
    ok, off = P(4096), P(4096 + 4)
    bwd = lib.wg2x2_conv_bwd
    bwd.argtypes = [P] * 6 + [ctypes.c_int] * 8 + [P, ctypes.c_size_t, P]
    B, H, W, C, K = 2, 8, 8, 64, 64
    ws = P(1 << 20)
    for bad in range(6):   # V, Wt, dY, mask, dV, dW in turn
        ptrs = [off if i == bad else ok for i in range(6)]
        assert bwd(*ptrs, B, H, W, C, K, 0, 1, 1, ws, 1 << 40, None) == -1, bad
    fwd = lib.wg2x2_conv_fwd_prepared_ws
    fwd.argtypes = [P] * 3 + [ctypes.c_int] * 8 + [P] * 3 + [P, ctypes.c_size_t, P]
    C = K = 256
    for bad in range(6):   # V, prepared, Y, out_scale, out_shift, residual
        ptrs = [off if i == bad else ok for i in range(6)]
        assert fwd(ptrs[0], ptrs[1], ptrs[2], B, 4, 4, C, K, 8, 8, 0, ptrs[3], ptrs[4], ptrs[5], ws, 1 << 40, None) == -1, bad
    # the stem kernel copies the image in 16-byte pieces; sizes it does not take are UNSUPPORTED (-5), not a launch
    stem = lib.wg2x2_stem7x7s2_pool
    stem.argtypes = [P] * 6 + [ctypes.c_int] * 3 + [P]
    assert stem(off, ok, ok, None, None, None, 2, 224, 224, None) == -1
    assert stem(ok, off, ok, None, None, None, 2, 224, 224, None) == -1
    assert stem(ok, ok, ok, None, ok, ok, 2, 224, 224, None) == -1          # an affine ReLU output without its tensor
    for h, w in ((226, 224), (224, 222), (224, 228), (2, 224)):
        assert stem(ok, ok, ok, None, None, None, 2, h, w, None) == -5, (h, w)
    assert lib.wg2x2_stem_prepared_floats() == 21 * 32 * 16


def test_wait_limit_argument(lib):
    f = lib.wg2x2_set_wait_limit
    f.argtypes = [ctypes.c_longlong]
    assert f(-5) == -1
    assert f(1000) == 0
    assert f(0) == 0          # back to the default
    assert lib.wg2x2_test_drop_load(-1) == 0


def test_workspace_queries(lib):
    q = lib.wg2x2_conv_bwd_workspace_bytes
    q.restype = ctypes.c_size_t
    assert q(256, 7, 7, 512, 512, 0, 0) == 0
    n = q(256, 7, 7, 512, 512, 0, 1)
    assert n % (16 * 512 * 512 * 4) == 0 and n > 0          # whole copies of dW
    q2 = lib.wg2x2_layer_fwd_workspace_bytes
    q2.restype = ctypes.c_size_t
    assert q2(4, 56, 56, 64, 64, 0, 0) >= 16 * 4 * 28 * 28 * 64 * 4   # holds V when the caller keeps none
    assert q2(4, 56, 56, 64, 64, 0, 1) == 0


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    """The Python binding has no fallback: without the shared library the import raises."""
    import importlib.util
    src = os.path.join(ROOT, "sparse-winograd-cnn_b200", "wg2x2", "_lib.py")
    pkg = tmp_path / "elsewhere" / "wg2x2"
    pkg.mkdir(parents=True)
    (pkg / "_lib.py").write_text(open(src).read())
    spec = importlib.util.spec_from_file_location("wg2x2_lib_copy", str(pkg / "_lib.py"))
    mod = importlib.util.module_from_spec(spec)
    with pytest.raises(ImportError, match="no fallback"):
        spec.loader.exec_module(mod)
