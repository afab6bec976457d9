"""CPU: the C-ABI shared library loads and exports every symbol that
include/bt_b200.h declares; host-side argument checking works without a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from bytetransformer_b200 import build, _abi
    build.build_core()
    return _abi.load()


def _declared_functions():
    src = open(os.path.join(ROOT, "include", "bt_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(bt_[a-z_0-9]+)\s*\(", src)))


def test_header_declares_the_expected_surface():
    names = _declared_functions()
    for n in ("bt_create", "bt_destroy", "bt_set_layer_weights", "bt_workspace_bytes", "bt_build_offsets",
              "bt_pack_rows", "bt_gemm", "bt_attention", "bt_add_bias_residual_layernorm",
              "bt_add_bias_residual_layernorm_restore", "bt_layer_forward_padded", "bt_stack_forward_padded",
              "bt_stack_forward_packed", "bt_last_error", "bt_device_status"):
        assert n in names


def test_library_exports_every_declared_symbol(lib):
    from bytetransformer_b200 import _abi
    for n in _declared_functions():
        assert hasattr(lib, n), f"libbt_b200.so does not export {n}"
        assert n in _abi.SIGNATURES, f"ctypes binding lacks a prototype for {n}"


def test_version_string(lib):
    assert b"sm_100a" in lib.bt_version()


def test_argument_checks_without_gpu(lib):
    from bytetransformer_b200 import _abi
    h = C.c_void_p()
    assert lib.bt_create(None, C.byref(h)) == _abi.BT_ERR_INVALID_ARG
    bad = _abi.bt_config(12, 32, 16, 512, 4, 1e-6, 0, 1.0, 0, -1)     # head size 32
    assert lib.bt_create(C.byref(bad), C.byref(h)) == _abi.BT_ERR_UNSUPPORTED
    long_seq = _abi.bt_config(12, 64, 16, 2048, 4, 1e-6, 0, 1.0, 0, -1)
    assert lib.bt_create(C.byref(long_seq), C.byref(h)) == _abi.BT_ERR_INVALID_ARG
    assert lib.bt_build_offsets(None, 1, 1, None, None, None) == _abi.BT_ERR_INVALID_ARG
    assert lib.bt_pack_rows(None, None, None, None, 1, 1, 8, None) == _abi.BT_ERR_INVALID_ARG
    assert lib.bt_add_bias_gelu(None, None, None, 1, 8, 0, None) == _abi.BT_ERR_INVALID_ARG
    assert lib.bt_workspace_bytes(None, 1, 1, None) == _abi.BT_ERR_INVALID_ARG
    assert lib.bt_last_error(None) == b"null handle"


def test_missing_library_fails_loudly(tmp_path):
    from bytetransformer_b200 import _abi
    with pytest.raises(RuntimeError, match="no fallback"):
        _abi.load(str(tmp_path / "libbt_b200.so"))
