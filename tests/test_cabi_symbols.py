"""The C-ABI library must build, load and export every symbol include/kf_b200.h declares (no compute calls here)."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def built_lib():
    from lightly_trian_quant_b200 import build

    return build.build()


def test_exports_every_declared_symbol(built_lib):
    from lightly_trian_quant_b200 import _lib

    names = _lib.declared_symbols()
    assert "kf_quant_rows" in names and "kf_ln_quant" in names
    L = ctypes.CDLL(str(built_lib))
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_host_side_argument_checks(built_lib):
    """bad arguments are rejected on the host with a message, before any launch."""
    from lightly_trian_quant_b200 import _lib

    L = _lib.lib()
    assert L.kf_version().decode().endswith("sm_100a")
    assert L.kf_sf_bytes(1605, 1024, 0) == 13 * 8 * 512
    assert L.kf_sf_bytes(1605, 1024, 1) == 13 * 16 * 512
    assert L.kf_sf_bytes(130, 768, 2) == 2 * 6 * 512
    assert L.kf_sf_bytes(-1, 1024, 0) < 0
    st = L.kf_quant_rows(0, 0, None, 1024, 16, 1000, None, None, 0, None, None, None)
    assert st == -1 and "multiple of 128" in L.kf_last_error_string().decode()
    st = L.kf_quant_rows(7, 0, None, 1024, 16, 1024, None, None, 0, None, None, None)
    assert st == -1 and "format" in L.kf_last_error_string().decode()
    st = L.kf_quant_rows(0, 0, None, 1024, 16, 1024, None, None, 0, None, None, None)
    assert st == -1 and "null" in L.kf_last_error_string().decode()
    st = L.kf_ln_quant(0, None, None, None, 1e-5, 4, 100, None, 0, None, None, None, None)
    assert st == -1


def test_ops_refuse_cpu_tensors(built_lib):
    import torch

    from lightly_trian_quant_b200 import ops
    from lightly_trian_quant_b200._lib import KfError

    buf = ops.ActBuf(4, 128, "mx8", device="cpu")
    with pytest.raises(KfError):
        ops.quant_rows(torch.zeros(4, 128), buf)


def test_set_pdl_switch(built_lib):
    from lightly_trian_quant_b200 import ops

    ops.set_pdl(True)
    ops.set_pdl(False)
