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


def test_gemm_params_mirror_matches_the_header(built_lib, tmp_path):
    """the ctypes mirror of kf_gemm_params has the size and the field offsets the C compiler gives the header's struct."""
    import ctypes as C
    import subprocess
    from pathlib import Path

    from lightly_trian_quant_b200 import _lib

    inc = Path(__file__).resolve().parents[1] / "include"
    fields = [name for name, _ in _lib.GemmParams._fields_]
    src = tmp_path / "layout.c"
    body = "".join(f'  printf("{f} %zu\\n", offsetof(kf_gemm_params, {f}));\n' for f in fields)
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "kf_b200.h"\nint main(void) {\n  printf("sizeof %zu\\n", sizeof(kf_gemm_params));\n'
                   + body + "  return 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(inc), str(src), "-o", str(exe)], check=True)
    out = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    assert int(out["sizeof"]) == C.sizeof(_lib.GemmParams)
    for f in fields:
        assert int(out[f]) == getattr(_lib.GemmParams, f).offset, f


def test_batched_products_are_checked_on_the_host(built_lib):
    """kf_gemm_bs with batch > 0 only takes bf16 operands with the PLAIN epilogue and consistent row counts."""
    from lightly_trian_quant_b200 import _lib

    L = _lib.lib()
    p = _lib.GemmParams()
    p.fmt, p.epi, p.M, p.N, p.K = _lib.KF_FMT["nv4"], _lib.KF_EPI["plain"], 400, 256, 256
    p.batch, p.a_rows_per_batch, p.w_rows_per_batch = 2, 200, 256
    p.A = p.W = p.SFA = p.SFW = p.C = 4096                    # never dereferenced: the call is rejected on the host
    assert L.kf_gemm_bs(p, None) == -1 and "batched" in L.kf_last_error_string().decode()
    p.fmt = _lib.KF_FMT["bf16"]
    p.a_rows_per_batch = 199                                   # M != batch * rows
    assert L.kf_gemm_bs(p, None) == -1 and "batched" in L.kf_last_error_string().decode()
    p.a_rows_per_batch, p.w_rows_per_batch = 200, 128          # fewer W rows per product than columns
    assert L.kf_gemm_bs(p, None) == -1 and "batched" in L.kf_last_error_string().decode()


def test_host_checks_of_the_head_kernels(built_lib):
    """kf_dw_ln takes channel counts in steps of 128 up to 1024; ops.bmm_nt refuses anything but matching contiguous bf16 batches."""
    import torch

    from lightly_trian_quant_b200 import _lib, ops
    from lightly_trian_quant_b200._lib import KfError

    L = _lib.lib()
    assert L.kf_dw_ln(4096, None, 4096, 4096, 4096, 4096, 1, 4, 4, 192, 1e-6, 1, None) == -1
    assert "multiple of 128" in L.kf_last_error_string().decode()
    assert L.kf_dw_ln(4096, None, 4096, 4096, 4096, 4096, 1, 4, 4, 1152, 1e-6, 1, None) == -1
    a = torch.zeros(2, 8, 64, dtype=torch.bfloat16)
    w = torch.zeros(2, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(KfError):
        ops.bmm_nt(a, w)                                     # CPU tensors
    with pytest.raises(KfError):
        ops.bmm_nt(a.float(), w)                             # wrong dtype (checked before the device)
