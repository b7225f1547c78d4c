"""The C-ABI library: it loads without a GPU, exports what include/apk.h declares, and rejects
bad arguments before touching a device."""
import ctypes as C
import re
from pathlib import Path

import pytest

from autoparallel_b200 import _native as nat
from autoparallel_b200.build import build_native

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def L():
    build_native()
    return nat.lib()


def _declared_symbols():
    text = (ROOT / "include" / "apk.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(apk_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(L):
    declared = _declared_symbols()
    assert declared == sorted(nat.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(L, name), name


def test_abi_version(L):
    assert L.apk_abi_version() == 1


def test_struct_layouts_match_header():
    # sizes the C compiler gives the structs in include/apk.h (LP64)
    assert C.sizeof(nat.ApkComm) == 8 + 8 * 8 + 8 * 8 + 8 + 8 + 8 + 8 + 8 + 4 + 4 + 8
    assert C.sizeof(nat.ApkOperand) == 80
    assert C.sizeof(nat.ApkAgGemmArgs) == 16 + 8 + 8 + 4 * 80 + 8 + 8 + 8 + 8 + 8
    assert C.sizeof(nat.ApkGemmRsArgs) == 16 + 8 + 8 + 80 + 8 + 8


def test_workspace_size_helpers(L):
    a = nat.ApkAgGemmArgs()
    a.dtype, a.rows_per_rank, a.K = nat.APK_BF16, 4096, 4096
    assert L.apk_ag_gemm_arena_bytes(C.byref(a), 8) == 4096 * 4096 * 2
    assert L.apk_ag_gemm_arena_bytes(C.byref(a), 1) == 0
    a.dtype, a.a_scale_mode = nat.APK_E4M3, nat.APK_SCALE_VECTOR
    assert L.apk_ag_gemm_arena_bytes(C.byref(a), 8) == 4096 * 4096 + 4096 * 4
    r = nat.ApkGemmRsArgs()
    r.M, r.B.N, r.B.out_dtype = 32768, 4096, nat.APK_BF16
    # 8 source slots of 32 x 16 bf16 tiles of 128 x 256, plus fp32 sums of one slot (= 2 bf16 slots)
    assert L.apk_gemm_rs_arena_bytes(C.byref(r), 8) == (8 + 2) * 4096 * 4096 * 2
    assert L.apk_ctrl_bytes(4096, 8) == 256 + 4 * 32 * 8


def test_argument_errors_without_device(L):
    assert L.apk_ag_gemm(None, None, None) == nat.APK_ERR_ARG
    assert b"comm" in L.apk_last_error()
    c = nat.ApkComm()
    c.rank, c.world = 0, 9
    assert L.apk_gemm_rs(C.byref(c), None, None) == nat.APK_ERR_ARG
    c.world = 1
    assert L.apk_gemm_rs(C.byref(c), None, None) == nat.APK_ERR_ARG  # status word missing
    with pytest.raises(nat.ApkError):
        nat.check(L.apk_symm_export(None, None))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(nat, "_lib", None)
    monkeypatch.setenv("APK_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        nat.lib()
