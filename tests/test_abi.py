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


_C_PROBE = r"""
#include <stddef.h>
#include <stdio.h>
#include "apk.h"
#define F(T, f) printf(#T "." #f " %zu\n", offsetof(T, f))
int main(void) {
  printf("sizeof.apk_comm %zu\nsizeof.apk_operand %zu\nsizeof.apk_ag_gemm_args %zu\nsizeof.apk_gemm_rs_args %zu\n",
         sizeof(apk_comm), sizeof(apk_operand), sizeof(apk_ag_gemm_args), sizeof(apk_gemm_rs_args));
  F(apk_comm, rank); F(apk_comm, world); F(apk_comm, data); F(apk_comm, flags); F(apk_comm, data_bytes);
  F(apk_comm, flag_bytes); F(apk_comm, ctrl); F(apk_comm, ctrl_bytes); F(apk_comm, status); F(apk_comm, epoch);
  F(apk_comm, reserved); F(apk_comm, timeout_s);
  F(apk_operand, B); F(apk_operand, ldb); F(apk_operand, n_major); F(apk_operand, N); F(apk_operand, out);
  F(apk_operand, ldo); F(apk_operand, out_dtype); F(apk_operand, b_scale_mode); F(apk_operand, b_scale);
  F(apk_operand, bias); F(apk_operand, bias_dtype); F(apk_operand, reserved); F(apk_operand, result_scale);
  F(apk_ag_gemm_args, dtype); F(apk_ag_gemm_args, rows_per_rank); F(apk_ag_gemm_args, K); F(apk_ag_gemm_args, nB);
  F(apk_ag_gemm_args, A_shard); F(apk_ag_gemm_args, lda); F(apk_ag_gemm_args, Bs); F(apk_ag_gemm_args, A_gathered);
  F(apk_ag_gemm_args, return_A); F(apk_ag_gemm_args, a_scale_mode); F(apk_ag_gemm_args, A_scale);
  F(apk_ag_gemm_args, A_scale_gathered); F(apk_ag_gemm_args, gather_k); F(apk_ag_gemm_args, reserved);
  F(apk_gemm_rs_args, dtype); F(apk_gemm_rs_args, M); F(apk_gemm_rs_args, K); F(apk_gemm_rs_args, reduce_op);
  F(apk_gemm_rs_args, A); F(apk_gemm_rs_args, lda); F(apk_gemm_rs_args, B); F(apk_gemm_rs_args, a_scale_mode);
  F(apk_gemm_rs_args, scatter_cols); F(apk_gemm_rs_args, A_scale);
  /* and the library is callable from plain C: version, an argument error, the tile schedule */
  int32_t n[2] = {1792, 1792};
  printf("call.abi_version %d\n", apk_abi_version());
  printf("call.null_comm %d\n", apk_ag_gemm(NULL, NULL, NULL));
  printf("call.schedule_units %d\n", apk_debug_schedule(1, 8, 3, 4096, 2, n, 0, 0, 0, NULL, 0));
  printf("const.max_b %d\nconst.max_world %d\n", APK_MAX_B, APK_MAX_WORLD);
  return 0;
}
"""


def test_header_is_plain_c_and_ctypes_mirror_matches_field_by_field(L, tmp_path):
    """include/apk.h compiles as C99 with no torch / CUDA / C++ headers, a plain C program links
    against the library and calls it, and every field of the ctypes mirror sits where the C
    compiler puts it."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "probe.c"
    src.write_text(_C_PROBE)
    exe = tmp_path / "probe"
    libdir = Path(nat.LIB_PATH).parent
    subprocess.run(
        [gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", f"-I{ROOT / 'include'}", str(src), "-o", str(exe),
         f"-L{libdir}", "-lapk", f"-Wl,-rpath,{libdir}"],
        check=True, capture_output=True, text=True,
    )
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    got = {k: int(v) for k, v in (line.split() for line in out.splitlines())}
    mirror = {"apk_comm": nat.ApkComm, "apk_operand": nat.ApkOperand, "apk_ag_gemm_args": nat.ApkAgGemmArgs,
              "apk_gemm_rs_args": nat.ApkGemmRsArgs}
    n_fields = 0
    for cname, cls in mirror.items():
        assert got[f"sizeof.{cname}"] == C.sizeof(cls), cname
        for fname, _ in cls._fields_:
            assert got[f"{cname}.{fname}"] == getattr(cls, fname).offset, (cname, fname)
            n_fields += 1
    assert n_fields == sum(1 for k in got if k.split(".")[0] in mirror)      # no field of the header left unchecked
    assert got["call.abi_version"] == 1 and got["call.null_comm"] == nat.APK_ERR_ARG
    assert got["call.schedule_units"] == 8 * 32 * 14
    assert (got["const.max_b"], got["const.max_world"]) == (nat.APK_MAX_B, nat.APK_MAX_WORLD)
