"""CPU: the shared library loads without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "aotriton_b200.h").read_text()
    return re.findall(r"AB200_API\s+[\w\s\*]+?\b(ab200_\w+)\s*\(", text)


def test_header_and_loader_agree():
    from aotriton_b200 import cabi
    assert _declared() == cabi.SYMBOLS


def test_library_exports_every_declared_symbol():
    from aotriton_b200 import cabi
    lib = cabi.lib()
    for name in _declared():
        assert hasattr(lib, name), name
    assert b"sm_100a" in lib.ab200_version()
    for name in ("hipGetLastError", "hipDeviceSynchronize"):
        assert hasattr(lib, name)


def test_struct_layout_matches_header(tmp_path):
    """Compile the header as plain C and compare sizeof/offsetof with the ctypes mirrors."""
    import subprocess
    from aotriton_b200 import cabi
    src = tmp_path / "layout.c"
    src.write_text(r"""
#include <stdio.h>
#include <stddef.h>
#include "aotriton_b200.h"
int main(void) {
  printf("%zu %zu %zu %zu ", sizeof(ab200_view4), sizeof(ab200_attn_problem), sizeof(ab200_attn_fwd_args),
         sizeof(ab200_attn_bwd_args));
  printf("%zu %zu %zu ", offsetof(ab200_attn_problem, cu_seqlens_q), offsetof(ab200_attn_problem, philox_offset2),
         offsetof(ab200_attn_problem, philox_num_head_q));
  printf("%zu %zu %zu ", offsetof(ab200_attn_fwd_args, lse), offsetof(ab200_attn_fwd_args, encoded_softmax_cols),
         offsetof(ab200_attn_fwd_args, persistent_atomic_counter));
  printf("%zu %zu %zu\n", offsetof(ab200_attn_bwd_args, dbias), offsetof(ab200_attn_bwd_args, deterministic),
         offsetof(ab200_attn_bwd_args, dq_acc));
  return 0;
}
""")
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [ctypes.sizeof(cabi.View4), ctypes.sizeof(cabi.Problem), ctypes.sizeof(cabi.FwdArgs),
            ctypes.sizeof(cabi.BwdArgs), cabi.Problem.cu_seqlens_q.offset, cabi.Problem.philox_offset2.offset,
            cabi.Problem.philox_num_head_q.offset, cabi.FwdArgs.lse.offset,
            cabi.FwdArgs.encoded_softmax_cols.offset, cabi.FwdArgs.persistent_atomic_counter.offset,
            cabi.BwdArgs.dbias.offset, cabi.BwdArgs.deterministic.offset, cabi.BwdArgs.dq_acc.offset]
    assert got == want


def test_cpp_api_symbols_present():
    import subprocess
    out = subprocess.run(["nm", "-DC", str(ROOT / "aotriton_b200" / "libaotriton_v2.so")], capture_output=True,
                         text=True).stdout
    for sym in ("aotriton::v3::flash::attn_fwd(", "aotriton::v3::flash::attn_bwd(",
                "aotriton::v2::flash::check_gpu(", "aotriton::v2::flash::debug_simulate_encoded_softmax(",
                "aotriton::v2::flash::attn_fwd_compact_varlen(", "aotriton::v2::flash::attn_bwd_compact_varlen(",
                "aotriton::getGpuFromStream(", "aotriton::getMultiProcessorCount(",
                "aotriton::v3::flash::attn_fwd_params::attn_fwd_params()"):
        assert sym in out, sym
