"""CPU tests of the C-ABI boundary: the library builds and loads, exports every symbol the header
declares, the ctypes structures match the C layout, and host-side validation answers without a GPU."""
import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "ssd_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ssd_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_entry_points(cabi):
    assert set(declared_functions()) == set(cabi.EXPORTS)


def test_library_exports_every_declared_symbol(cabi):
    lib = cabi.load()
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert lib.ssd_b200_abi_version() == cabi.ABI_VERSION


def test_ctypes_structs_match_c_layout(cabi, tmp_path):
    src = tmp_path / "layout.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "ssd_b200.h"\n'
        'int main(void){printf("%zu %zu %zu %zu %zu %zu %zu\\n", sizeof(ssd_b200_shape), sizeof(ssd_b200_fwd_args),'
        'sizeof(ssd_b200_bwd_args), offsetof(ssd_b200_fwd_args, workspace), offsetof(ssd_b200_bwd_args, dinit),'
        'offsetof(ssd_b200_bwd_args, workspace_bytes), offsetof(ssd_b200_fwd_args, a_cumsum));return 0;}\n')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(src), "-o", str(exe)],
                   check=True)
    got = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(cabi.Shape), C.sizeof(cabi.FwdArgs), C.sizeof(cabi.BwdArgs), cabi.FwdArgs.workspace.offset,
            cabi.BwdArgs.dinit.offset, cabi.BwdArgs.workspace_bytes.offset, cabi.FwdArgs.a_cumsum.offset]
    assert got == want


def _shape(cabi, **kw):
    base = dict(abi_version=cabi.ABI_VERSION, dtype=cabi.F32, a_dtype=cabi.F32, path=cabi.PATH_SIMT, batch=2,
                seqlen=512, nheads=8, headdim=64, dstate=64, ngroups=1, chunk=64)
    base.update(kw)
    return cabi.Shape(**base)


def test_host_validation_without_gpu(cabi):
    lib = cabi.load()
    s = _shape(cabi)
    assert lib.ssd_b200_resolve_path(C.byref(s)) == cabi.PATH_SIMT
    fwd = lib.ssd_b200_workspace_bytes(C.byref(s), cabi.PASS_FWD)
    bwd = lib.ssd_b200_workspace_bytes(C.byref(s), cabi.PASS_BWD)
    assert fwd >= 2 * 8 * 8 * 64 * 64 * 4 and bwd > 2 * fwd
    bad = _shape(cabi, seqlen=500)
    assert lib.ssd_b200_resolve_path(C.byref(bad)) == cabi.EINVAL
    assert "not divisible by chunk_size" in cabi.last_error()
    with pytest.raises(AssertionError, match="not divisible"):
        cabi.check(cabi.EINVAL)
    assert lib.ssd_b200_workspace_bytes(C.byref(bad), cabi.PASS_FWD) == 0
    assert lib.ssd_b200_resolve_path(C.byref(_shape(cabi, ngroups=3))) == cabi.EINVAL
    assert lib.ssd_b200_resolve_path(C.byref(_shape(cabi, abi_version=99))) == cabi.EINVAL
    assert lib.ssd_b200_resolve_path(C.byref(_shape(cabi, headdim=512))) == cabi.EUNSUPPORTED
    # argument checks happen before any CUDA call
    args = cabi.FwdArgs(shape=s)
    assert lib.ssd_b200_fwd(C.byref(args), None) == cabi.EINVAL
    assert lib.ssd_b200_fwd(None, None) == cabi.EINVAL
    assert lib.ssd_b200_bwd(None, None) == cabi.EINVAL


def test_operator_rejects_cpu_tensors(pkg, cabi):
    import torch
    x = torch.zeros(1, 64, 2, 8)
    with pytest.raises(AssertionError):
        pkg.fused_ssd_scan(x, torch.zeros(1, 64, 2), torch.zeros(1, 64, 2, 4), torch.zeros(1, 64, 2, 4), 32)


def test_missing_library_fails_loudly(cabi, monkeypatch, tmp_path):
    monkeypatch.setattr(cabi, "_lib", None)
    monkeypatch.setattr(cabi, "library_path", lambda: tmp_path / "libssd_b200.so")
    with pytest.raises(ImportError, match="no fallback"):
        cabi.load()
