"""The C-ABI library loads without a GPU, exports every symbol the header declares,
its ctypes mirror has the compiler's struct sizes, and host-side validation rejects
bad calls without launching anything."""

import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import pytest

from instantmimic_b200 import _lib, abi

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "imnewton.h"


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(imn_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    names = _declared_functions()
    assert "imn_solve" in names and "imn_tree_ldl_solve" in names and len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(abi.SYMBOLS) == names
    assert lib.imn_abi_version() == abi.IMN_ABI_VERSION


def test_ctypes_structs_match_the_compiler(tmp_path):
    structs = ["ImnModel", "ImnData", "ImnCtx", "ImnSparsePlan", "ImnTreePlan", "ImnBlockedPlan", "ImnLaunchInfo",
               "ImnImplicit", "ImnAdvance", "ImnBallLimits"]
    src = tmp_path / "sizes.c"
    body = "".join(f'  printf("{s} %zu\\n", sizeof({s}));\n' for s in structs)
    src.write_text(f'#include <stdio.h>\n#include "{HEADER}"\nint main(void) {{\n{body}  return 0;\n}}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["/usr/bin/gcc", "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    sizes = dict(line.split() for line in out.strip().splitlines())
    for s in structs:
        assert C.sizeof(getattr(abi, s)) == int(sizes[s]), s


def test_validation_rejects_bad_calls_before_any_launch():
    lib = _lib.lib()
    m, d, c = abi.ImnModel(), abi.ImnData(), abi.ImnCtx()
    assert lib.imn_solve(None, C.byref(d), C.byref(c), None) == abi.IMN_ERR_NULL
    m.nv, m.nv_pad, m.iterations = 80, 96, 4  # beyond the fused path
    assert lib.imn_solve(C.byref(m), C.byref(d), C.byref(c), None) == abi.IMN_ERR_UNSUPPORTED
    assert b"nv 80" in lib.imn_last_error()
    m.nv, m.nv_pad = 34, 40  # nv_pad not a multiple of 16
    assert lib.imn_solve(C.byref(m), C.byref(d), C.byref(c), None) == abi.IMN_ERR_UNSUPPORTED
    m.nv, m.nv_pad, m.iterations = 34, 48, 0
    assert lib.imn_solve(C.byref(m), C.byref(d), C.byref(c), None) == abi.IMN_ERR_UNSUPPORTED
    m.iterations = 4
    m.n_tolerance = m.n_ls_tolerance = m.n_meaninertia = 1
    assert lib.imn_solve(C.byref(m), C.byref(d), C.byref(c), None) == abi.IMN_ERR_NULL  # no buffers
    plan = abi.ImnTreePlan()
    assert lib.imn_tree_ldl_solve(C.byref(plan), None, 0, None, 0, None, 0, 1, None) == abi.IMN_ERR_NULL
    bp = abi.ImnBlockedPlan()
    bp.nv, bp.pad = 35, 40
    one = C.c_float(0)
    p = C.addressof(one)
    assert lib.imn_blocked_dense_factor_solve(C.byref(bp), p, 0, p, p, p, None, 1, 1, 1, None) == abi.IMN_ERR_SHAPE


def test_copy_wait_limit_is_validated():
    lib = _lib.lib()
    assert lib.imn_set_copy_wait_limit(0, 0) == abi.IMN_ERR_SHAPE
    assert b"positive" in lib.imn_last_error()
    assert lib.imn_set_copy_wait_limit(1 << 22, 0) == 0


def test_launch_info_reports_geometry_without_a_gpu():
    """Host-only: which kernel variant and how much shared memory a model gets."""
    import numpy as np

    from instantmimic_b200 import binding, synthetic
    from helpers import host_ctx

    lib = _lib.lib()
    # humanoid: J stays in shared memory; the SNU-like model streams it (the 128-row J would
    # leave room for 4 worlds per SM, the row tile for 7)
    for name, resident, threads in (("humanoid", 1, 32), ("snu", 0, 64)):
        m, d, _ = synthetic.make_workload(name, 4, seed=0)
        ms, ds = binding.model_struct(m), binding.data_struct(m, d)
        cs = binding.ctx_struct(ds, host_ctx(m, d), np.zeros(1, np.int32))
        info = abi.ImnLaunchInfo()
        assert lib.imn_launch_info(C.byref(ms), C.byref(ds), C.byref(cs), C.byref(info)) == 0
        assert (info.j_resident, info.world_threads, info.grid) == (resident, threads, 4)
        assert 0 < info.smem_bytes <= 227 * 1024
    m, d, _ = synthetic.make_sweep_point(64, 512, 2, seed=0)
    ms, ds = binding.model_struct(m), binding.data_struct(m, d)
    cs = binding.ctx_struct(ds, None, None)
    info = abi.ImnLaunchInfo()
    assert lib.imn_launch_info(C.byref(ms), C.byref(ds), C.byref(cs), C.byref(info)) == 0
    assert info.j_resident == 0  # 512 rows x 64 dofs stream through the staging tile


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "_PATH", tmp_path / "absent.so")
    with pytest.raises(_lib.ImnError, match="no CPU or PyTorch fallback"):
        _lib.lib()
