"""The C-ABI library builds, loads without a GPU and exports every symbol that
include/cdeep.h declares (no compute call is made here)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "cdeep.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cd_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    from complexity_deep_b200 import build, _lib
    path = build.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    declared = _declared_symbols()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in cdeep.h but not exported"
    # the ctypes table binds exactly the declared entry points
    assert sorted(_lib.SIGNATURES) == declared
    # the checking build exports the same entry points and says what it is
    checks = _lib.open_library(build.build(checks=True))
    assert checks.cd_checks_enabled() == 1 and _lib.load().cd_checks_enabled() == 0
    assert checks.cd_error_string(5).startswith(b"checking build")


def test_version_and_error_strings():
    from complexity_deep_b200 import _lib
    lib = _lib.load()
    assert lib.cd_version() == _lib.ABI_VERSION
    assert lib.cd_error_string(0) == b"ok"
    assert lib.cd_error_string(4) == b"a kernel gave up on a bounded wait"
    assert lib.cd_gate_up_packed_rows(704, 128) == 1408
    assert lib.cd_gate_up_packed_rows(704, 256) == 1536
    assert lib.cd_gate_up_packed_rows(5632, 256) == 11264
    assert lib.cd_route_workspace_bytes(65536, 8) == 32 * 8 * 4


def test_argument_checks_need_no_gpu():
    from complexity_deep_b200 import _lib
    lib = _lib.load()
    # invalid sizes are rejected before any CUDA call
    assert lib.cd_route(None, None, 0, 8, 16, None, None, None, None, None, None, 0, None) == 1
    assert lib.cd_linear(None, None, None, None, None, None, 16, 12, 64, None) == 1  # K % 8 != 0
    assert lib.cd_moe_up(None, None, 1, None, None, 16, 64, 48, 100, None) == 1  # block_n
    assert lib.cd_gate_up_packed_rows(704, 32) == 1408
    assert lib.cd_max_groups() == 128
    # sum_out without a residual / aliasing x is refused (the header's contract)
    assert lib.cd_rmsnorm(64, None, 64, 1e-6, 128, 192, None, 4, 8, None) == 1
    assert lib.cd_rmsnorm(64, 64, 64, 1e-6, 64, 192, None, 4, 8, None) == 1
