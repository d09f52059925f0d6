"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, the ctypes
table matches the header, and compute calls fail loudly instead of falling back to anything."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "kai_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"KAI_API\s+[\w\s\*]+?\b(kai_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load()
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in kai_b200.h but not exported"


def test_ctypes_table_matches_header(pkg):
    assert sorted(pkg.capi.SIGNATURES) == declared_symbols()


def test_version_and_options(pkg):
    lib = pkg.load()
    assert b"sm_100a" in lib.kai_version()
    assert lib.kai_get_option(b"tc_bn") in (128, 256)
    assert lib.kai_set_option(b"tc_bn", 100) == pkg.capi.E_INVALID_ARG
    assert lib.kai_set_option(b"no_such_option", 1) == pkg.capi.E_INVALID_ARG
    assert b"no_such_option" in lib.kai_last_error_string()
    assert lib.kai_get_option(b"no_such_option") == -1


def test_no_host_branch(pkg):
    """device = -1 selects the reference's CPU loop; this library has none and says so."""
    lib = pkg.load()
    rc = lib.kai_matmul(-1, None, None, None, 4, 4, 4, 0, None)
    assert rc == pkg.capi.E_NO_HOST_PATH
    assert b"no CPU branch" in lib.kai_last_error_string()


def test_compute_fails_loudly_without_gpu(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this machine has a GPU")
    with pytest.raises(pkg.KaiError) as e:
        pkg.vmath.mem_alloc(0, 1024)
    assert e.value.code > 0 and "cuda:" in e.value.message  # a cudaError_t, the reference's text


def test_missing_library_is_an_error(pkg, tmp_path):
    with pytest.raises(FileNotFoundError):
        pkg.capi.load(tmp_path / "libkai_b200.so")
