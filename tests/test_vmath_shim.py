"""The C++ host side of the drop-in (csrc/vmath_shim.*): compiled with g++ against the C ABI, it
keeps the reference's VMath signatures and error convention."""
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "deep-learning-framework_b200"


@pytest.fixture(scope="module")
def driver(tmp_path_factory, pkg):
    pkg.load()  # the library must exist
    out = tmp_path_factory.mktemp("shim") / "shim_driver"
    cmd = ["g++", "-std=c++14", "-O1", "-Wall", "-I", str(PKG / "csrc"), "-I", "/usr/local/cuda/include",
           str(ROOT / "tests" / "shim_driver.cpp"), str(PKG / "csrc" / "vmath_shim.cpp"),
           "-L", str(PKG / "lib"), "-lkai_b200", f"-Wl,-rpath,{PKG / 'lib'}",
           "-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64", "-o", str(out)]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return out


def test_shim_error_convention(driver):
    r = subprocess.run([str(driver), "cpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "code=50002" in r.stdout and "what=cuda:" in r.stdout


@pytest.mark.gpu
def test_shim_linear_forward_backward(driver, port):
    r = subprocess.run([str(driver), "gpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    v = {}
    for line in r.stdout.splitlines():
        name, *vals = line.split()
        if name in ("x", "w", "gy", "b", "y", "gx", "gw", "gb"):
            v[name] = np.array(vals, np.float32)
    ndat, xvec, yvec = 48, 40, 72
    x, w, gy = v["x"].reshape(ndat, xvec), v["w"].reshape(yvec, xvec), v["gy"].reshape(ndat, yvec)
    y = port.activate(port.add_bias(port.matmul(w, x), v["b"]), 1)
    np.testing.assert_allclose(v["y"].reshape(ndat, yvec), y, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(v["gx"].reshape(ndat, xvec), port.matmul_backward_x(gy, w), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(v["gw"].reshape(yvec, xvec), port.matmul_backward_w(gy, x, yvec, xvec), rtol=1e-5,
                               atol=1e-5)
    np.testing.assert_allclose(v["gb"], port.add_bias_backward_b(gy), rtol=1e-5, atol=1e-5)
