"""Runs the C++ host-API test binary (csrc/tests/host_api_test.cu): provider fault modes, context life cycle,
workspace format, multicast switches and an emulated four-rank all-reduce through purlin::initialize/finalize."""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def test_cpp_host_api_binary():
    from purlin_b200 import _build
    exes = _build.build_cpp_tests()
    exe = [e for e in exes if e.name == "host_api_test"][0]
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    print(res.stdout[-4000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "PASSED" in res.stdout
