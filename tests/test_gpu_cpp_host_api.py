"""Runs the C++ test binaries of csrc/tests on a GPU:
  host_api_test    provider fault modes, context life cycle, workspace format, multicast switches, emulated all-reduce
                   through purlin::initialize / finalize (the reference's csrc/tests/setup.cu re-expressed)
  device_api_test  a user kernel that computes and then calls purlin::allReduce from device code, and the Atom alone
"""
import subprocess

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["host_api_test", "device_api_test"])
def test_cpp_binary(name):
    from purlin_b200 import _build
    exes = _build.build_cpp_tests()
    exe = [e for e in exes if e.name == name][0]
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    print(res.stdout[-4000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "PASSED" in res.stdout
