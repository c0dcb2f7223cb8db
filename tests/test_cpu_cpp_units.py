"""Runs the host-only C++ unit tests of csrc/tests/*.cpp (compile-time loop, prefetch-ring driver, partitioning).

Counterpart of the single-GPU unit binaries csrc/tests/static_for.cu and csrc/tests/pipeline.cu of the reference;
the headers under test are host/device code, so the logic is checked here without a GPU and again inside a kernel
by csrc/tests/device_api_test.cu.
"""
import subprocess


def test_cpu_unit_binary():
    from purlin_b200 import _build
    exes = _build.build_cpu_tests()
    assert exes, "no host-only C++ tests were found"
    for exe in exes:
        res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
        print(res.stdout[-4000:])
        assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
        assert "PASSED" in res.stdout and "FAIL " not in res.stdout
