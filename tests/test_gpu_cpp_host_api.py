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


@pytest.mark.multigpu
@pytest.mark.parametrize("args", [
    ["all", "8K", "4M", "0", "3", "1", "--provider", "vmm", "--staging", "8M"],
    ["all", "32K", "2M", "2", "3", "1", "--provider", "peer", "--staging", "8M", "--reduction-mode", "deterministic"],
    ["ar", "16M", "32M", "0", "3", "1", "--provider", "vmm", "--staging", "8M"],     # payload larger than the staging buffer
], ids=["vmm-stream", "peer-graph-deterministic", "vmm-segmented"])
def test_multi_gpu_bench_binary(args):
    """One process, one thread per GPU, all seven collectives through purlin::initialize / allReduce / ... / finalize
    with the native virtual-memory provider (NVLS alias included) or plain peer memory; every size compared exactly."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    from purlin_b200 import _build
    exe = [e for e in _build.build_cpp_tests() if e.name == "multi_gpu_bench"][0]
    res = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=600)
    print(res.stdout[-6000:])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "PASSED" in res.stdout


@pytest.mark.parametrize("name,args", [
    ("device_collectives", ["ar", "262144", "24", "3"]),
    ("device_collectives", ["ag", "262144", "24", "3"]),
    ("device_collectives", ["rs", "262144", "24", "3"]),
    ("device_collectives", ["a2a", "262144", "24", "3"]),
    ("device_collectives", ["ar", "98304", "12", "2", "8"]),
    ("copy_engine", ["4194304", "16", "3"]),
], ids=["device-ar", "device-ag", "device-rs", "device-a2a", "device-ar-8-ranks", "copy-engine"])
def test_cpp_example(name, args):
    """The example programs of csrc/examples: user kernels calling the device-side collectives with hand-set launch
    configurations (virtual ranks on one GPU), and the copy-engine / push / pull point-to-point comparison."""
    from purlin_b200 import _build
    exe = [e for e in _build.build_examples() if e.name == name][0]
    res = subprocess.run([str(exe), *args], capture_output=True, text=True, timeout=300)
    print(res.stdout[-3000:])
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "PASSED" in res.stdout
