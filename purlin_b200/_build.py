"""Offline builder of the native libraries (no network, no CMake, no package fetch).

The reference compiles its binding at first use with CMake + CPM package
downloads and caches the result under ``~/.cache/purlin_jit`` keyed by a hash of
module name, exact architecture, Python version and sources, under an ``flock``
build lock (purlin/jit.py:33-46, 49-109, 112-202).  This builder keeps those
semantics (content-addressed key, one builder at a time, atomic install) but
calls ``nvcc``/``g++`` directly for sm_100a and installs the libraries inside
the package directory, so a tree built on one machine runs on another without a
compiler or a network.

Libraries:
  libpurlin_host.so   layout engine, tuning table, CPU interpreter (g++ only)
  libpurlin_cuda.so   contexts, collectives, fused kernels (nvcc, sm_100a) + the host half
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB_DIR = Path(__file__).resolve().parent / "_lib"
ARCH = "100a"

HOST_SOURCES = ["src/host_core.cpp", "src/split_policy.cpp"]
CUDA_SOURCES = ["src/collectives.cu", "src/provider.cu", "src/gemm_sm100.cu", "src/moe.cu", "src/no_alloc.cu", "src/symm_ops.cu", "src/vmm_provider.cu"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr",
    "-gencode", f"arch=compute_{ARCH},code=sm_{ARCH}",
    "-Xcompiler", "-fPIC", "-DPURLIN_NVTX=1",
]
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _existing(names):
    return [CSRC / n for n in names if (CSRC / n).exists()]


def _headers():
    return sorted((CSRC / "include").rglob("*.*"))


def cache_key(lib: str, sources, flags) -> str:
    """Order-stable key over library name, exact arch, compiler flags and source contents."""
    h = hashlib.sha256()
    h.update(lib.encode())
    h.update(ARCH.encode())
    h.update(" ".join(flags).encode())
    for p in sorted(str(s) for s in list(sources) + _headers()):
        h.update(Path(p).name.encode())   # contents decide, not where the tree is checked out
        h.update(Path(p).read_bytes())
    return h.hexdigest()[:16]


class BuildLock:
    """Exclusive inter-process lock with a time-out (two ranks importing at once build once)."""

    def __init__(self, path: Path, timeout_s: float = 1800.0):
        self.path, self.timeout_s, self.fd = path, timeout_s, None

    def __enter__(self):
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.fd = os.open(self.path, os.O_CREAT | os.O_RDWR)
        deadline = time.monotonic() + self.timeout_s
        while True:
            try:
                fcntl.flock(self.fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
                return self
            except BlockingIOError:
                if time.monotonic() > deadline:
                    os.close(self.fd)
                    raise TimeoutError(f"could not take the build lock {self.path}")
                time.sleep(0.05)

    def __exit__(self, *exc):
        fcntl.flock(self.fd, fcntl.LOCK_UN)
        os.close(self.fd)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(str(c) for c in cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout, res.stderr, flush=True)


def _build_one(lib: str, sources, compile_cmd, link_cmd, flags, force: bool, verbose: bool) -> Path:
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    out = LIB_DIR / lib
    stamp = LIB_DIR / (lib + ".key")
    key = cache_key(lib, sources, flags)
    if not force and out.exists() and stamp.exists() and stamp.read_text().strip() == key:
        return out
    with BuildLock(LIB_DIR / ".build.lock"):
        if not force and out.exists() and stamp.exists() and stamp.read_text().strip() == key:
            return out   # another process finished while this one waited
        obj_dir = LIB_DIR / "obj"
        obj_dir.mkdir(exist_ok=True)
        objs, procs = [], []
        for s in sources:
            o = obj_dir / (lib + "." + s.name + ".o")
            okey = obj_dir / (o.name + ".key")
            k = cache_key(o.name, [s], flags)
            objs.append(o)
            if not force and o.exists() and okey.exists() and okey.read_text().strip() == k:
                continue
            cmd = compile_cmd(s, o)
            if verbose:
                print(" ".join(str(c) for c in cmd), flush=True)
            procs.append((subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True), cmd, okey, k))
        for p, cmd, okey, k in procs:   # translation units compile in parallel
            text, _ = p.communicate()
            if p.returncode != 0:
                raise RuntimeError(f"build failed: {' '.join(str(c) for c in cmd)}\n{text}")
            if verbose and text:
                print(text, flush=True)
            okey.write_text(k)
        tmp = LIB_DIR / f".{lib}.{os.getpid()}.tmp"
        _run(link_cmd(objs, tmp), verbose)
        tmp.replace(out)   # atomic install
        stamp.write_text(key)
    return out


def build_host(force: bool = False, verbose: bool = False) -> Path:
    srcs = _existing(HOST_SOURCES)
    inc = ["-I", str(CSRC / "include")]
    return _build_one(
        "libpurlin_host.so", srcs,
        lambda s, o: ["g++", *CXX_FLAGS, *inc, "-c", str(s), "-o", str(o)],
        lambda objs, out: ["g++", "-shared", "-o", str(out), *map(str, objs), "-lpthread"],
        CXX_FLAGS, force, verbose)


def build_cuda(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    srcs = _existing(CUDA_SOURCES) + _existing(HOST_SOURCES)
    inc = ["-I", str(CSRC / "include")]
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])
    nvcc = _nvcc()
    return _build_one(
        "libpurlin_cuda.so", srcs,
        lambda s, o: [nvcc, *flags, *inc, "-x", "cu" if s.suffix == ".cu" else "c++", "-c", str(s), "-o", str(o)],
        lambda objs, out: [nvcc, "-shared", "-o", str(out), *map(str, objs), "-lpthread"],
        flags, force, verbose)


def fastcall_name() -> str:
    import sysconfig
    return "_purlin_fastcall" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so")


def build_fastcall(force: bool = False, verbose: bool = False) -> Path:
    """The CPython extension of the launch-bound call path (csrc/src/fastcall.c); it links against nothing but libc."""
    import sysconfig
    src = CSRC / "src" / "fastcall.c"
    flags = ["-O2", "-fPIC", "-Wall", "-I", sysconfig.get_paths()["include"]]
    return _build_one(
        fastcall_name(), [src],
        lambda s, o: ["gcc", *flags, "-c", str(s), "-o", str(o)],
        lambda objs, out: ["gcc", "-shared", "-o", str(out), *map(str, objs)],
        flags, force, verbose)


def build_cpp_tests(force: bool = False, verbose: bool = False, folder: str = "tests"):
    """The C++ test binaries (csrc/tests) or example programs (csrc/examples), linked against the in-tree libpurlin_cuda.so."""
    lib = build_cuda(force, verbose)
    out = []
    for src in sorted((CSRC / folder).glob("*.cu")):
        exe = LIB_DIR / src.stem
        stamp = LIB_DIR / (src.stem + ".key")
        key = cache_key(src.stem, [src, lib], NVCC_FLAGS)
        if force or not exe.exists() or not stamp.exists() or stamp.read_text().strip() != key:
            with BuildLock(LIB_DIR / ".build.lock"):
                tmp = LIB_DIR / f".{src.stem}.{os.getpid()}.tmp"
                _run([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC / "include"), str(src), "-o", str(tmp), "-L", str(LIB_DIR),
                      "-lpurlin_cuda", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"], verbose)
                tmp.replace(exe)
                stamp.write_text(key)
        out.append(exe)
    return out


def build_cpu_tests(force: bool = False, verbose: bool = False):
    """Host-only C++ unit tests (csrc/tests/*.cpp): header-level checks that need neither nvcc nor a GPU."""
    out = []
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    for src in sorted((CSRC / "tests").glob("*.cpp")):
        exe = LIB_DIR / src.stem
        stamp = LIB_DIR / (src.stem + ".key")
        key = cache_key(src.stem, [src], CXX_FLAGS)
        if force or not exe.exists() or not stamp.exists() or stamp.read_text().strip() != key:
            with BuildLock(LIB_DIR / ".build.lock"):
                tmp = LIB_DIR / f".{src.stem}.{os.getpid()}.tmp"
                _run(["g++", *CXX_FLAGS, "-I", str(CSRC / "include"), str(src), "-o", str(tmp)], verbose)
                tmp.replace(exe)
                stamp.write_text(key)
        out.append(exe)
    return out


def build_examples(force: bool = False, verbose: bool = False):
    """The C++ example programs of csrc/examples (device-side collectives, copy-engine baselines, push/pull)."""
    return build_cpp_tests(force, verbose, folder="examples")


def build_all(force: bool = False, verbose: bool = False):
    return (build_host(force, verbose), build_cuda(force, verbose), build_fastcall(force, verbose), *build_cpp_tests(force, verbose),
            *build_examples(force, verbose), *build_cpu_tests(force, verbose))


if __name__ == "__main__":
    t0 = time.time()
    paths = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(f"built {[str(p) for p in paths]} in {time.time() - t0:.1f}s")
