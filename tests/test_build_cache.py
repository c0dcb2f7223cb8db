"""Offline builder: content key, build lock, single build under contention.
Counterpart of tests/test_jit.py in the reference (cache key includes the exact architecture and is order-stable;
two concurrent callers build once), for a builder that calls nvcc/g++ directly instead of CMake."""
import threading
import time
from pathlib import Path

from purlin_b200 import _build


def test_cache_key_depends_on_contents_flags_and_arch(tmp_path, monkeypatch):
    a, b = tmp_path / "a.cu", tmp_path / "b.cu"
    a.write_text("int a;")
    b.write_text("int b;")
    k1 = _build.cache_key("lib", [a, b], ["-O3"])
    assert k1 == _build.cache_key("lib", [b, a], ["-O3"]), "order of sources does not matter"
    assert k1 != _build.cache_key("lib", [a, b], ["-O2"])
    assert k1 != _build.cache_key("other", [a, b], ["-O3"])
    monkeypatch.setattr(_build, "ARCH", "90a")
    assert k1 != _build.cache_key("lib", [a, b], ["-O3"]), "the exact architecture is part of the key"
    monkeypatch.setattr(_build, "ARCH", "100a")
    a.write_text("int a2;")
    assert k1 != _build.cache_key("lib", [a, b], ["-O3"])
    assert any("sm_100a" in f or "100a" in f for f in _build.NVCC_FLAGS) and "-lineinfo" in _build.NVCC_FLAGS


def test_build_lock_serialises_and_times_out(tmp_path):
    lock = tmp_path / "x.lock"
    order = []

    def worker(i):
        with _build.BuildLock(lock):
            order.append(("in", i))
            time.sleep(0.05)
            order.append(("out", i))
    ts = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for k in range(0, len(order), 2):
        assert order[k][0] == "in" and order[k + 1] == ("out", order[k][1]), "no two holders overlap"
    import fcntl, os
    fd = os.open(lock, os.O_CREAT | os.O_RDWR)
    fcntl.flock(fd, fcntl.LOCK_EX)
    try:
        t0 = time.monotonic()
        try:
            with _build.BuildLock(lock, timeout_s=0.2):
                raise AssertionError("lock should not have been granted")
        except TimeoutError:
            assert time.monotonic() - t0 < 2.0
    finally:
        fcntl.flock(fd, fcntl.LOCK_UN)
        os.close(fd)


def test_concurrent_callers_build_once(tmp_path, monkeypatch):
    src = tmp_path / "csrc" / "src"
    src.mkdir(parents=True)
    (tmp_path / "csrc" / "include").mkdir()
    (src / "one.cpp").write_text("int one() { return 1; }\n")
    monkeypatch.setattr(_build, "CSRC", tmp_path / "csrc")
    monkeypatch.setattr(_build, "LIB_DIR", tmp_path / "lib")
    compiles = []
    real_popen = _build.subprocess.Popen

    def counting_popen(cmd, **kw):
        if "-c" in cmd:          # compile steps only (the link step goes through subprocess.run -> Popen too)
            compiles.append(cmd)
            time.sleep(0.1)
        return real_popen(cmd, **kw)
    monkeypatch.setattr(_build.subprocess, "Popen", counting_popen)

    def build():
        return _build._build_one("libone.so", [src / "one.cpp"],
                                 lambda s, o: ["g++", "-fPIC", "-c", str(s), "-o", str(o)],
                                 lambda objs, out: ["g++", "-shared", "-o", str(out), *map(str, objs)], ["-fPIC"], False, False)
    results = []
    ts = [threading.Thread(target=lambda: results.append(build())) for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert len(compiles) == 1, "the first holder of the lock builds, the others find the result"
    assert all(Path(r).exists() for r in results) and len(set(results)) == 1
    (src / "one.cpp").write_text("int one() { return 2; }\n")
    build()
    assert len(compiles) == 2, "changed contents rebuild"
