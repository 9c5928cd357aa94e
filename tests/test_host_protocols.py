"""Host-side runtime protocols: the shm ring between two processes, and the ring + the
epoch/flag barrier model under ThreadSanitizer (host threads only; no GPU involved)."""
import multiprocessing as mp
import os
import pathlib
import shutil
import subprocess
import uuid

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]


def _producer(name, n):
    from vllm_omni_b200.utils.shm_ring import ShmRing
    r = ShmRing(name, create=False)
    for i in range(n):
        assert r.put_obj({"i": i, "payload": b"x" * (i % 50)}, timeout=10)
    r.close()


def test_shm_ring_between_processes():
    from vllm_omni_b200.utils.shm_ring import ShmRing
    name = f"/omni_test_ring_{uuid.uuid4().hex[:8]}"
    ring = ShmRing(name, create=True, slot_bytes=512, num_slots=8)
    try:
        assert ring.pop() is None and len(ring) == 0
        with pytest.raises(ValueError):
            ring.push(b"y" * 600)
        p = mp.get_context("spawn").Process(target=_producer, args=(name, 200))
        p.start()
        for i in range(200):
            m = ring.get_obj(timeout=20)
            assert m is not None and m["i"] == i and len(m["payload"]) == i % 50
        p.join(20)
        assert p.exitcode == 0 and len(ring) == 0
        for i in range(8):
            assert ring.push(b"z")
        assert not ring.push(b"z", timeout=0.01)          # full: bounded wait, then False
    finally:
        ring.close()


def test_protocols_under_thread_sanitizer(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = tmp_path / "protocol_tsan"
    src = ROOT / "vllm_omni_b200" / "csrc" / "host_tests" / "protocol_tsan.cpp"
    b = subprocess.run([gxx, "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-o", str(exe), str(src), "-pthread", "-lrt"],
                       capture_output=True, text=True)
    if b.returncode != 0 and "sanitize" in (b.stderr or ""):
        pytest.skip("ThreadSanitizer runtime is not installed")
    assert b.returncode == 0, b.stderr[-2000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300,
                       env={**os.environ, "TSAN_OPTIONS": "halt_on_error=1 exitcode=66"})
    assert r.returncode == 0, (r.stdout + r.stderr)[-3000:]
    assert "ring_errors=0 barrier_errors=0" in r.stdout
    assert "ThreadSanitizer" not in r.stderr
