"""The C++ host runtime under AddressSanitizer + UBSan and under ThreadSanitizer.

The sanitizer runtimes cannot be loaded into the Python interpreter after the fact, so the library's sources are
compiled together with a self-test driver (csrc/host/selftest/host_selftest.cc) into a plain executable per sanitizer.
The driver covers malformed inputs of every parser and the threaded batch loader under contention, and walks an LMDB
environment written by the Python writer."""
import os
import shutil
import subprocess

import pytest

from rembrandt_b200 import _native
from rembrandt_b200.data.lmdb_reader import write_env

HOST = os.path.join(os.path.dirname(os.path.abspath(_native.__file__)), "csrc", "host")


def _build(tmp_path, name, flags):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / name)
    srcs = [os.path.join(HOST, f) for f in sorted(os.listdir(HOST)) if f.endswith(".cc")]
    srcs.append(os.path.join(HOST, "selftest", "host_selftest.cc"))
    r = subprocess.run([cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags, *srcs, "-o", exe, "-pthread"],
                       capture_output=True, text=True, timeout=600)
    if r.returncode != 0 and ("sanitize" in r.stderr or "cannot find -l" in r.stderr):
        pytest.skip("sanitizer runtime not installed")
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


@pytest.mark.parametrize("name,flags", [("asan_ubsan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=all"]),
                                        ("tsan", ["-fsanitize=thread"])])
def test_host_runtime_is_clean_under_sanitizers(tmp_path, name, flags):
    exe = _build(tmp_path, "selftest_" + name, flags)
    env_dir = tmp_path / "env"
    env_dir.mkdir()
    items = [(b"%08d" % i, bytes([i & 0xFF]) * (10 + 37 * i % 3000)) for i in range(300)]   # some go to overflow pages
    write_env(str(env_dir), items, max_leaf_nodes=7)
    r = subprocess.run([exe, str(env_dir), str(len(items))], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1", TSAN_OPTIONS="halt_on_error=1"))
    assert r.returncode == 0, (r.stdout[-2000:] + "\n" + r.stderr[-6000:])
    assert "host self-test: ok" in r.stdout and "lmdb: 300 entries" in r.stdout
