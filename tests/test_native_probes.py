"""Builds and runs the stand-alone CUDA probes of tests/native (IPC map + remote read, remote
store visibility, bounded flag ping-pong). The reference ships the equivalent programs to be run
by hand (src/test/{segfault,writeremote,remotesync}/test.sh: `mpirun -n 2 ./simple_test`)."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "native")
BIN = os.path.join(HERE, "peer_probe")


def _build():
    src = os.path.join(HERE, "peer_probe.cu")
    if os.path.exists(BIN) and os.path.getmtime(BIN) >= os.path.getmtime(src):
        return
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-lineinfo", "-o", BIN, src], check=True)


def test_probe_builds_for_sm100a():
    _build()
    assert os.access(BIN, os.X_OK)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["ipc", "pingpong"])
def test_probe_runs(mode):
    _build()
    r = subprocess.run([BIN, mode], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr
