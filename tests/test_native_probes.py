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


BOUNDS = os.path.join(HERE, "bounds_probe")


def _build_bounds():
    src = os.path.join(HERE, "bounds_probe.cu")
    root = os.path.dirname(os.path.dirname(HERE))
    hdr = os.path.join(root, "csrc", "cuda", "kernels", "comm.cuh")
    if os.path.exists(BOUNDS) and os.path.getmtime(BOUNDS) >= max(os.path.getmtime(src), os.path.getmtime(hdr)):
        return
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "--expt-relaxed-constexpr", "-DCCL_DEBUG_BOUNDS=1",
                    "-I" + os.path.join(root, "csrc"), "-I" + os.path.join(root, "csrc", "cuda", "kernels"), "-o", BOUNDS, src], check=True)


def test_checked_accessor_build_compiles():
    """The CCL_DEBUG_BOUNDS variant of the staging accessors builds for sm_100a (probe + the collective kernels)."""
    _build_bounds()
    root = os.path.dirname(os.path.dirname(HERE))
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "--expt-relaxed-constexpr", "-O1", "-DCCL_DEBUG_BOUNDS=1",
                    "-I" + os.path.join(root, "csrc"), "-I" + os.path.join(root, "csrc", "cuda", "kernels"), "-c",
                    os.path.join(root, "csrc", "cuda", "kernels", "moe_a2a.cu"), "-o", os.devnull], check=True)


@pytest.mark.gpu
def test_checked_accessors_skip_and_record_out_of_bounds():
    _build_bounds()
    r = subprocess.run([BOUNDS], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["ipc", "pingpong"])
def test_probe_runs(mode):
    _build()
    r = subprocess.run([BIN, mode], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout + r.stderr


PEER_BW = os.path.join(HERE, "peer_bw")


def _build_peer_bw():
    src = os.path.join(HERE, "peer_bw.cu")
    if os.path.exists(PEER_BW) and os.path.getmtime(PEER_BW) >= os.path.getmtime(src):
        return
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-lineinfo", "-o", PEER_BW, src], check=True)


def test_peer_bandwidth_probe_builds_for_sm100a():
    _build_peer_bw()
    assert os.access(PEER_BW, os.X_OK)


@pytest.mark.gpu
def test_peer_bandwidth_probe_runs():
    """16 MB copies, 2 launches each, load-flavour table only: a few seconds. With one GPU the probe says so and exits 0."""
    _build_peer_bw()
    r = subprocess.run([PEER_BW, "16", "2", "quick"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and ("done" in r.stdout or "skipped" in r.stdout), r.stdout + r.stderr


def _build_shm_stress(tag, flags):
    import torch

    out = os.path.join(HERE, "shm_stress_" + tag)
    root = os.path.dirname(os.path.dirname(HERE))
    srcs = [os.path.join(HERE, "shm_stress.cpp"), os.path.join(root, "csrc", "cpu", "ShmComm.cpp"),
            os.path.join(root, "csrc", "cpu", "CpuCollectives.cpp")]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(s) for s in srcs):
        return out
    inc = ["-I" + os.path.join(root, "csrc"), "-I" + os.path.join(os.path.dirname(torch.__file__), "include"),
           "-I/usr/local/cuda/include"]
    subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer"] + flags + inc + srcs + ["-o", out, "-lrt", "-lpthread"],
                   check=True)
    return out


@pytest.mark.parametrize("tag,flags", [("asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]),
                                       ("tsan", ["-fsanitize=thread"])])
def test_cpu_backend_under_sanitizers(tag, flags):
    """The shared-memory collectives and send/recv channels, ranks as threads, under ASan+UBSan and TSan."""
    exe = _build_shm_stress(tag, flags)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=1")
    r = subprocess.run([exe, "4", "12"], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    assert "ERROR: AddressSanitizer" not in r.stderr and "WARNING: ThreadSanitizer" not in r.stderr and "runtime error" not in r.stderr


def test_epoch_protocol_model_under_tsan():
    """Host-thread model of the flag / epoch / parity protocol: random programs of all_reduce,
    all_gather, broadcast and broadcast through the switch with slow ranks are race-free under
    ThreadSanitizer, and the same model without the broadcast release step shows the corruption
    that the step prevents."""
    src = os.path.join(HERE, "epoch_model.cpp")
    exe = os.path.join(HERE, "epoch_model_tsan")
    if not (os.path.exists(exe) and os.path.getmtime(exe) >= os.path.getmtime(src)):
        subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", src, "-o", exe, "-lpthread"], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "PASS" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    assert "ThreadSanitizer" not in r.stderr, r.stderr[-4000:]
    r = subprocess.run([exe, "norelease"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 3, "the model must detect the hazard when the release step is removed: " + r.stdout


def test_worker_thread_under_tsan():
    """The polling FIFO worker (csrc/pg/TaskThread.h): posts that land while it polls, while it goes to sleep and
    while it sleeps all run once and in order, race-free under ThreadSanitizer."""
    root = os.path.dirname(os.path.dirname(HERE))
    src = os.path.join(HERE, "task_thread_stress.cpp")
    hdr = os.path.join(root, "csrc", "pg", "TaskThread.h")
    exe = os.path.join(HERE, "task_thread_tsan")
    if not (os.path.exists(exe) and os.path.getmtime(exe) >= max(os.path.getmtime(src), os.path.getmtime(hdr))):
        subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-I" + os.path.join(root, "csrc"), src, "-o", exe, "-lpthread"],
                       check=True)
    for _ in range(3):
        r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and "PASS" in r.stdout and "ThreadSanitizer" not in r.stderr, r.stdout + r.stderr[-3000:]
