"""CUDAPipe (the C++ ForwardPipe implementation): scheduler behaviour on the
CPU with a fake backend, and the real thing on a GPU driven from many threads
like UCTSearch drives a ForwardPipe."""
import os
import shutil
import struct
import subprocess

import numpy as np
import pytest

from conftest import ROOT, reference_root

HOST = os.path.join(ROOT, "leela-zero_b200", "host")
CPP = os.path.join(ROOT, "tests", "cpp")
PKG = os.path.join(ROOT, "leela-zero_b200")


def _compile(src, out, extra=()):
    cmd = ["g++", "-std=c++14", "-O1", "-pthread", "-I" + os.path.join(ROOT, "include"), "-I" + HOST,
           os.path.join(CPP, src), os.path.join(HOST, "CUDAPipe.cpp"), "-L" + PKG, "-llzb200",
           "-Wl,-rpath," + PKG, "-o", out] + list(extra)
    subprocess.run(cmd, check=True)


def test_scheduler_with_fake_backend(tmp_path, lzb):
    """Batch forming, adaptive wait, partial batches, drain/resume, failure of
    one GPU, bad arguments: tests/cpp/test_cudapipe.cpp (behaviour of
    src/OpenCLScheduler.cpp:257-441)."""
    lzb.lib()   # the C-ABI library must exist to link against
    exe = str(tmp_path / "test_cudapipe")
    _compile("test_cudapipe.cpp", exe)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "ALL OK" in r.stdout, r.stdout + r.stderr


def test_scheduler_under_thread_sanitizer(tmp_path, lzb):
    lzb.lib()
    exe = str(tmp_path / "test_cudapipe_tsan")
    try:
        _compile("test_cudapipe.cpp", exe, ["-fsanitize=thread", "-g"])
    except subprocess.CalledProcessError:
        pytest.skip("ThreadSanitizer runtime not available")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert "WARNING: ThreadSanitizer" not in r.stderr, r.stderr[-3000:]
    assert r.returncode == 0 and "ALL OK" in r.stdout, r.stdout + r.stderr


def test_cudapipe_builds_against_the_reference_headers(tmp_path):
    """With LZ_REFERENCE_TREE the class derives from the engine's own
    ForwardPipe (drop-in check; only where the reference tree is present)."""
    ref = os.path.join(reference_root(), "src")
    if not os.path.exists(os.path.join(ref, "ForwardPipe.h")):
        pytest.skip("reference tree not present")
    out = str(tmp_path / "CUDAPipe.o")
    subprocess.run(["g++", "-std=c++14", "-c", "-DLZ_REFERENCE_TREE", "-DUSE_CPU_ONLY",
                    "-I" + ref, "-I" + os.path.join(ROOT, "include"), "-I" + HOST,
                    os.path.join(HOST, "CUDAPipe.cpp"), "-o", out], check=True)
    assert os.path.getsize(out) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("precision,threads,batch", [(0, 16, 8), (1, 48, 16)])
def test_cudapipe_on_gpu_from_many_threads(tmp_path, lzb, oracle, precision, threads, batch):
    """The real backend behind the virtual interface: 96 positions pushed by
    `threads` caller threads, compared per position with the oracle (fp32:
    1e-5 of the largest plane value; fp16: 1e-2 of it)."""
    W = lzb.weights
    net = W.synthetic_network(2, 64, 2070, calibrated=True)
    n = 96
    x = W.synthetic_positions(n, 1070).reshape(n, -1)
    blob = str(tmp_path / "net.bin")
    with open(blob, "wb") as f:
        f.write(struct.pack("7i", 64, 2, n, threads, batch, 1, precision))
        for l in range(5):
            f.write(net["U"][l].tobytes())
            f.write(net["bn_mean"][l].tobytes())
            f.write(net["bn_invstd"][l].tobytes())
        f.write(net["pol_w"].tobytes())
        f.write(net["val_w"].tobytes())
        f.write(np.ascontiguousarray(x, np.float32).tobytes())
    exe = str(tmp_path / "run_cudapipe_gpu")
    _compile("run_cudapipe_gpu.cpp", exe)
    outp = str(tmp_path / "out.bin")
    r = subprocess.run([exe, blob, outp], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(outp, np.float32).reshape(n, 1083)
    pol, val = oracle.cpu_pipe(net).forward(x)
    scale = max(np.abs(pol).max(), np.abs(val).max())
    rel = 1e-5 if precision == 0 else 1e-2
    assert np.abs(got[:, :722] - pol).max() <= rel * scale
    assert np.abs(got[:, 722:] - val).max() <= rel * scale
    assert "positions %d" % (n + 1) in r.stdout     # every request reached the backend exactly once


@pytest.mark.gpu
@pytest.mark.parametrize("precision,rel", [("fp32", 1e-5), ("fp16x2", 1e-2)])
def test_scheduler_blocks_of_positions_from_threads(lzb, oracle, precision, rel):
    """The C view of CUDAPipe (include/lzb200_sched.h): 8 threads hand in blocks
    of 1 to 40 positions (batch size 16, so large blocks are cut), every
    position compared with the CPU reference.  The positions are stone planes,
    so the batches travel to the GPU as bit planes; one block with a value that
    is neither 0 nor 1 takes the fp32 route and must agree too."""
    import threading
    W = lzb.weights
    net = W.synthetic_network(2, 64, 2071, calibrated=True)
    n = 8 * 61
    x = W.synthetic_positions(n, 1071).reshape(n, -1)
    x[5, 100] = 0.5
    pol_ref, val_ref = oracle.cpu_pipe(net).forward(x)
    sched = lzb.Scheduler(net, precision, gpus=(0,), batch_size=16, num_threads=32, eager=True)
    pol = np.empty((n, 2, 361), np.float32)
    val = np.empty((n, 361), np.float32)

    def caller(t):
        at = t * 61
        for size in (1, 40, 7, 13):
            pol[at:at + size], val[at:at + size] = sched.forward(x[at:at + size])
            at += size

    ts = [threading.Thread(target=caller, args=(t,)) for t in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    st = sched.stats()
    scale = max(np.abs(pol_ref).max(), np.abs(val_ref).max())
    assert np.abs(pol.reshape(n, -1) - pol_ref).max() <= rel * scale
    assert np.abs(val - val_ref).max() <= rel * scale
    assert st["positions"] == n and st["live_gpus"] == 1
    assert 0 < st["bit_plane_batches"] < st["batches"]
    sched.drain()
    with pytest.raises(lzb.SchedulerHalted):
        sched.forward(x[:2])
    sched.resume()
    p2, _ = sched.forward(x[:2])
    assert np.abs(p2 - pol[:2]).max() <= rel * scale
    sched.close()
