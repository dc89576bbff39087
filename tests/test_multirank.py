"""The N > 1 form of the path: positions are sharded over ranks, every rank
holds the full network, nothing is exchanged on the data path; the process
group only provides a barrier and the max over ranks of the device times.
Exercised here with two gloo ranks on the CPU (the arithmetic each rank would
run on its GPU is replaced by a per-rank number), and with two GPUs inside one
process through CUDAPipe when two are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT

WORKER = r'''
import os, sys, json
sys.path.insert(0, %(root)r)
import torch, torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
W = bench.load_package().weights
x = W.synthetic_positions(4, bench.INPUT_SEED + rank)       # each rank draws its own shard
ms = 5.0 + 3.0 * rank                                        # rank 1 is the slow one
dist.barrier()
slowest = bench.max_over_ranks(ms, world)
raw = bench.calibrated_raw_network(W, 2, 16, 77, rank, world)   # calibrated on rank 0, handed over
out = {"rank": rank, "slowest": slowest, "value": bench.whole_job_rate(256, world, slowest),
       "checksum": float(x.sum()),
       "bn": [float(sum(float(m.sum()) for m in raw["bn_mean"])), float(sum(float(v.sum()) for v in raw["bn_var"])),
              float(raw["bn_val_mean"].sum())]}
gathered = [None] * world
dist.all_gather_object(gathered, out)
if rank == 0:
    print(json.dumps(gathered))
dist.barrier()
dist.destroy_process_group()
'''


def test_two_gloo_ranks_shard_and_take_the_slowest(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": ROOT})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    import json
    line = [l for l in r.stdout.splitlines() if l.startswith("[{")][-1]
    got = json.loads(line)
    assert [g["rank"] for g in got] == [0, 1]
    assert all(g["slowest"] == 8.0 for g in got)                    # max over ranks, on every rank
    assert all(abs(g["value"] - 2 * 256 / 8.0e-3) < 1e-6 for g in got)   # whole-job aggregate
    assert got[0]["bn"] == got[1]["bn"]                              # rank 1 got rank 0's calibration
    import bench
    W = bench.load_package().weights
    plain = W.synthetic_raw_network(2, 16, 77)
    assert got[0]["bn"][1] != float(sum(float(v.sum()) for v in plain["bn_var"]))   # and it is a calibrated one
    assert got[0]["checksum"] != got[1]["checksum"]                 # different shards


def test_reference_arm_runs_on_rank_zero_only():
    """`bench.py --impl reference` under a multi-rank launch: rank 1 leaves
    without work and without output."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


@pytest.mark.gpu
def test_cudapipe_spreads_batches_over_two_gpus(tmp_path, lzb, oracle):
    """One process, two replicas: CUDAPipe with gpus {0, 1}; every position
    gets the right answer whichever GPU served it."""
    if lzb.device_count() < 2:
        pytest.skip("needs two GPUs")
    import struct
    from test_scheduler import _compile
    W = lzb.weights
    net = W.synthetic_network(2, 64, 2071, calibrated=True)
    n = 128
    x = W.synthetic_positions(n, 1071).reshape(n, -1)
    blob = str(tmp_path / "net.bin")
    with open(blob, "wb") as f:
        f.write(struct.pack("7i", 64, 2, n, 32, 8, 2, 0))    # 32 threads, batch 8, 2 GPUs, fp32
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
    assert np.abs(got[:, :722] - pol).max() <= 1e-5 * scale
    assert np.abs(got[:, 722:] - val).max() <= 1e-5 * scale
