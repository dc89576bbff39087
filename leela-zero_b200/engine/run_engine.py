"""Run the leela-zero engine on top of CUDAPipe (engine_bench) on a random-init
network and report NN evaluations/s, visits/s and the engine's own playouts/s.

    python leela-zero_b200/engine/run_engine.py --blocks 15 --filters 192 \
        --threads 8 --batch 8 --gpus 1 --visits 1600 --moves 50
    python leela-zero_b200/engine/run_engine.py --games 16 --threads 8 --batch 128 --moves 30

The binary is built by the Makefile beside this file from the engine's own
sources (only where the reference tree is present; the built binary is used
otherwise).
"""
import argparse
import importlib.util
import json
import os
import re
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
EXE = os.path.join(HERE, "_build", "engine_bench")
# the same engine with the reference's CPUPipe behind the scheduler: the checker of the engine tests
EXE_CHECK = os.path.join(HERE, "_build", "engine_check")


def _weights_module():
    spec = importlib.util.spec_from_file_location("lzb_weights", os.path.join(PKG, "weights.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def write_network(blocks, filters, seed, path):
    """Random-init network with calibrated batch-norm statistics, v1 text format."""
    W = _weights_module()
    raw = W.synthetic_raw_network(blocks, filters, seed)
    raw = W.calibrate_batchnorm(raw, W.synthetic_positions(4, seed + 1))
    W.write_v1(raw, path)


def run(blocks, filters, threads, batch, gpus, visits, moves, precision="auto", seed=2004,
        weights=None, verbose=True, timeout=600, games=1, batching="eager", cpu_only=False,
        selfchecks=0, deterministic=0, inject_half_init_failure=0, exe=None):
    """One engine_bench run; returns its summary line as a dict plus the moves
    the engine answered over GTP and the text it logged ("log").  precision:
    auto / single / half as the engine's --precision, or a mode name of the
    library; cpu_only runs the reference's own CPUPipe (the engine's --cpu-only);
    selfchecks forces that many of the engine's built-in GPU-against-CPU checks;
    deterministic is a tree-size limit in bytes that makes the game repeatable."""
    exe = exe or EXE
    if not os.path.exists(exe):
        raise RuntimeError("%s is missing: make -C %s (needs the reference tree)" % (exe, HERE))
    tmp = None
    if weights is None:
        tmp = tempfile.NamedTemporaryFile(suffix=".txt.gz", delete=False)
        tmp.close()
        weights = tmp.name
        write_network(blocks, filters, seed, weights)
    cmd = [exe, "--weights", weights, "--threads", str(threads), "--batch", str(batch), "--gpus",
           str(gpus), "--visits", str(visits), "--moves", str(moves), "--precision", precision,
           "--games", str(games), "--batching", batching]
    if cpu_only:
        cmd.append("--cpu-only")
    if selfchecks:
        cmd += ["--selfchecks", str(selfchecks)]
    if deterministic:
        cmd += ["--deterministic", str(deterministic)]
    if inject_half_init_failure:
        cmd += ["--inject-half-init-failure", str(inject_half_init_failure)]
    if verbose and games == 1:
        cmd.append("--verbose")
    env = dict(os.environ, OPENBLAS_NUM_THREADS="1")   # as the engine sets it (src/Network.cpp:498-499)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    if tmp is not None:
        os.unlink(weights)
    if r.returncode != 0:
        raise RuntimeError("engine_bench failed (%d): %s" % (r.returncode, r.stderr[-2000:]))
    summary = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    summary["log"] = r.stderr
    summary["gtp_moves"] = re.findall(r"^= (\S+)", r.stdout, flags=re.M)
    # the engine's own per-move line: "<visits> visits, <nodes> nodes, <playouts> playouts, <n/s> n/s"
    rates = [(int(a), int(b)) for a, b in re.findall(r"(\d+) playouts, (\d+) n/s", r.stderr)]
    if rates:
        summary["engine_playouts"] = sum(a for a, _ in rates)
        summary["engine_playouts_per_s_mean"] = sum(b for _, b in rates) / len(rates)
    return summary


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", type=int, default=15)
    ap.add_argument("--filters", type=int, default=192)
    ap.add_argument("--threads", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--visits", type=int, default=1600)
    ap.add_argument("--moves", type=int, default=50)
    ap.add_argument("--games", type=int, default=1,
                    help="games played at once in one process, sharing the pipe's queue")
    ap.add_argument("--batching", default="eager", choices=("eager", "wait"),
                    help="wait: the reference's full-batch-or-timeout rule; eager: take what is waiting")
    ap.add_argument("--precision", default="auto",
                    help="auto, single, half (the engine's own choices) or a mode name: fp32, fp16, fp16x2, bf16 ...")
    ap.add_argument("--cpu-only", action="store_true", help="the reference's CPUPipe instead of the GPU")
    ap.add_argument("--selfchecks", type=int, default=0)
    ap.add_argument("--deterministic", type=int, default=0, metavar="BYTES")
    ap.add_argument("--weights", default=None,
                    help="weights file to play with; if it does not exist yet, the random-init network "
                         "of --blocks x --filters is written there first (and kept)")
    a = ap.parse_args()
    if a.weights and not os.path.exists(a.weights):
        write_network(a.blocks, a.filters, 2004, a.weights)
    out = run(a.blocks, a.filters, a.threads, a.batch, a.gpus, a.visits, a.moves,
              a.precision, weights=a.weights, games=a.games, batching=a.batching,
              cpu_only=a.cpu_only, selfchecks=a.selfchecks, deterministic=a.deterministic)
    out.pop("log")
    print(json.dumps(out))
