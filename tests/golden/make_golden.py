"""Generate the golden vectors in this folder.

Runs the reference's own CPUPipe (src/CPUPipe.cpp compiled unchanged by
oracle/Makefile into oracle/_ref/libref_cpupipe.so) on seeded synthetic
networks and positions and stores inputs' seeds and the outputs.  Networks and
positions are regenerated from their seeds by the package's weights module, so
the fixtures stay small.  Needs the reference tree; run from the repo root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

from conftest import load_package  # noqa: E402
import oracle as O  # noqa: E402

CASES = {
    # name: (blocks, filters, weight seed, calibrated, positions, position seed)
    "tiny_1x8": (1, 8, 2100, False, 3, 1100),
    "c0_6x64": (6, 64, 2001, False, 2, 1000),
    "c1_10x128": (10, 128, 2011, False, 2, 1001),
    "deep_20x256_cal": (20, 256, 2003, True, 1, 1002),
}


def main():
    assert O.ref_available(), "build oracle/_ref first (make -C oracle)"
    W = load_package().weights
    out = {}
    for name, (blocks, filters, wseed, cal, n, pseed) in CASES.items():
        net = W.synthetic_network(blocks, filters, wseed, calibrated=cal)
        x = W.synthetic_positions(n, pseed)
        pol, val = O.RefPipe(net).forward(x)
        policy, win = O.heads(net, pol, val)
        out[name + "/meta"] = np.array([blocks, filters, wseed, int(cal), n, pseed])
        out[name + "/pol"] = pol
        out[name + "/val"] = val
        out[name + "/policy"] = policy
        out[name + "/winrate"] = win
        # a checksum of the generated inputs guards against RNG drift
        out[name + "/input_sum"] = np.array([x.sum(), float(np.abs(net["U"][-1]).sum())])
        print(name, "winrate", win, "policy max", policy.max(1))
    np.savez_compressed(os.path.join(HERE, "cpupipe_golden.npz"), **out)


if __name__ == "__main__":
    main()
