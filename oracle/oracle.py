"""Python face of the CPU oracle (TEST INFRASTRUCTURE).

Loads the C restatement (``liblz_oracle.so``) and, where it was built, the
reference's own ``CPUPipe`` (``_ref/libref_cpupipe.so``); provides the seeded
synthetic positions and networks every parity test and the benchmark use, the
v1 text weight format, and the weight preparation ``Network::initialize``
performs before a pipe sees the weights.

Nothing in the product library may import this module; it is the checker.
Reference citations are paths inside the leela-zero source tree.
"""
import ctypes
import gzip
import os
import subprocess
import threading

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BOARD = 19
SQ = 361
INPUT_PLANES = 18
MOVES = 362
VALUE_HIDDEN = 256
SQ2 = np.float32(1.4142135623730951)

_f32p = ctypes.POINTER(ctypes.c_float)


def _ptr(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def build(ref_root="/root/reference"):
    """Compile the checker libraries with the Makefile beside this file."""
    subprocess.run(["make", "-C", HERE, "REF=" + ref_root], check=True,
                   stdout=subprocess.DEVNULL)


# --------------------------------------------------------------------------
# C restatement
# --------------------------------------------------------------------------

class _Tower(ctypes.Structure):
    _fields_ = [("channels", ctypes.c_int), ("blocks", ctypes.c_int),
                ("U", ctypes.POINTER(_f32p)), ("bn_mean", ctypes.POINTER(_f32p)),
                ("bn_invstd", ctypes.POINTER(_f32p)),
                ("pol_w", _f32p), ("val_w", _f32p)]


class _Heads(ctypes.Structure):
    _fields_ = [(n, _f32p) for n in (
        "bn_pol_mean", "bn_pol_invstd", "ip_pol_w", "ip_pol_b", "bn_val_mean",
        "bn_val_invstd", "ip1_val_w", "ip1_val_b", "ip2_val_w", "ip2_val_b")]
    _fields_.append(("softmax_temp", ctypes.c_float))


_port = None


def port_lib():
    global _port
    if _port is None:
        path = os.path.join(HERE, "liblz_oracle.so")
        if not os.path.exists(path):
            build()
        lib = ctypes.CDLL(path)
        lib.lzo_selfcheck_l2.restype = ctypes.c_float
        _port = lib
    return _port


def ref_available():
    return os.path.exists(os.path.join(HERE, "_ref", "libref_cpupipe.so"))


_ref = None


def ref_lib():
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(os.path.join(HERE, "_ref", "libref_cpupipe.so"))
        lib.ref_pipe_create.restype = ctypes.c_void_p
        lib.ref_pipe_create.argtypes = [ctypes.c_int, ctypes.c_int] + [_f32p] * 5
        lib.ref_pipe_forward.argtypes = [ctypes.c_void_p] + [_f32p] * 3
        lib.ref_pipe_destroy.argtypes = [ctypes.c_void_p]
        lib.ref_set_blas_threads(1)  # src/Network.cpp:498-499
        _ref = lib
    return _ref


# --------------------------------------------------------------------------
# Synthetic positions and networks
# --------------------------------------------------------------------------

def synthetic_positions(n, seed):
    """``[n][18][19][19]`` fp32 0/1 planes.

    Planes 0-7 own stones and 8-15 opponent stones per history step: each
    cell is occupied with probability 0.3, split evenly and without overlap.
    Planes 16/17: side to move, all-ones / all-zeros from one coin per
    position.  (Plane meaning: src/Network.cpp:935-966.)
    """
    rng = np.random.default_rng(seed)
    x = np.zeros((n, INPUT_PLANES, BOARD, BOARD), np.float32)
    u = rng.random((n, 8, BOARD, BOARD))
    x[:, 0:8] = (u < 0.15)
    x[:, 8:16] = (u >= 0.15) & (u < 0.30)
    coin = rng.random(n) < 0.5
    x[coin, 16] = 1.0
    x[~coin, 17] = 1.0
    return x


def synthetic_raw_network(blocks, channels, seed):
    """Random-init network in the shape of a v1 weights file (before any
    preparation): 3x3 convs He-normal, BN means N(0, 0.1), BN variances
    U(0.5, 1.5), conv biases 0, 1x1 convs and FC layers He-normal, FC biases 0.
    File order: src/Network.cpp:225-355."""
    rng = np.random.default_rng(seed)
    C = channels

    def normal(shape, sigma):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma))

    raw = {"blocks": blocks, "channels": C, "conv_w": [], "conv_b": [],
           "bn_mean": [], "bn_var": []}
    for l in range(1 + 2 * blocks):
        cin = INPUT_PLANES if l == 0 else C
        raw["conv_w"].append(normal((C, cin, 3, 3), np.sqrt(2.0 / (9 * cin))))
        raw["conv_b"].append(np.zeros(C, np.float32))
        raw["bn_mean"].append(normal((C,), 0.1))
        raw["bn_var"].append(rng.uniform(0.5, 1.5, C).astype(np.float32))
    raw["pol_w"] = normal((2, C), np.sqrt(2.0 / C))
    raw["pol_b"] = np.zeros(2, np.float32)
    raw["bn_pol_mean"] = normal((2,), 0.1)
    raw["bn_pol_var"] = rng.uniform(0.5, 1.5, 2).astype(np.float32)
    raw["ip_pol_w"] = normal((MOVES, 2 * SQ), np.sqrt(2.0 / (2 * SQ)))
    raw["ip_pol_b"] = np.zeros(MOVES, np.float32)
    raw["val_w"] = normal((1, C), np.sqrt(2.0 / C))
    raw["val_b"] = np.zeros(1, np.float32)
    raw["bn_val_mean"] = normal((1,), 0.1)
    raw["bn_val_var"] = rng.uniform(0.5, 1.5, 1).astype(np.float32)
    raw["ip1_val_w"] = normal((VALUE_HIDDEN, SQ), np.sqrt(2.0 / SQ))
    raw["ip1_val_b"] = np.zeros(VALUE_HIDDEN, np.float32)
    raw["ip2_val_w"] = normal((1, VALUE_HIDDEN), np.sqrt(2.0 / VALUE_HIDDEN))
    raw["ip2_val_b"] = np.zeros(1, np.float32)
    return raw


_HEAD_ORDER = ("pol_w", "pol_b", "bn_pol_mean", "bn_pol_var", "ip_pol_w",
               "ip_pol_b", "val_w", "val_b", "bn_val_mean", "bn_val_var",
               "ip1_val_w", "ip1_val_b", "ip2_val_w", "ip2_val_b")


def write_v1(raw, path):
    """Write the v1 text format: version line, 4 lines per conv layer, 14 head
    lines (src/Network.cpp:225-355; writer in training/tf/tfprocess.py:482-517)."""
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "wt") as f:
        f.write("1")
        rows = []
        for l in range(len(raw["conv_w"])):
            rows += [raw["conv_w"][l], raw["conv_b"][l], raw["bn_mean"][l],
                     raw["bn_var"][l]]
        rows += [raw[k] for k in _HEAD_ORDER]
        for r in rows:
            f.write("\n" + " ".join(repr(float(v)) for v in np.asarray(r).ravel()))


def read_v1(path):
    """Parse a v1/v2 text weights file the way ``Network::load_v1_network``
    does: blocks = (lines - 19) / 8, channels = token count of the third line
    (src/Network.cpp:243-259), gzip handled like gzopen (``:357-380``)."""
    with open(path, "rb") as f:
        magic = f.read(2)
    opener = gzip.open if magic == b"\x1f\x8b" else open
    with opener(path, "rt") as f:
        lines = f.read().split("\n")
    if lines and lines[-1] == "":
        lines.pop()
    version = int(lines[0])
    if version not in (1, 2):
        raise ValueError("Weights file is the wrong version.")
    body = lines[1:]
    residual_lines = len(body) - (4 + 14)
    if residual_lines < 0 or residual_lines % 8 != 0:
        raise ValueError("Inconsistent number of weights in the file.")
    blocks = residual_lines // 8
    channels = len(body[1].split())
    rows = [np.array(l.split(), dtype=np.float32) for l in body]
    raw = {"blocks": blocks, "channels": channels, "version": version,
           "conv_w": [], "conv_b": [], "bn_mean": [], "bn_var": []}
    nconv = 1 + 2 * blocks
    for l in range(nconv):
        cin = INPUT_PLANES if l == 0 else channels
        raw["conv_w"].append(rows[4 * l].reshape(channels, cin, 3, 3))
        raw["conv_b"].append(rows[4 * l + 1])
        raw["bn_mean"].append(rows[4 * l + 2])
        raw["bn_var"].append(rows[4 * l + 3])
    for i, k in enumerate(_HEAD_ORDER):
        raw[k] = rows[4 * nconv + i]
    if raw["ip_pol_w"].size != 2 * SQ * MOVES:
        raise ValueError("The weights file is not for 19x19 boards.")
    raw["pol_w"] = raw["pol_w"].reshape(2, channels)
    raw["val_w"] = raw["val_w"].reshape(1, channels)
    raw["ip_pol_w"] = raw["ip_pol_w"].reshape(MOVES, 2 * SQ)
    raw["ip1_val_w"] = raw["ip1_val_w"].reshape(VALUE_HIDDEN, SQ)
    raw["ip2_val_w"] = raw["ip2_val_w"].reshape(1, VALUE_HIDDEN)
    return raw


_G = np.array([[1.0, 0.0, 0.0],
               [-2.0 / 3.0, -SQ2 / 3.0, -1.0 / 3.0],
               [-2.0 / 3.0, SQ2 / 3.0, -1.0 / 3.0],
               [1.0 / 6.0, SQ2 / 6.0, 1.0 / 3.0],
               [1.0 / 6.0, -SQ2 / 6.0, 1.0 / 3.0],
               [0.0, 0.0, 1.0]], np.float32)


def winograd_transform_f(f, exact=None):
    """``f[K][C][3][3]`` -> ``U[36][C][K]`` (src/Network.cpp:159-223).

    ``exact=True`` runs the C restatement (same operation order as the
    reference); otherwise a vectorised numpy contraction whose results can
    differ from it in the last bit.  Small filters default to the exact path.
    """
    f = np.ascontiguousarray(f, np.float32)
    K, C = f.shape[:2]
    if exact is None:
        exact = f.size <= 9 * 64 * 64
    if exact:
        U = np.empty((36, C, K), np.float32)
        port_lib().lzo_winograd_transform_f(_ptr(f), K, C, _ptr(U))
        return U
    gf = np.einsum("ik,ockj->ocij", _G, f, dtype=np.float32)
    u = np.einsum("ocik,nk->inco", gf, _G, dtype=np.float32)
    return np.ascontiguousarray(u.reshape(36, C, K))


def prepare(raw, exact=None):
    """What ``Network::initialize`` does to a loaded file before a pipe sees
    it (src/Network.cpp:540-576): Winograd-transform every 3x3 filter,
    var -> 1/sqrt(var + 1e-5), fold conv biases into the BN means."""
    eps = np.float32(1e-5)

    def invstd(v):
        return (np.float32(1.0) / np.sqrt(np.asarray(v, np.float32) + eps)).astype(np.float32)

    net = {"blocks": raw["blocks"], "channels": raw["channels"]}
    net["U"] = [winograd_transform_f(w, exact) for w in raw["conv_w"]]
    net["bn_mean"] = [np.ascontiguousarray(m - b, np.float32)
                      for m, b in zip(raw["bn_mean"], raw["conv_b"])]
    net["bn_invstd"] = [invstd(v) for v in raw["bn_var"]]
    net["pol_w"] = np.ascontiguousarray(raw["pol_w"], np.float32)
    net["val_w"] = np.ascontiguousarray(raw["val_w"], np.float32)
    net["heads"] = {
        "bn_pol_mean": np.ascontiguousarray(raw["bn_pol_mean"] - raw["pol_b"], np.float32),
        "bn_pol_invstd": invstd(raw["bn_pol_var"]),
        "ip_pol_w": np.ascontiguousarray(raw["ip_pol_w"], np.float32),
        "ip_pol_b": np.ascontiguousarray(raw["ip_pol_b"], np.float32),
        "bn_val_mean": np.ascontiguousarray(raw["bn_val_mean"] - raw["val_b"], np.float32),
        "bn_val_invstd": invstd(raw["bn_val_var"]),
        "ip1_val_w": np.ascontiguousarray(raw["ip1_val_w"], np.float32),
        "ip1_val_b": np.ascontiguousarray(raw["ip1_val_b"], np.float32),
        "ip2_val_w": np.ascontiguousarray(raw["ip2_val_w"], np.float32).reshape(-1),
        "ip2_val_b": np.ascontiguousarray(raw["ip2_val_b"], np.float32),
    }
    return net


def synthetic_network(blocks, channels, seed, exact=None):
    return prepare(synthetic_raw_network(blocks, channels, seed), exact)


# --------------------------------------------------------------------------
# Running the checkers
# --------------------------------------------------------------------------

class PortPipe:
    """The C restatement of ``CPUPipe::forward`` (one position per call)."""

    def __init__(self, net):
        self.net = net
        L = len(net["U"])
        arr = _f32p * L
        self._keep = (arr(*[_ptr(u) for u in net["U"]]),
                      arr(*[_ptr(m) for m in net["bn_mean"]]),
                      arr(*[_ptr(s) for s in net["bn_invstd"]]))
        self.t = _Tower(net["channels"], net["blocks"], self._keep[0],
                        self._keep[1], self._keep[2], _ptr(net["pol_w"]),
                        _ptr(net["val_w"]))

    def forward(self, x):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, INPUT_PLANES * SQ)
        pol = np.empty((x.shape[0], 2 * SQ), np.float32)
        val = np.empty((x.shape[0], SQ), np.float32)
        lib = port_lib()
        for i in range(x.shape[0]):
            lib.lzo_forward(ctypes.byref(self.t), _ptr(x[i]), _ptr(pol[i]), _ptr(val[i]))
        return pol, val


class RefPipe:
    """The reference's own ``CPUPipe`` behind its ``ForwardPipe`` interface."""

    def __init__(self, net):
        lib = ref_lib()
        U = np.concatenate([u.ravel() for u in net["U"]])
        mean = np.concatenate(net["bn_mean"])
        inv = np.concatenate(net["bn_invstd"])
        self.h = lib.ref_pipe_create(net["channels"], net["blocks"], _ptr(U),
                                     _ptr(mean), _ptr(inv), _ptr(net["pol_w"]),
                                     _ptr(net["val_w"]))

    def forward(self, x, threads=1):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, INPUT_PLANES * SQ)
        n = x.shape[0]
        pol = np.empty((n, 2 * SQ), np.float32)
        val = np.empty((n, SQ), np.float32)
        lib = ref_lib()

        def work(lo, hi):
            for i in range(lo, hi):
                lib.ref_pipe_forward(self.h, _ptr(x[i]), _ptr(pol[i]), _ptr(val[i]))

        if threads <= 1 or n == 1:
            work(0, n)
        else:
            # T host threads, each looping forward over its own positions,
            # like Network::benchmark (src/Network.cpp:128-149).
            bounds = np.linspace(0, n, threads + 1).astype(int)
            ts = [threading.Thread(target=work, args=(bounds[i], bounds[i + 1]))
                  for i in range(threads)]
            [t.start() for t in ts]
            [t.join() for t in ts]
        return pol, val

    def close(self):
        if self.h:
            ref_lib().ref_pipe_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def cpu_pipe(net):
    """The reference CPUPipe where it was built, else the C restatement."""
    return RefPipe(net) if ref_available() else PortPipe(net)


def heads(net, pol, val, softmax_temp=1.0):
    """Raw head planes ``pol[n][722]``, ``val[n][361]`` -> ``policy[n][362]``
    (softmax) and ``winrate[n]`` (src/Network.cpp:833-851)."""
    h = net["heads"]
    hw = _Heads(*[_ptr(h[k]) for k in (
        "bn_pol_mean", "bn_pol_invstd", "ip_pol_w", "ip_pol_b", "bn_val_mean",
        "bn_val_invstd", "ip1_val_w", "ip1_val_b", "ip2_val_w", "ip2_val_b")],
        softmax_temp)
    pol = np.array(pol, np.float32).reshape(-1, 2 * SQ)
    val = np.array(val, np.float32).reshape(-1, SQ)
    n = pol.shape[0]
    policy = np.empty((n, MOVES), np.float32)
    win = np.empty(n, np.float32)
    lib = port_lib()
    w1 = ctypes.c_float()
    for i in range(n):
        lib.lzo_heads(ctypes.byref(hw), _ptr(pol[i]), _ptr(val[i]), _ptr(policy[i]),
                      ctypes.byref(w1))
        win[i] = w1.value
    return policy, win


def selfcheck_l2(policy_a, win_a, policy_b, win_b):
    """src/Network.cpp:667-690."""
    a = np.ascontiguousarray(policy_a, np.float32)
    b = np.ascontiguousarray(policy_b, np.float32)
    return float(port_lib().lzo_selfcheck_l2(_ptr(a), ctypes.c_float(win_a),
                                             _ptr(b), ctypes.c_float(win_b)))
