"""Python face of the CPU oracle (TEST INFRASTRUCTURE).

Loads the C restatement (``liblz_oracle.so``) and, where it was built, the
reference's own ``CPUPipe`` (``_ref/libref_cpupipe.so``), and runs them on
numpy arrays: the tower, the heads, the self-check distance and the weight
preparation steps.

Nothing in the product library may import this module; it is the checker.
Reference citations are paths inside the leela-zero source tree.
"""
import ctypes
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


def reference_root():
    """Where the leela-zero source tree lies: the LZ_REFERENCE environment
    variable, else the place this build environment mounts it."""
    return os.environ.get("LZ_REFERENCE", "/root/reference")


def build(ref_root=None):
    """Compile the checker libraries with the Makefile beside this file."""
    subprocess.run(["make", "-C", HERE, "REF=" + (ref_root or reference_root())], check=True,
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
# Weight preparation, restated (checks the package's loader-side math)
# --------------------------------------------------------------------------

def winograd_transform_f(f):
    """``f[K][C][3][3]`` -> ``U[36][C][K]`` by the C restatement, which keeps
    the reference's operation order (src/Network.cpp:159-223)."""
    f = np.ascontiguousarray(f, np.float32)
    K, C = f.shape[:2]
    U = np.empty((36, C, K), np.float32)
    port_lib().lzo_winograd_transform_f(_ptr(f), K, C, _ptr(U))
    return U


def process_bn_var(v):
    """var -> 1/sqrt(var + 1e-5) (src/Network.cpp:151-157)."""
    w = np.array(v, np.float32).ravel().copy()
    port_lib().lzo_process_bn_var(_ptr(w), w.size)
    return w


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
