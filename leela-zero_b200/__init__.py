"""Python binding of the lzb200 C ABI (``include/lzb200.h``).

The arithmetic lives in ``liblzb200.so`` (hand-written sm_100a CUDA); this
module only marshals numpy arrays through ctypes, the way a cgo/JNI stub would.
There is no fallback: if the library is missing or no B200 is visible, calls
raise.
"""
import ctypes
import os

import numpy as np

from . import weights  # noqa: F401  (loader, preparation, synthetic data)

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblzb200.so")

FP32, FP16, BF16, FP16_WINOGRAD, BF16_WINOGRAD = 0, 1, 2, 3, 4
FP16_X2, FP16_X3, BF16_X3 = 5, 6, 7
PRECISIONS = {"fp32": FP32, "fp16": FP16, "bf16": BF16, "fp16-winograd": FP16_WINOGRAD,
              "bf16-winograd": BF16_WINOGRAD, "fp16x2": FP16_X2, "fp16x3": FP16_X3,
              "bf16x3": BF16_X3}
IN_FLOATS, POL_FLOATS, VAL_FLOATS, MOVES = 18 * 361, 2 * 361, 361, 362

# every symbol include/lzb200.h declares
SYMBOLS = (
    "lzb_last_error", "lzb_device_count", "lzb_pipe_create", "lzb_pipe_destroy",
    "lzb_pipe_push_conv", "lzb_pipe_push_head_convs", "lzb_pipe_push_heads",
    "lzb_pipe_finalize", "lzb_ctx_create", "lzb_ctx_destroy", "lzb_ctx_forward",
    "lzb_ctx_forward_device", "lzb_ctx_forward_heads", "lzb_ctx_forward_heads_device",
    "lzb_ctx_sync", "lzb_ctx_stream", "lzb_ctx_set_micro_batch", "lzb_ctx_launch_count",
    "lzb_ctx_debug_conv", "lzb_ctx_profile_begin", "lzb_ctx_profile_end",
    "lzb_conv3x3_static", "lzb_ctx_debug_wait_probe", "lzb_host_alloc", "lzb_host_free",
    "lzb_pipe_push_conv_filters", "lzb_ctx_forward_packed", "lzb_ctx_forward_heads_packed",
    "lzb_pipe_set_low_plane_blocks", "lzb_ctx_micro_batch",
)

_f32p = ctypes.POINTER(ctypes.c_float)
_lib = None


class LzbError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("lzb200 error %d: %s" % (code, text))
        self.code = code


def lib():
    """Load liblzb200.so (raises if it was not built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: run `python leela-zero_b200/build.py`" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        L.lzb_last_error.restype = ctypes.c_char_p
        L.lzb_ctx_stream.restype = ctypes.c_void_p
        L.lzb_ctx_launch_count.restype = ctypes.c_longlong
        vp = ctypes.c_void_p
        L.lzb_pipe_create.argtypes = [ctypes.POINTER(vp)] + [ctypes.c_int] * 4
        L.lzb_pipe_destroy.argtypes = [vp]
        L.lzb_pipe_set_low_plane_blocks.argtypes = [vp, ctypes.c_int, ctypes.c_int]
        L.lzb_pipe_push_conv.argtypes = [vp, ctypes.c_int, _f32p, ctypes.c_int, _f32p, _f32p]
        L.lzb_pipe_push_head_convs.argtypes = [vp, _f32p, _f32p]
        L.lzb_pipe_push_heads.argtypes = [vp] + [_f32p] * 10
        L.lzb_pipe_finalize.argtypes = [vp]
        L.lzb_ctx_create.argtypes = [ctypes.POINTER(vp), vp, ctypes.c_int]
        L.lzb_ctx_destroy.argtypes = [vp]
        L.lzb_ctx_forward.argtypes = [vp, vp, ctypes.c_int, vp, vp]
        L.lzb_ctx_forward_device.argtypes = [vp, vp, ctypes.c_int, vp, vp]
        L.lzb_ctx_forward_heads.argtypes = [vp, vp, ctypes.c_int, ctypes.c_float, vp, vp]
        L.lzb_ctx_forward_heads_device.argtypes = [vp, vp, ctypes.c_int, ctypes.c_float, vp, vp]
        L.lzb_ctx_sync.argtypes = [vp]
        L.lzb_ctx_stream.argtypes = [vp]
        L.lzb_ctx_set_micro_batch.argtypes = [vp, ctypes.c_int]
        L.lzb_ctx_micro_batch.argtypes = [vp]
        L.lzb_ctx_launch_count.argtypes = [vp]
        L.lzb_ctx_debug_conv.argtypes = [vp, ctypes.c_int, _f32p, ctypes.c_int, _f32p, _f32p]
        L.lzb_ctx_profile_begin.argtypes = [vp]
        L.lzb_ctx_profile_end.argtypes = [vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_longlong)]
        L.lzb_pipe_push_conv_filters.argtypes = [vp, ctypes.c_int, _f32p, ctypes.c_int, _f32p, _f32p]
        L.lzb_ctx_forward_packed.argtypes = [vp, vp, ctypes.c_int, vp, vp]
        L.lzb_ctx_forward_heads_packed.argtypes = [vp, vp, ctypes.c_int, ctypes.c_float, vp, vp]
        L.lzb_host_alloc.argtypes = [ctypes.POINTER(vp), ctypes.c_size_t]
        L.lzb_host_free.argtypes = [vp]
        L.lzb_host_free.restype = None
        L.lzb_ctx_debug_wait_probe.argtypes = [vp, ctypes.c_int]
        L.lzb_conv3x3_static.argtypes = [ctypes.c_int, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                         vp, vp, vp, vp, vp, vp]
        _lib = L
    return _lib


def check(code):
    if code != 0:
        raise LzbError(code, lib().lzb_last_error().decode())


def _ptr(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def pack_positions(x):
    """0/1 planes ``[n][18][19][19]`` -> ``[n][18][12]`` uint32, bit i of word w of a
    plane = board cell 32 w + i (the layout lzb_ctx_forward_packed takes)."""
    x = np.asarray(x).reshape(-1, 18, 361)
    bits = np.zeros((x.shape[0], 18, 384), np.uint8)
    bits[:, :, :361] = x != 0
    words = np.packbits(bits.reshape(-1, 18, 12, 32), axis=-1, bitorder="little")
    return np.ascontiguousarray(words).view(np.uint32).reshape(-1, 18, 12)


def device_count():
    n = ctypes.c_int(0)
    check(lib().lzb_device_count(ctypes.byref(n)))
    return n.value


class Pipe:
    """A network resident on one GPU (``lzb_pipe``).

    ``net`` is a dict with the arrays a ``ForwardPipe`` receives in
    ``push_weights`` (src/ForwardPipe.h:40-54): ``U`` (list of fp32
    ``[36][c_in][C]``), ``bn_mean``, ``bn_invstd`` (lists of ``[C]``),
    ``pol_w`` ``[2][C]``, ``val_w`` ``[1][C]``, plus optionally ``heads``.
    ``low_plane_blocks`` (``"fp16x2"`` only) overrides how many residual blocks carry
    the e5m2 plane of the activations, ``weight_blocks`` how many of them also
    correct their weights.  With ``from_filters`` the layers come from ``net["filters"]`` (untransformed
    ``[C][c_in][3][3]``, as ``weights.load_network`` returns them) instead of ``U``.
    """

    def __init__(self, net, precision="fp16", device=0, heads=True, from_filters=False,
                 low_plane_blocks=None, weight_blocks=None):
        L = lib()
        self.h = ctypes.c_void_p()
        self.channels, self.blocks = net["channels"], net["blocks"]
        self.precision = PRECISIONS[precision] if isinstance(precision, str) else precision
        check(L.lzb_pipe_create(ctypes.byref(self.h), device, self.channels, self.blocks,
                                self.precision))
        if low_plane_blocks is not None:     # fp16x2: blocks that carry the e5m2 planes (-1 = all)
            check(L.lzb_pipe_set_low_plane_blocks(self.h, low_plane_blocks,
                                                  4 if weight_blocks is None else weight_blocks))
        for l in range(len(net["bn_mean"])):
            mean = _ptr(np.ascontiguousarray(net["bn_mean"][l], np.float32))
            inv = _ptr(np.ascontiguousarray(net["bn_invstd"][l], np.float32))
            if from_filters:      # untransformed filters [K][c_in][3][3], as in a weights file
                f = np.ascontiguousarray(net["filters"][l], np.float32)
                check(L.lzb_pipe_push_conv_filters(self.h, l, _ptr(f), f.shape[1], mean, inv))
            else:                 # Winograd-transformed, as the engine hands them to a pipe
                U = np.ascontiguousarray(net["U"][l], np.float32)
                check(L.lzb_pipe_push_conv(self.h, l, _ptr(U), U.shape[1], mean, inv))
        check(L.lzb_pipe_push_head_convs(self.h, _ptr(np.ascontiguousarray(net["pol_w"], np.float32)),
                                         _ptr(np.ascontiguousarray(net["val_w"], np.float32))))
        self.has_heads = bool(heads and "heads" in net)
        if self.has_heads:
            hw = net["heads"]
            keys = ("bn_pol_mean", "bn_pol_invstd", "ip_pol_w", "ip_pol_b", "bn_val_mean",
                    "bn_val_invstd", "ip1_val_w", "ip1_val_b", "ip2_val_w", "ip2_val_b")
            arrs = [np.ascontiguousarray(hw[k], np.float32) for k in keys]
            check(L.lzb_pipe_push_heads(self.h, *[_ptr(a) for a in arrs]))
        check(L.lzb_pipe_finalize(self.h))

    def context(self, max_batch):
        return Context(self, max_batch)

    def close(self):
        if self.h:
            lib().lzb_pipe_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Context:
    """Stream + activation buffers on a pipe (``lzb_ctx``)."""

    def __init__(self, pipe, max_batch):
        self.pipe = pipe
        self.max_batch = max_batch
        self.h = ctypes.c_void_p()
        check(lib().lzb_ctx_create(ctypes.byref(self.h), pipe.h, max_batch))

    def forward(self, x):
        """Host ``[n][18][19][19]`` fp32 -> raw head planes ``pol[n][722]``, ``val[n][361]``."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, IN_FLOATS)
        n = x.shape[0]
        pol = np.empty((n, POL_FLOATS), np.float32)
        val = np.empty((n, VAL_FLOATS), np.float32)
        check(lib().lzb_ctx_forward(self.h, x.ctypes.data, n, pol.ctypes.data, val.ctypes.data))
        return pol, val

    def forward_heads(self, x, softmax_temp=1.0):
        """Host positions -> ``policy[n][362]`` (softmax) and ``winrate[n]``."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, IN_FLOATS)
        n = x.shape[0]
        policy = np.empty((n, MOVES), np.float32)
        win = np.empty(n, np.float32)
        check(lib().lzb_ctx_forward_heads(self.h, x.ctypes.data, n, softmax_temp,
                                          policy.ctypes.data, win.ctypes.data))
        return policy, win

    def forward_packed(self, packed):
        """Bit-packed positions ``[n][18][12]`` uint32 (see :func:`pack_positions`)."""
        packed = np.ascontiguousarray(packed, np.uint32).reshape(-1, 18 * 12)
        n = packed.shape[0]
        pol = np.empty((n, POL_FLOATS), np.float32)
        val = np.empty((n, VAL_FLOATS), np.float32)
        check(lib().lzb_ctx_forward_packed(self.h, packed.ctypes.data, n, pol.ctypes.data,
                                           val.ctypes.data))
        return pol, val

    def forward_heads_packed(self, packed, softmax_temp=1.0):
        packed = np.ascontiguousarray(packed, np.uint32).reshape(-1, 18 * 12)
        n = packed.shape[0]
        policy = np.empty((n, MOVES), np.float32)
        win = np.empty(n, np.float32)
        check(lib().lzb_ctx_forward_heads_packed(self.h, packed.ctypes.data, n, softmax_temp,
                                                 policy.ctypes.data, win.ctypes.data))
        return policy, win

    def forward_ptr(self, in_ptr, n, pol_ptr, val_ptr):
        """Raw host pointers (e.g. pinned buffers); blocking."""
        check(lib().lzb_ctx_forward(self.h, in_ptr, n, pol_ptr, val_ptr))

    def forward_heads_ptr(self, in_ptr, n, temp, policy_ptr, win_ptr):
        check(lib().lzb_ctx_forward_heads(self.h, in_ptr, n, temp, policy_ptr, win_ptr))

    def forward_heads_packed_ptr(self, packed_ptr, n, temp, policy_ptr, win_ptr):
        """Bit-packed positions and results at raw host pointers (pinned buffers); blocking."""
        check(lib().lzb_ctx_forward_heads_packed(self.h, packed_ptr, n, temp, policy_ptr, win_ptr))

    def forward_device(self, in_dev, n, pol_dev, val_dev):
        """Device pointers, enqueued on the context's stream; no wait."""
        check(lib().lzb_ctx_forward_device(self.h, in_dev, n, pol_dev, val_dev))

    def forward_heads_device(self, in_dev, n, temp, policy_dev, win_dev):
        check(lib().lzb_ctx_forward_heads_device(self.h, in_dev, n, temp, policy_dev, win_dev))

    def sync(self):
        check(lib().lzb_ctx_sync(self.h))

    @property
    def stream(self):
        return lib().lzb_ctx_stream(self.h)

    def set_micro_batch(self, n):
        check(lib().lzb_ctx_set_micro_batch(self.h, n))

    @property
    def micro_batch(self):
        """Positions per pass through the tower (the library's choice unless set)."""
        return lib().lzb_ctx_micro_batch(self.h)

    @property
    def launches(self):
        return lib().lzb_ctx_launch_count(self.h)

    def profile_begin(self):
        check(lib().lzb_ctx_profile_begin(self.h))

    def profile_end(self):
        """-> {class name: (milliseconds, launches)} since profile_begin."""
        ms = (ctypes.c_double * 4)()
        cnt = (ctypes.c_longlong * 4)()
        check(lib().lzb_ctx_profile_end(self.h, ms, cnt))
        names = ("contraction", "transform", "input", "head")
        return {k: (ms[i], cnt[i]) for i, k in enumerate(names)}

    def debug_wait_probe(self, limit_ms=50):
        """Enqueue a bounded wait that runs out (see lzb_ctx_debug_wait_probe)."""
        check(lib().lzb_ctx_debug_wait_probe(self.h, limit_ms))

    def debug_conv(self, layer, x, residual=None):
        """One 3x3 layer on fp32 NCHW host data (diagnostics)."""
        x = np.ascontiguousarray(x, np.float32)
        n = x.shape[0]
        out = np.empty((n, self.pipe.channels, 361), np.float32)
        r = None if residual is None else _ptr(np.ascontiguousarray(residual, np.float32))
        check(lib().lzb_ctx_debug_conv(self.h, layer, _ptr(x), n, r, _ptr(out)))
        return out

    def close(self):
        if self.h:
            lib().lzb_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---------------------------------------------------------------------------
# The batching scheduler (C++ CUDAPipe) through its C view, include/lzb200_sched.h
# ---------------------------------------------------------------------------

SCHED_LIB_PATH = os.path.join(HERE, "libcudapipe.so")
SCHED_SYMBOLS = (
    "lzb_sched_last_error", "lzb_sched_create", "lzb_sched_destroy", "lzb_sched_add_conv",
    "lzb_sched_start", "lzb_sched_forward", "lzb_sched_drain", "lzb_sched_resume", "lzb_sched_stats",
)
_sched_lib = None


class SchedulerHalted(RuntimeError):
    """The pipe is draining (NetworkHaltException in the C++ class)."""


def sched_lib():
    """Load libcudapipe.so (raises if it was not built)."""
    global _sched_lib
    if _sched_lib is None:
        if not os.path.exists(SCHED_LIB_PATH):
            raise RuntimeError("%s is missing: run `python leela-zero_b200/build.py`" % SCHED_LIB_PATH)
        lib()   # liblzb200.so first: libcudapipe.so links against it
        L = ctypes.CDLL(SCHED_LIB_PATH)
        vp = ctypes.c_void_p
        L.lzb_sched_last_error.restype = ctypes.c_char_p
        L.lzb_sched_create.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(ctypes.c_int)] + [ctypes.c_int] * 5
        L.lzb_sched_destroy.argtypes = [vp]
        L.lzb_sched_destroy.restype = None
        L.lzb_sched_add_conv.argtypes = [vp, _f32p, ctypes.c_int, ctypes.c_int, _f32p, _f32p]
        L.lzb_sched_start.argtypes = [vp, ctypes.c_int, _f32p, _f32p]
        L.lzb_sched_forward.argtypes = [vp, vp, ctypes.c_int, vp, vp]
        L.lzb_sched_drain.argtypes = [vp]
        L.lzb_sched_resume.argtypes = [vp]
        L.lzb_sched_stats.argtypes = [vp, ctypes.POINTER(ctypes.c_ulonglong)]
        _sched_lib = L
    return _sched_lib


class Scheduler:
    """CUDAPipe: one queue in front of a network replica on each of ``gpus``.

    ``forward(x)`` blocks until its positions are evaluated and may be called
    from any number of threads; positions of different callers share batches.
    Returns the raw 1x1 head planes ``pol[n][2][361]``, ``val[n][361]`` like
    ``ForwardPipe::forward``."""

    def __init__(self, net, precision="fp16x2", gpus=(0,), batch_size=256, num_threads=64, eager=True):
        L = sched_lib()
        self._h = ctypes.c_void_p()
        ids = (ctypes.c_int * len(gpus))(*gpus)
        self._check(L.lzb_sched_create(ctypes.byref(self._h), ids, len(gpus), batch_size, num_threads,
                                       PRECISIONS[precision], 1 if eager else 0))
        channels = int(net["U"][0].shape[2])
        for U, mean, inv in zip(net["U"], net["bn_mean"], net["bn_invstd"]):
            U = np.ascontiguousarray(U, np.float32)
            self._check(L.lzb_sched_add_conv(self._h, _ptr(U), U.shape[1], U.shape[2],
                                             _ptr(np.ascontiguousarray(mean, np.float32)),
                                             _ptr(np.ascontiguousarray(inv, np.float32))))
        self._check(L.lzb_sched_start(self._h, channels,
                                      _ptr(np.ascontiguousarray(net["pol_w"], np.float32)),
                                      _ptr(np.ascontiguousarray(net["val_w"], np.float32))))

    @staticmethod
    def _check(code):
        if code == 2:
            raise SchedulerHalted(sched_lib().lzb_sched_last_error().decode())
        if code != 0:
            raise RuntimeError("CUDAPipe: " + sched_lib().lzb_sched_last_error().decode())

    def forward(self, x, pol=None, val=None):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, IN_FLOATS)
        n = x.shape[0]
        pol = np.empty((n, 2, 361), np.float32) if pol is None else pol
        val = np.empty((n, 361), np.float32) if val is None else val
        self._check(sched_lib().lzb_sched_forward(self._h, x.ctypes.data, n, pol.ctypes.data, val.ctypes.data))
        return pol, val

    def drain(self):
        self._check(sched_lib().lzb_sched_drain(self._h))

    def resume(self):
        self._check(sched_lib().lzb_sched_resume(self._h))

    def stats(self):
        out = (ctypes.c_ulonglong * 8)()
        self._check(sched_lib().lzb_sched_stats(self._h, out))
        keys = ("batches", "positions", "full_batches", "timeouts", "bit_plane_batches", "halted",
                "live_gpus", "wait_ms")
        return dict(zip(keys, (int(v) for v in out)))

    def close(self):
        if self._h:
            sched_lib().lzb_sched_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
