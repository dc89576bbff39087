"""lzb_conv3x3_static: the entry point for callers that cannot allocate device
memory (hosts that own all of it through their own pool, threads that must not
take cudaMalloc's device-wide synchronisation).  It keeps its working memory in
a fixed array inside the library, so this test checks four things through the
C ABI: that it agrees with the allocating entry point (lzb_ctx_debug_conv of an
fp32 pipe) on the same layer, that both agree with the CPU restatement of the
reference's layer (the checker the other parity tests use), that a second call
right after the first is not disturbed by what the first left in the shared
array (the second call is smaller and uses other channel counts), and that
sizes beyond the stated limits are refused.  Tolerance: 2e-6 of the largest
output, the bound the single-layer fp32 tests use.

This file is collected last on purpose: a run that stops at the first failure
has then already run every other test."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL = 2e-6


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()


def _static_layer(lzb, net, layer, x, residual=None):
    """Run one layer through lzb_conv3x3_static with device buffers that the
    test (not the library) owns."""
    import torch
    U = net["U"][layer]
    c_in, channels = U.shape[1], U.shape[2]
    n = x.shape[0]
    d_in, d_U = _dev(x.reshape(n, c_in, 361)), _dev(U)
    d_mean, d_inv = _dev(net["bn_mean"][layer]), _dev(net["bn_invstd"][layer])
    d_res = None if residual is None else _dev(residual)
    d_out = torch.full((n, channels, 361), float("nan"), device="cuda")
    torch.cuda.synchronize()
    rc = lzb.lib().lzb_conv3x3_static(
        0, d_in.data_ptr(), n, c_in, channels, d_U.data_ptr(), d_mean.data_ptr(), d_inv.data_ptr(),
        None if d_res is None else d_res.data_ptr(), d_out.data_ptr(), None)
    lzb.check(rc)
    torch.cuda.synchronize()
    return d_out.cpu().numpy()


def _cpu_layer(oracle, net, layer, x, res=None):
    """The layer on the CPU: input transform, 36 contractions, output
    transform, batch-norm [+ residual] + ReLU, stage by stage as CPUPipe runs
    them (src/CPUPipe.cpp:63-284, 352-377)."""
    lib = oracle.port_lib()
    U = net["U"][layer]
    cin, C = U.shape[1], U.shape[2]
    out = np.empty((x.shape[0], C, 361), np.float32)
    V = np.empty((36, cin, 25), np.float32)
    M = np.empty((36, C, 25), np.float32)
    for i in range(x.shape[0]):
        xi = np.ascontiguousarray(x[i].reshape(cin, 361))
        lib.lzo_transform_in(oracle._ptr(xi), oracle._ptr(V), cin)
        lib.lzo_sgemm36(oracle._ptr(U), oracle._ptr(V), oracle._ptr(M), cin, C)
        lib.lzo_transform_out(oracle._ptr(M), oracle._ptr(out[i]), C)
        r = None if res is None else oracle._ptr(np.ascontiguousarray(res[i]))
        lib.lzo_batchnorm(C, 361, oracle._ptr(out[i]), oracle._ptr(net["bn_mean"][layer]),
                          oracle._ptr(net["bn_invstd"][layer]), r)
    return out


def test_static_entry_point_matches_allocating_one(lzb, oracle):
    W = lzb.weights
    net = W.synthetic_network(1, 64, 4000)
    small = W.synthetic_network(1, 24, 4001)
    pipe, pipe_small = lzb.Pipe(net, "fp32"), lzb.Pipe(small, "fp32")
    ctx, ctx_small = pipe.context(8), pipe_small.context(8)

    # call 1: the largest supported case, a residual layer (64 -> 64 channels, 8 positions)
    x8 = W.synthetic_positions(8, 4100)
    a0 = ctx.debug_conv(0, x8)
    a1 = ctx.debug_conv(1, a0)
    want = ctx.debug_conv(2, a1, a0)
    got = _static_layer(lzb, net, 2, a1, a0)
    assert np.abs(got - want).max() <= REL * max(1.0, np.abs(want).max())
    cpu = _cpu_layer(oracle, net, 2, a1, a0)
    assert np.abs(got - cpu).max() <= REL * max(1.0, np.abs(cpu).max())

    # call 2, straight after: fewer positions, 18 -> 24 channels, no residual;
    # the array still holds call 1's tiles, weights and batch-norm vectors
    x2 = W.synthetic_positions(2, 4101)
    want2 = ctx_small.debug_conv(0, x2)
    got2 = _static_layer(lzb, small, 0, x2)
    assert np.abs(got2 - want2).max() <= REL * max(1.0, np.abs(want2).max())
    cpu2 = _cpu_layer(oracle, small, 0, x2)
    assert np.abs(got2 - cpu2).max() <= REL * max(1.0, np.abs(cpu2).max())

    # and once more the first case, to see that call 2 left nothing behind either
    got3 = _static_layer(lzb, net, 2, a1, a0)
    assert np.array_equal(got3, got)


def test_static_entry_point_refuses_sizes_beyond_its_limits(lzb):
    import torch
    buf = torch.zeros(1 << 20, device="cuda")
    p = buf.data_ptr()
    L = lzb.lib()
    assert L.lzb_conv3x3_static(0, p, 9, 18, 64, p, p, p, None, p, None) == 1      # 9 positions
    assert b"positions" in L.lzb_last_error()
    assert L.lzb_conv3x3_static(0, p, 1, 18, 65, p, p, p, None, p, None) == 1      # 65 filters
    assert b"channels" in L.lzb_last_error()
    assert L.lzb_conv3x3_static(0, p, 1, 128, 64, p, p, p, None, p, None) == 1     # 128 inputs
    assert L.lzb_conv3x3_static(0, None, 1, 18, 64, p, p, p, None, p, None) == 1   # null input
