"""GPU parity tests: the CUDA pipe, called through the C ABI, against the CPU
oracle (the reference's own CPUPipe where it was built, else the C
restatement) on the same seeded inputs and weights.

Tolerances (max-abs after the heads, i.e. on policy[362] and winrate):
  fp32 mode                 policy <= 1e-4, winrate <= 1e-4
  fp16 / bf16 operand modes policy <= 2e-3, winrate <= 5e-3
and the engine's self-check distance (src/Network.cpp:667-690) <= 0.2.

"fp16x2" (fp16 activations with an e5m2 correction plane) is the mode the
benchmark is quoted on and the one held to these bounds as max-abs over every
position of every configuration.  Plain "fp16" is the fast mode: it misses the
winrate bound on a few per cent of the positions of deep networks, and the
tests that touch it say which bound they characterise it by.
"""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-4
TOL_POLICY_16 = 2e-3
TOL_VALUE_16 = 5e-3
SELFCHECK_MAX = 0.2


@pytest.fixture(scope="module")
def W(lzb):
    return lzb.weights


def _threads(n):
    import os
    return max(1, min(n, os.cpu_count() or 1))


def _reference(oracle, net, x):
    pipe = oracle.cpu_pipe(net)
    if oracle.ref_available():
        pol, val = pipe.forward(x, threads=_threads(x.shape[0]))
    else:
        pol, val = pipe.forward(x)
    policy, win = oracle.heads(net, pol, val)
    return pol, val, policy, win


def _errors(oracle, got_policy, got_win, ref_policy, ref_win):
    ep = np.abs(got_policy - ref_policy).max(1)
    ew = np.abs(got_win - ref_win)
    l2 = max(oracle.selfcheck_l2(got_policy[i], got_win[i], ref_policy[i], ref_win[i])
             for i in range(len(ew)))
    return ep, ew, l2


# ---------------------------------------------------------------------------
# single layers (every intermediate, not just the final outputs)
# ---------------------------------------------------------------------------

def _oracle_layer(oracle, net, layer, x, res=None):
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


@pytest.mark.parametrize("filters,n", [(8, 1), (18, 2), (64, 3), (192, 7), (256, 8), (64, 32)])
@pytest.mark.parametrize("mode,rel", [("fp32", 2e-6), ("fp16", 4e-3), ("fp16-winograd", 1.5e-2),
                                      ("bf16", 3e-2), ("bf16-winograd", 1.2e-1)])
def test_single_layers(lzb, oracle, W, filters, n, mode, rel):
    """Input layer, a plain tower layer and a residual layer, each compared
    with the restated CPUPipe stages; tolerance relative to the largest output
    (fp32: summation order only; 16-bit modes: operand rounding)."""
    net = W.synthetic_network(1, filters, 3000 + filters)
    x = W.synthetic_positions(n, 3100 + n)
    pipe = lzb.Pipe(net, mode)
    ctx = pipe.context(max(n, 8))
    r0 = _oracle_layer(oracle, net, 0, x)
    y0 = ctx.debug_conv(0, x)
    assert np.abs(y0 - r0).max() <= rel * max(1.0, np.abs(r0).max())
    r1 = _oracle_layer(oracle, net, 1, r0)
    y1 = ctx.debug_conv(1, r0)
    assert np.abs(y1 - r1).max() <= rel * max(1.0, np.abs(r1).max())
    r2 = _oracle_layer(oracle, net, 2, r1, r0)
    y2 = ctx.debug_conv(2, r1, r0)
    assert np.abs(y2 - r2).max() <= rel * max(1.0, np.abs(r2).max())
    ctx.close()
    pipe.close()


# ---------------------------------------------------------------------------
# whole networks: the configurations of the benchmark definition
# ---------------------------------------------------------------------------

def test_config0_fp32_batch1(lzb, oracle, W):
    """6 blocks x 64 filters, fp32, batch 1, literal random-init spec."""
    net = W.synthetic_network(6, 64, 2001)
    x = W.synthetic_positions(1, 1000)
    _, _, rp, rw = _reference(oracle, net, x)
    ctx = lzb.Pipe(net, "fp32").context(1)
    policy, win = ctx.forward_heads(x)
    ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
    assert ep.max() <= TOL_FP32 and ew.max() <= TOL_FP32 and l2 <= SELFCHECK_MAX


def test_golden_fixture_fp32(lzb, oracle, W):
    """Outputs of the reference CPUPipe committed under tests/golden."""
    import os
    from conftest import ROOT
    g = np.load(os.path.join(ROOT, "tests", "golden", "cpupipe_golden.npz"))
    for name in ("tiny_1x8", "c0_6x64", "c1_10x128", "deep_20x256_cal"):
        blocks, filters, wseed, cal, n, pseed = [int(v) for v in g[name + "/meta"]]
        net = W.synthetic_network(blocks, filters, wseed, calibrated=bool(cal))
        x = W.synthetic_positions(n, pseed)
        ctx = lzb.Pipe(net, "fp32").context(8)
        pol, val = ctx.forward(x)
        scale = max(np.abs(g[name + "/pol"]).max(), np.abs(g[name + "/val"]).max())
        assert np.abs(pol - g[name + "/pol"]).max() <= 2e-5 * scale, name
        assert np.abs(val - g[name + "/val"]).max() <= 2e-5 * scale, name
        policy, win = ctx.forward_heads(x)
        assert np.abs(policy - g[name + "/policy"]).max() <= TOL_FP32, name
        assert np.abs(win - g[name + "/winrate"]).max() <= TOL_FP32, name


def test_config1_batch8(lzb, oracle, W):
    """10 blocks x 128 filters, batch 8, fp32 and fp16.  With the literal
    random-init spec the raw head planes reach ~150 and the softmax is close to
    one-hot, which magnifies operand rounding: fp32 holds 1e-4; fp16 is held to
    the engine's self-check.  The BN-calibrated variant of the same network is
    held to the 16-bit tolerances."""
    x = W.synthetic_positions(8, 1001)
    lit = W.synthetic_network(10, 128, 2011)
    _, _, rp, rw = _reference(oracle, lit, x)
    policy, win = lzb.Pipe(lit, "fp32").context(8).forward_heads(x)
    ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
    assert ep.max() <= TOL_FP32 and ew.max() <= TOL_FP32
    # the Winograd transforms in 16 bits carry 4-5x the rounding of the direct
    # convolution, so that mode gets twice the winrate allowance here
    for mode, wtol in (("fp16", 1e-2), ("fp16-winograd", 2e-2)):
        policy, win = lzb.Pipe(lit, mode).context(8).forward_heads(x)
        ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
        assert l2 <= SELFCHECK_MAX and ew.max() <= wtol and ep.max() <= 5e-2, mode
    cal = W.synthetic_network(10, 128, 2011, calibrated=True)
    _, _, rp, rw = _reference(oracle, cal, x)
    for mode in ("fp16x2", "fp16"):
        policy, win = lzb.Pipe(cal, mode).context(8).forward_heads(x)
        ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
        assert ep.max() <= TOL_POLICY_16 and ew.max() <= TOL_VALUE_16 and l2 <= SELFCHECK_MAX, mode


@pytest.mark.parametrize("n", [1, 8, 32, 128])
def test_config2_20x256_batch_sweep(lzb, oracle, W, n):
    """20 blocks x 256 filters (BN-calibrated random init), batch 1/8/32/128.

    fp32: 1e-4.  fp16x2, the benchmarked mode: policy 2e-3 and winrate 5e-3 as
    max-abs over every position, at every batch size (small batches take other
    kernels than large ones).  The fast mode fp16 is characterised, not held to
    the bound: policy within 2e-3; winrate within 5e-3 for at least 95 % of the
    positions and within 1e-2 for all (its maximum over 128 positions is about
    6e-3, the rounding floor of fp16 operands: an exact-accumulation emulation
    gives 6.5e-3 over 96 positions).  bf16 has 3 fewer mantissa bits (8x
    coarser) and is held to the engine's self-check only."""
    net = W.synthetic_network(20, 256, 2003, calibrated=True)
    x = W.synthetic_positions(n, 1020)
    _, _, rp, rw = _reference(oracle, net, x)
    policy, win = lzb.Pipe(net, "fp32").context(n).forward_heads(x)
    ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
    assert ep.max() <= TOL_FP32 and ew.max() <= TOL_FP32
    policy, win = lzb.Pipe(net, "fp16x2").context(n).forward_heads(x)
    ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
    assert ep.max() <= TOL_POLICY_16 and ew.max() <= TOL_VALUE_16 and l2 <= SELFCHECK_MAX
    policy, win = lzb.Pipe(net, "fp16").context(n).forward_heads(x)     # fast mode, characterised
    ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
    assert ep.max() <= TOL_POLICY_16
    assert np.percentile(ew, 95) <= TOL_VALUE_16 and ew.max() <= 1e-2
    assert l2 <= SELFCHECK_MAX
    for mode in ("bf16", "fp16-winograd"):
        policy, win = lzb.Pipe(net, mode).context(n).forward_heads(x)
        ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
        assert l2 <= SELFCHECK_MAX, mode


def test_config3_40x256_batch256(lzb, oracle, W):
    """The headline configuration: 40 blocks x 256 filters, 256 positions,
    exactly the network and precision (fp16x2, its default low-plane schedule)
    bench.py times: policy 2e-3 and winrate 5e-3 as max-abs over all 256
    positions.  The same with the low plane on every block must hold them too;
    the fast mode fp16 is characterised as in config 2."""
    net = W.synthetic_network(40, 256, 2003, calibrated=True)
    x = W.synthetic_positions(256, 1040)
    _, _, rp, rw = _reference(oracle, net, x)
    for blocks_with_low_plane in (None, -1):
        policy, win = lzb.Pipe(net, "fp16x2", low_plane_blocks=blocks_with_low_plane).context(256).forward_heads(x)
        ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
        print("fp16x2 low-plane blocks %s: policy %.3g winrate %.3g" % (blocks_with_low_plane, ep.max(), ew.max()))
        assert ep.max() <= TOL_POLICY_16 and ew.max() <= TOL_VALUE_16 and l2 <= SELFCHECK_MAX
    policy, win = lzb.Pipe(net, "fp16").context(256).forward_heads(x)       # fast mode, characterised
    ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
    assert ep.max() <= TOL_POLICY_16
    assert np.percentile(ew, 95) <= TOL_VALUE_16 and ew.max() <= 1e-2
    assert l2 <= SELFCHECK_MAX
    policy, win = lzb.Pipe(net, "fp32").context(256).forward_heads(x[:16])
    ep, ew, l2 = _errors(oracle, policy, win, rp[:16], rw[:16])
    assert ep.max() <= TOL_FP32 and ew.max() <= TOL_FP32
    # weights as hi + lo too: an order of magnitude closer than "fp16"
    policy, win = lzb.Pipe(net, "fp16x3").context(64).forward_heads(x[:64])
    ep, ew, l2 = _errors(oracle, policy, win, rp[:64], rw[:64])
    assert ep.max() <= 4e-4 and ew.max() <= 1e-3
    # the same on bf16 planes: the bf16 mode that holds the half-precision bounds
    policy, win = lzb.Pipe(net, "bf16x3").context(256).forward_heads(x)
    ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
    print("bf16x3: policy %.3g winrate %.3g" % (ep.max(), ew.max()))
    assert ep.max() <= TOL_POLICY_16 and ew.max() <= TOL_VALUE_16 and l2 <= SELFCHECK_MAX


def test_low_plane_schedule_is_a_knob(lzb, oracle, W):
    """How many blocks carry the correction planes is adjustable
    (lzb_pipe_set_low_plane_blocks).  A random 40 x 256 network with sharper
    outputs than the benchmark network (weight seed 2203: plain fp16 errs by
    1e-2 on it, the default schedule by 5.1e-3 on one of these positions): with
    30 activation blocks and 8 weight blocks the half-precision bounds hold on
    every position, and more planes never make it worse than fewer."""
    net = W.synthetic_network(40, 256, 2203, calibrated=True)
    x = W.synthetic_positions(256, 1040)
    _, _, rp, rw = _reference(oracle, net, x)
    worst = {}
    for sched in ((20, 4), (30, 8), (-1, -1)):
        ctx = lzb.Pipe(net, "fp16x2", low_plane_blocks=sched[0], weight_blocks=sched[1]).context(256)
        policy, win = ctx.forward_heads(x)
        ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
        worst[sched] = (ep.max(), ew.max())
        assert l2 <= SELFCHECK_MAX
        ctx.close()
    assert worst[(30, 8)][0] <= TOL_POLICY_16 and worst[(30, 8)][1] <= TOL_VALUE_16
    assert worst[(-1, -1)][0] <= 0.5 * TOL_POLICY_16 and worst[(-1, -1)][1] <= 0.5 * TOL_VALUE_16
    assert worst[(30, 8)][1] <= worst[(20, 4)][1] and worst[(-1, -1)][1] <= worst[(30, 8)][1]


@pytest.mark.parametrize("blocks,filters,n", [(1, 8, 3), (3, 64, 9), (10, 128, 8), (6, 192, 33), (20, 256, 5)])
def test_two_plane_modes(lzb, oracle, W, blocks, filters, n):
    """fp16x2 / fp16x3 / bf16x3 on shallow and deep networks, small and medium
    batches, from Winograd-transformed weights and from plain filters: always
    inside the half-precision bounds, fp16x3 ten times inside; results do not depend on
    where the weights came from beyond fp32 rounding of the filter recovery."""
    net = W.synthetic_network(blocks, filters, 2090 + filters, calibrated=True)
    x = W.synthetic_positions(n, 1090 + n)
    _, _, rp, rw = _reference(oracle, net, x)
    for mode, tp, tv in (("fp16x2", TOL_POLICY_16, TOL_VALUE_16), ("fp16x3", 2e-4, 5e-4),
                         ("bf16x3", TOL_POLICY_16, TOL_VALUE_16)):
        ctx = lzb.Pipe(net, mode).context(n)
        policy, win = ctx.forward_heads(x)
        ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
        assert ep.max() <= tp and ew.max() <= tv and l2 <= SELFCHECK_MAX, mode
        p2, w2 = lzb.Pipe(net, mode, from_filters=True).context(n).forward_heads(x)
        assert np.abs(p2 - policy).max() <= tp and np.abs(w2 - win).max() <= tv, mode
        one = ctx.forward_heads(x[:1])
        assert np.abs(one[0] - policy[:1]).max() <= tp and np.abs(one[1] - win[:1]).max() <= tv, mode
        with pytest.raises(lzb.LzbError):
            ctx.debug_conv(0, x)



def test_literal_deep_network_fp32(lzb, oracle, W):
    """The literal (uncalibrated) random-init spec at depth 20: activations
    reach ~1e4, so only fp32 is meaningful; compared on the raw planes,
    relative to their largest value."""
    net = W.synthetic_network(20, 128, 2002)
    x = W.synthetic_positions(4, 1021)
    rpol, rval, _, _ = _reference(oracle, net, x)
    pol, val = lzb.Pipe(net, "fp32").context(4).forward(x)
    scale = max(np.abs(rpol).max(), np.abs(rval).max())
    assert np.abs(pol - rpol).max() <= 1e-5 * scale
    assert np.abs(val - rval).max() <= 1e-5 * scale


# ---------------------------------------------------------------------------
# edge cases and size-independent properties
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("mode", ["fp32", "fp16", "fp16-winograd"])
def test_ragged_batches_and_micro_batches(lzb, W, mode):
    """Every batch size and every cut into micro-batches gives the same
    numbers for a position, bit for bit: positions never mix."""
    net = W.synthetic_network(2, 64, 2050, calibrated=True)
    x = W.synthetic_positions(70, 1050)
    ctx = lzb.Pipe(net, mode).context(70)
    full_pol, full_val = ctx.forward(x)
    for n in (1, 2, 5, 6, 7, 64, 65, 69):
        pol, val = ctx.forward(x[:n])
        assert np.array_equal(pol, full_pol[:n]) and np.array_equal(val, full_val[:n]), n
    for micro in (1, 3, 32, 64):
        ctx.set_micro_batch(micro)
        pol, val = ctx.forward(x)
        assert np.array_equal(pol, full_pol) and np.array_equal(val, full_val), micro
    perm = np.random.default_rng(0).permutation(70)
    ctx.set_micro_batch(0)
    pol, val = ctx.forward(x[perm])
    assert np.array_equal(pol, full_pol[perm]) and np.array_equal(val, full_val[perm])


def test_batches_beyond_the_micro_batch_capacity(lzb, W):
    """600 positions in one call: the context cuts them into passes of at most
    256; every position comes out as it does in a call of its own pass size."""
    net = W.synthetic_network(2, 64, 2052, calibrated=True)
    x = W.synthetic_positions(600, 1052)
    ctx = lzb.Pipe(net, "fp16").context(600)
    pol, val = ctx.forward(x)
    for lo, hi in ((0, 256), (256, 512), (512, 600)):
        p, v = ctx.forward(x[lo:hi])
        assert np.array_equal(p, pol[lo:hi]) and np.array_equal(v, val[lo:hi]), lo
    policy, win = ctx.forward_heads(x)
    assert policy.shape == (600, 362) and np.allclose(policy.sum(1), 1.0, atol=1e-5)
    assert np.all((win >= 0) & (win <= 1))


def test_maximum_batch_and_repeatability(lzb, W):
    """256 positions (the largest benchmarked batch) twice: identical results;
    a blank board and a full board are evaluated without special cases."""
    net = W.synthetic_network(4, 128, 2051, calibrated=True)
    x = W.synthetic_positions(256, 1051)
    x[0] = 0.0
    x[1] = 1.0
    ctx = lzb.Pipe(net, "fp16").context(256)
    a = ctx.forward_heads(x)
    b = ctx.forward_heads(x)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    assert np.allclose(a[0].sum(1), 1.0, atol=1e-5)
    assert np.all(np.isfinite(a[1])) and np.all((a[1] >= 0) & (a[1] <= 1))


def test_argument_errors(lzb, W):
    net = W.synthetic_network(1, 8, 2052)
    pipe = lzb.Pipe(net, "fp32")
    ctx = pipe.context(4)
    with pytest.raises(lzb.LzbError) as e:
        ctx.forward(W.synthetic_positions(5, 1))      # more than max_batch
    assert e.value.code == 1
    with pytest.raises(lzb.LzbError):
        ctx.forward_heads(W.synthetic_positions(1, 1), softmax_temp=0.0)
    with pytest.raises(lzb.LzbError):
        lzb.Pipe(W.synthetic_network(1, 320, 2053), "fp16")   # tensor path: <= 256 filters
    headless = dict(net)
    del headless["heads"]
    c2 = lzb.Pipe(headless, "fp32").context(2)
    with pytest.raises(lzb.LzbError):
        c2.forward_heads(W.synthetic_positions(1, 1))
    # empty input is an argument error, not a launch
    import ctypes
    assert lzb.lib().lzb_ctx_forward(ctx.h, None, 0, None, None) == 1


def test_softmax_temperature(lzb, oracle, W):
    net = W.synthetic_network(2, 32, 2054, calibrated=True)
    x = W.synthetic_positions(3, 1054)
    pol, val, _, _ = _reference(oracle, net, x)
    ref_policy, _ = oracle.heads(net, pol, val, softmax_temp=0.7)
    policy, _ = lzb.Pipe(net, "fp32").context(4).forward_heads(x, softmax_temp=0.7)
    assert np.abs(policy - ref_policy).max() <= TOL_FP32


def test_contexts_on_concurrent_threads(lzb, W):
    """Several contexts of one pipe driven from different host threads (the
    way search threads drive a ForwardPipe) agree with a single context."""
    net = W.synthetic_network(3, 64, 2055, calibrated=True)
    x = W.synthetic_positions(24, 1055)
    pipe = lzb.Pipe(net, "fp16")
    want = pipe.context(24).forward(x)
    ctxs = [pipe.context(8) for _ in range(3)]
    got = [None] * 3

    def work(i):
        for _ in range(5):
            got[i] = ctxs[i].forward(x[8 * i:8 * i + 8])

    ts = [threading.Thread(target=work, args=(i,)) for i in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for i in range(3):
        assert np.array_equal(got[i][0], want[0][8 * i:8 * i + 8])
        assert np.array_equal(got[i][1], want[1][8 * i:8 * i + 8])


def test_single_cta_and_cta_pair_kernels_agree(lzb, W, monkeypatch):
    """The implicit-GEMM convolution exists as a one-CTA-per-tile kernel and as
    a CTA-pair (tcgen05 cta_group::2) kernel; both accumulate in the same order,
    so their outputs are identical."""
    net = W.synthetic_network(3, 128, 2057, calibrated=True)
    x = W.synthetic_positions(37, 1057)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("LZB_CONV_PAIRS", flag)
        pipe = lzb.Pipe(net, "fp16")
        outs.append(pipe.context(37).forward(x))
        pipe.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("mode", ["fp16", "fp16x2"])
@pytest.mark.parametrize("filters,n", [(128, 5), (192, 3), (256, 1), (256, 8)])
def test_reduction_split_kernel_agrees_with_sliced_kernel(lzb, oracle, W, monkeypatch, filters, n, mode):
    """Small batches run each tile on one cluster whose CTA pairs split the
    input channels and add their partial sums through distributed shared
    memory; LZB_CONV_KSPLIT=0 keeps them on the CTA-pair kernel with sliced
    output channels.  Same operands, different order of the fp32 additions:
    the raw head planes agree to fp16 rounding, and both hold the 16-bit
    tolerances against the oracle.  In fp16x2 the pairs of the cluster run the
    e5m2 planes as a second pass (5 blocks: layers with the weight remainder,
    with the activation plane only are all present in a 4-block default
    schedule only up to the remainder kind, so one more block is added)."""
    net = W.synthetic_network(5 if mode == "fp16x2" else 4, filters, 2070 + filters, calibrated=True)
    x = W.synthetic_positions(n, 1070 + n)
    _, _, rp, rw = _reference(oracle, net, x)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("LZB_CONV_KSPLIT", flag)
        pipe = lzb.Pipe(net, mode)
        ctx = pipe.context(n)
        outs.append(ctx.forward(x))
        policy, win = ctx.forward_heads(x)
        ep, ew, _ = _errors(oracle, policy, win, rp, rw)
        assert ep.max() <= TOL_POLICY_16 and ew.max() <= TOL_VALUE_16, flag
        again = ctx.forward(x)
        assert np.array_equal(again[0], outs[-1][0]) and np.array_equal(again[1], outs[-1][1]), flag
        ctx.close()
        pipe.close()
    scale = max(np.abs(outs[1][0]).max(), np.abs(outs[1][1]).max(), 1.0)
    assert np.abs(outs[0][0] - outs[1][0]).max() <= 1e-2 * scale
    assert np.abs(outs[0][1] - outs[1][1]).max() <= 1e-2 * scale


@pytest.mark.parametrize("mode", ["fp16", "fp16x2"])
def test_per_tile_dependencies_give_the_same_bits(lzb, W, monkeypatch, mode):
    """LZB_TILE_FLAGS=1 (read when a context is created; the default in fp16x2):
    the layers of a large batch wait for each other tile by tile (flags raised
    by the epilogues) instead of launch by launch, and a CTA pair visits its
    tiles middle-out.
    Same arithmetic in the same order per tile, so the outputs must agree bit
    for bit with the default path, whatever batch sizes follow one another (the
    arrival counters are never reset) and on repeated runs."""
    net = W.synthetic_network(12, 256, 2095, calibrated=True)
    x = W.synthetic_positions(256, 1095)
    pipe = lzb.Pipe(net, mode)
    monkeypatch.setenv("LZB_TILE_FLAGS", "0")
    plain = pipe.context(256)
    monkeypatch.setenv("LZB_TILE_FLAGS", "1")
    tiled = pipe.context(256)
    # LZB_TOWER_KERNEL=1 on top of it: all layers of a large batch in ONE
    # cooperative launch whose CTA pairs walk the layers (conv_tower.cuh)
    monkeypatch.setenv("LZB_TOWER_KERNEL", "1")
    tower = pipe.context(256)
    for n in (256, 64, 200, 256, 24, 131, 256):      # 24 positions: below the range it applies to
        for _ in range(3):
            a, b, t = plain.forward(x[:n]), tiled.forward(x[:n]), tower.forward(x[:n])
            assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]), n
            assert np.array_equal(a[0], t[0]) and np.array_equal(a[1], t[1]), n
    before = tower.launches
    tower.forward(x)
    assert tower.launches - before <= 4       # input planes, the tower, the 1x1 head convolutions
    plain.close()
    tiled.close()
    tower.close()
    pipe.close()


def test_untransformed_filters_and_packed_positions(lzb, oracle, W):
    """The two data formats either side of the path: filters as they stand in a
    weights file (transformed on the GPU, or used directly by the convolution
    kernel) and positions as bit planes.  fp32: same 1e-4 bound against the
    oracle; packed input must reproduce the fp32-plane entry point exactly."""
    net = W.synthetic_network(3, 64, 2059, calibrated=True)
    x = W.synthetic_positions(9, 1059)
    _, _, rp, rw = _reference(oracle, net, x)
    packed = lzb.pack_positions(x)
    assert packed.shape == (9, 18, 12) and packed.dtype == np.uint32
    for mode, tol_p, tol_v in (("fp32", TOL_FP32, TOL_FP32), ("fp16", TOL_POLICY_16, TOL_VALUE_16),
                               ("fp16-winograd", 1e-2, 2e-2)):
        a = lzb.Pipe(net, mode).context(9)
        b = lzb.Pipe(net, mode, from_filters=True).context(9)
        pa, wa = a.forward_heads(x)
        pb, wb = b.forward_heads(x)
        ep, ew, l2 = _errors(oracle, pb, wb, rp, rw)
        assert ep.max() <= tol_p and ew.max() <= tol_v and l2 <= SELFCHECK_MAX, mode
        assert np.abs(pa - pb).max() <= tol_p and np.abs(wa - wb).max() <= tol_v, mode
        pk, wk = a.forward_heads_packed(packed)
        assert np.array_equal(pk, pa) and np.array_equal(wk, wa), mode
        raw_a, raw_k = a.forward(x), a.forward_packed(packed)
        assert np.array_equal(raw_a[0], raw_k[0]) and np.array_equal(raw_a[1], raw_k[1]), mode


def test_weights_file_to_pipe(lzb, oracle, W, tmp_path):
    """A gzip'd v1 weights file through the cached loader and the GPU-side
    filter transform gives the oracle's outputs (fp32, 1e-4), from the first
    parse and from the cache alike."""
    raw = W.synthetic_raw_network(2, 32, 2060)
    path = str(tmp_path / "net.txt.gz")
    W.write_v1(raw, path)
    x = W.synthetic_positions(3, 1060)
    _, _, rp, rw = _reference(oracle, W.prepare(W.read_v1(path)), x)
    for _ in range(2):
        net = W.load_network(path, str(tmp_path / "cache"))
        policy, win = lzb.Pipe(net, "fp32", from_filters=True).context(3).forward_heads(x)
        ep, ew, l2 = _errors(oracle, policy, win, rp, rw)
        assert ep.max() <= TOL_FP32 and ew.max() <= TOL_FP32


def test_device_wait_that_runs_out_is_reported_and_survivable(lzb, W):
    """Failure detection without a fault: a kernel whose barrier nobody signals
    gives up after its limit, the host sees LZB_ERR_DEVICE_WAIT (code 3) with
    the kernel's own code in the text, and the same context then evaluates
    positions correctly."""
    import time
    net = W.synthetic_network(2, 64, 2058, calibrated=True)
    x = W.synthetic_positions(4, 1058)
    ctx = lzb.Pipe(net, "fp16").context(4)
    want = ctx.forward(x)
    t0 = time.perf_counter()
    ctx.debug_wait_probe(limit_ms=50)
    with pytest.raises(lzb.LzbError) as e:
        ctx.sync()
    waited = time.perf_counter() - t0
    assert e.value.code == 3 and "900" in str(e.value)
    assert 0.04 <= waited < 1.0                   # it waited for its limit, not forever
    ctx.sync()                                     # the flag is cleared once reported
    got = ctx.forward(x)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_profile_counters(lzb, W):
    net = W.synthetic_network(2, 64, 2056)
    ctx = lzb.Pipe(net, "fp16").context(4)
    x = W.synthetic_positions(4, 1056)
    before = ctx.launches
    ctx.profile_begin()
    ctx.forward(x)
    prof = ctx.profile_end()
    assert ctx.launches - before == sum(v[1] for v in prof.values()) == 1 + 5 + 1
    assert prof["contraction"][1] == 5 and prof["contraction"][0] > 0
