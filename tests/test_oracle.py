"""CPU tests of the checker itself: the C restatement against the reference's
own CPUPipe (when that build is present) and against the committed golden
vectors, plus the algebra the path rests on."""
import os

import numpy as np
import pytest

from conftest import ROOT, load_package, reference_root as _reference_root

GOLDEN = os.path.join(ROOT, "tests", "golden", "cpupipe_golden.npz")


@pytest.fixture(scope="module")
def W():
    return load_package().weights


def _case(golden, name, W):
    blocks, filters, wseed, cal, n, pseed = [int(v) for v in golden[name + "/meta"]]
    net = W.synthetic_network(blocks, filters, wseed, calibrated=bool(cal))
    x = W.synthetic_positions(n, pseed)
    chk = golden[name + "/input_sum"]
    assert x.sum() == chk[0], "position generator drifted from the fixture"
    assert np.isclose(np.abs(net["U"][-1]).sum(), chk[1], rtol=1e-5), "weight generator drifted"
    return net, x


@pytest.mark.parametrize("name", ["tiny_1x8", "c0_6x64", "c1_10x128"])
def test_port_matches_golden(oracle, W, name):
    """C restatement vs outputs of the reference CPUPipe stored in the fixture.
    Tolerance: sums are taken in a different order than OpenBLAS (1e-5 of the
    largest value), then policy/winrate within 1e-5."""
    g = np.load(GOLDEN)
    net, x = _case(g, name, W)
    pol, val = oracle.PortPipe(net).forward(x)
    scale = max(np.abs(g[name + "/pol"]).max(), np.abs(g[name + "/val"]).max())
    assert np.abs(pol - g[name + "/pol"]).max() <= 1e-5 * scale
    assert np.abs(val - g[name + "/val"]).max() <= 1e-5 * scale
    policy, win = oracle.heads(net, pol, val)
    assert np.abs(policy - g[name + "/policy"]).max() <= 1e-5
    assert np.abs(win - g[name + "/winrate"]).max() <= 1e-5


def test_port_matches_reference_build(oracle, W):
    """Where the reference's CPUPipe was compiled, the restatement must agree
    with it on fresh inputs (not only on the fixture)."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (no reference tree)")
    for blocks, filters, seed in ((1, 8, 5), (2, 32, 6), (3, 64, 7)):
        net = W.synthetic_network(blocks, filters, seed)
        x = W.synthetic_positions(3, seed + 100)
        a = oracle.PortPipe(net).forward(x)
        b = oracle.RefPipe(net).forward(x)
        scale = max(np.abs(b[0]).max(), np.abs(b[1]).max())
        assert np.abs(a[0] - b[0]).max() <= 1e-5 * scale
        assert np.abs(a[1] - b[1]).max() <= 1e-5 * scale


def test_reference_build_threaded_is_deterministic(oracle, W):
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built")
    net = W.synthetic_network(2, 32, 9)
    x = W.synthetic_positions(8, 10)
    p = oracle.RefPipe(net)
    a = p.forward(x, threads=1)
    b = p.forward(x, threads=4)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_winograd_equals_direct_convolution(oracle, W):
    """Filter transform + input transform + contraction + output transform is a
    zero-padded 3x3 cross-correlation (src/Network.cpp:159-223 with
    src/CPUPipe.cpp:63-284)."""
    rng = np.random.default_rng(3)
    C, K = 8, 8
    f = rng.standard_normal((K, C, 3, 3)).astype(np.float32)
    x = rng.standard_normal((1, C, 19, 19)).astype(np.float32)
    U = oracle.winograd_transform_f(f)
    lib = oracle.port_lib()
    V = np.empty((36, C, 25), np.float32)
    M = np.empty((36, K, 25), np.float32)
    Y = np.empty((K, 361), np.float32)
    lib.lzo_transform_in(oracle._ptr(np.ascontiguousarray(x[0].reshape(C, 361))), oracle._ptr(V), C)
    lib.lzo_sgemm36(oracle._ptr(U), oracle._ptr(V), oracle._ptr(M), C, K)
    lib.lzo_transform_out(oracle._ptr(M), oracle._ptr(Y), K)
    direct = W.conv3x3_direct(x, f)[0].reshape(K, 361)
    assert np.abs(Y - direct).max() <= 1e-5 * np.abs(direct).max()


def test_package_preparation_matches_restatement(oracle, W):
    """The package's numpy preparation (filter transform, BN variance, bias
    fold) against the C restatement that keeps the reference's operation
    order."""
    raw = W.synthetic_raw_network(2, 16, 11)
    raw["conv_b"][1] = np.linspace(-1, 1, 16).astype(np.float32)   # exercise the bias fold
    net = W.prepare(raw)
    for l in range(5):
        ref = oracle.winograd_transform_f(raw["conv_w"][l])
        assert np.abs(net["U"][l] - ref).max() <= 2e-7 * max(1.0, np.abs(ref).max())
        assert np.array_equal(net["bn_invstd"][l], oracle.process_bn_var(raw["bn_var"][l]))
    assert np.allclose(net["bn_mean"][1], raw["bn_mean"][1] - raw["conv_b"][1])


def test_v1_file_round_trip(W, tmp_path):
    raw = W.synthetic_raw_network(2, 8, 12)
    for path in (str(tmp_path / "net.txt"), str(tmp_path / "net.txt.gz")):
        W.write_v1(raw, path)
        back = W.read_v1(path)
        assert back["blocks"] == 2 and back["channels"] == 8
        for l in range(5):
            assert np.array_equal(back["conv_w"][l], raw["conv_w"][l])
            assert np.array_equal(back["bn_var"][l], raw["bn_var"][l])
        for k in ("ip_pol_w", "ip1_val_w", "ip2_val_w", "bn_val_mean", "pol_w"):
            assert np.array_equal(back[k].ravel(), raw[k].ravel())


def test_load_network_cache(W, tmp_path, monkeypatch):
    """load_network parses once, then serves the same arrays from the cache
    keyed by the file's hash; a changed file gets its own entry."""
    import os
    raw = W.synthetic_raw_network(1, 8, 14)
    path, cache = str(tmp_path / "net.txt.gz"), str(tmp_path / "cache")
    W.write_v1(raw, path)
    first = W.load_network(path, cache)
    assert len(os.listdir(cache)) == 1 and first["U"] == [None] * 3
    want = W.prepare(raw)

    def no_parse(_):
        raise AssertionError("parsed again although cached")
    monkeypatch.setattr(W, "read_v1", no_parse)
    second = W.load_network(path, cache)
    for net in (first, second):
        for l in range(3):
            assert np.array_equal(net["filters"][l], raw["conv_w"][l])
            assert np.array_equal(net["bn_mean"][l], want["bn_mean"][l])
            assert np.array_equal(net["bn_invstd"][l], want["bn_invstd"][l])
        for k, v in want["heads"].items():
            assert np.array_equal(net["heads"][k], v)
    monkeypatch.undo()
    raw["bn_mean"][0] = raw["bn_mean"][0] + 1
    W.write_v1(raw, path)
    third = W.load_network(path, cache)
    assert len(os.listdir(cache)) == 2
    assert np.array_equal(third["bn_mean"][0], want["bn_mean"][0] + 1)


def test_v1_file_rejects_bad_files(W, tmp_path):
    raw = W.synthetic_raw_network(1, 8, 13)
    path = str(tmp_path / "net.txt")
    W.write_v1(raw, path)
    lines = open(path).read().split("\n")
    open(path, "w").write("\n".join(["3"] + lines[1:]))
    with pytest.raises(ValueError):
        W.read_v1(path)
    open(path, "w").write("\n".join(lines[:-1]))          # one line short
    with pytest.raises(ValueError):
        W.read_v1(path)


def test_reference_fixture_file_parses(W):
    """src/tests/0k.txt, the only network file in the reference tree: 27 lines
    -> 1 block x 8 filters (src/Network.cpp:243-259)."""
    path = os.path.join(_reference_root(), "src", "tests", "0k.txt")
    if not os.path.exists(path):
        pytest.skip("reference tree not present")
    raw = W.read_v1(path)
    assert (raw["blocks"], raw["channels"]) == (1, 8)
    assert raw["conv_w"][0].shape == (8, 18, 3, 3)
    assert raw["ip_pol_w"].shape == (362, 722)


def test_reference_fixture_file_runs_through_the_oracle(oracle, W):
    path = os.path.join(_reference_root(), "src", "tests", "0k.txt")
    if not os.path.exists(path) or not oracle.ref_available():
        pytest.skip("reference tree not present")
    net = W.prepare(W.read_v1(path))
    x = W.synthetic_positions(2, 14)
    a = oracle.PortPipe(net).forward(x)
    b = oracle.RefPipe(net).forward(x)
    assert np.abs(a[0] - b[0]).max() <= 1e-5 * max(1.0, np.abs(b[0]).max())
    policy, win = oracle.heads(net, *b)
    assert np.allclose(policy.sum(1), 1.0, atol=1e-5)
    assert np.all((win >= 0) & (win <= 1))


def test_heads_and_selfcheck(oracle, W):
    net = W.synthetic_network(1, 8, 15)
    x = W.synthetic_positions(2, 16)
    pol, val = oracle.PortPipe(net).forward(x)
    policy, win = oracle.heads(net, pol, val)
    assert np.allclose(policy.sum(1), 1.0, atol=1e-5)
    assert oracle.selfcheck_l2(policy[0], win[0], policy[0], win[0]) == 0.0
    p2 = policy[0].copy()
    p2[5] += 0.3
    assert np.isclose(oracle.selfcheck_l2(p2, win[0] + 0.4, policy[0], win[0]), 0.5, atol=1e-6)
    hot, _ = oracle.heads(net, pol, val, softmax_temp=0.5)   # sharper
    assert hot.max() > policy.max()


def test_calibrated_network_keeps_activations_bounded(oracle, W):
    """The literal random-init spec grows with depth; the calibrated variant
    does not (this is why the deep configurations use it)."""
    x = W.synthetic_positions(2, 17)
    lit = oracle.PortPipe(W.synthetic_network(20, 32, 18)).forward(x)
    cal = oracle.PortPipe(W.synthetic_network(20, 32, 18, calibrated=True)).forward(x)
    assert np.abs(cal[0]).max() < 100
    assert np.abs(lit[0]).max() > 10 * np.abs(cal[0]).max()


def test_calibrated_network_behaves_alike_on_calibration_and_test_positions(lzb):
    """The batch-norm statistics of the deep benchmark networks are measured on
    4 synthetic positions (weights.calibrate_batchnorm); every accuracy figure
    is then taken on other positions.  Per layer, the activation RMS on test
    positions must stay within a factor of 2 of the RMS on the calibration
    positions (it stays within 10 %), and over the 41 layers it may grow like
    the square root of the depth (measured 3.8x), not geometrically."""
    W = lzb.weights
    seed = 2003
    raw = W.synthetic_raw_network(20, 256, seed)
    cal_x = W.synthetic_positions(4, seed + 1)
    raw = W.calibrate_batchnorm(raw, cal_x)
    on_cal = np.array(W.layer_activation_rms(raw, cal_x))
    on_test = np.array(W.layer_activation_rms(raw, W.synthetic_positions(6, 1020)))
    ratio = on_test / on_cal
    assert ratio.max() <= 2.0 and ratio.min() >= 0.5, ratio
    assert on_test[-1] <= 6.5 * on_test[2], on_test
