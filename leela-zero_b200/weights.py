"""Host-side weight handling for the forward pipe: the v1/v2 text weights
format, the preparation ``Network::initialize`` applies before a pipe sees the
weights (Winograd filter transform, batch-norm variance -> 1/sqrt(var + eps),
conv-bias folding), and seeded synthetic networks and positions.

Mirrors src/Network.cpp:151-223 (math), :225-405 (file format), :540-576
(preparation).  Pure numpy; no GPU work happens here.
"""
import gzip

import numpy as np

BOARD = 19
SQ = 361
INPUT_PLANES = 18
MOVES = 362
VALUE_HIDDEN = 256
SQ2 = np.float32(1.4142135623730951)



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


def winograd_transform_f(f):
    """``f[K][C][3][3]`` -> ``U[36][C][K]`` with ``U[xi*6+nu][c][o] =
    (G f G^T)[xi][nu]`` (src/Network.cpp:159-223), as two fp32 contractions."""
    f = np.ascontiguousarray(f, np.float32)
    K, C = f.shape[:2]
    gf = np.einsum("ik,ockj->ocij", _G, f, dtype=np.float32)
    u = np.einsum("ocik,nk->inco", gf, _G, dtype=np.float32)
    return np.ascontiguousarray(u.reshape(36, C, K))


def prepare(raw, transform=True):
    """What ``Network::initialize`` does to a loaded file before a pipe sees
    it (src/Network.cpp:540-576): Winograd-transform every 3x3 filter,
    var -> 1/sqrt(var + 1e-5), fold conv biases into the BN means.  With
    ``transform=False`` the filter transform is left to the GPU (the pipe is
    then built with ``from_filters=True``) and ``U`` holds ``None``."""
    eps = np.float32(1e-5)

    def invstd(v):
        return (np.float32(1.0) / np.sqrt(np.asarray(v, np.float32) + eps)).astype(np.float32)

    net = {"blocks": raw["blocks"], "channels": raw["channels"]}
    net["filters"] = [np.ascontiguousarray(w, np.float32) for w in raw["conv_w"]]
    net["version"] = raw.get("version", 1)   # 2: value head from black's view (src/Network.cpp:393-400)
    net["U"] = [winograd_transform_f(w) if transform else None for w in raw["conv_w"]]
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


_CACHE_KEYS = ("conv_w", "conv_b", "bn_mean", "bn_var")


def load_network(path, cache_dir=None):
    """Weights file -> network dict for ``Pipe(net, ..., from_filters=True)``.

    The text format is slow to parse (a 40 x 256 network is about 1.7 GB of
    decimal text), so with ``cache_dir`` the parsed fp32 arrays are kept there
    as ``<sha256 of the file bytes>.npz`` and the next load of the same file
    reads that instead.  The 3x3 filters stay untransformed: the pipe runs the
    filter transform (src/Network.cpp:159-223) on the GPU at upload."""
    import hashlib
    import os
    cached = None
    if cache_dir is not None:
        h = hashlib.sha256()
        with open(path, "rb") as f:
            for chunk in iter(lambda: f.read(1 << 22), b""):
                h.update(chunk)
        cached = os.path.join(cache_dir, h.hexdigest() + ".npz")
    if cached is not None and os.path.exists(cached):
        z = np.load(cached)
        raw = {"blocks": int(z["blocks"]), "channels": int(z["channels"]),
               "version": int(z["version"])}
        nconv = 1 + 2 * raw["blocks"]
        for k in _CACHE_KEYS:
            raw[k] = [z["%s/%d" % (k, l)] for l in range(nconv)]
        for k in _HEAD_ORDER:
            raw[k] = z[k]
    else:
        raw = read_v1(path)
        if cached is not None:
            os.makedirs(cache_dir, exist_ok=True)
            arrays = {"blocks": raw["blocks"], "channels": raw["channels"],
                      "version": raw["version"]}
            for k in _CACHE_KEYS:
                for l, a in enumerate(raw[k]):
                    arrays["%s/%d" % (k, l)] = a
            for k in _HEAD_ORDER:
                arrays[k] = raw[k]
            tmp = cached + ".tmp%d.npz" % os.getpid()
            np.savez(tmp, **arrays)
            os.replace(tmp, cached)      # readers never see a half-written cache file
    return prepare(raw, transform=False)


def conv3x3_direct(x, w):
    """Zero-padded 3x3 cross-correlation, ``x[n][C][19][19]``, ``w[K][C][3][3]``
    -> ``[n][K][19][19]`` (the operation the Winograd pipeline evaluates)."""
    n, C = x.shape[:2]
    K = w.shape[0]
    xp = np.pad(x, ((0, 0), (0, 0), (1, 1), (1, 1)))
    cols = np.empty((n, C, 9, BOARD, BOARD), np.float32)
    for dy in range(3):
        for dx in range(3):
            cols[:, :, dy * 3 + dx] = xp[:, :, dy:dy + BOARD, dx:dx + BOARD]
    out = np.matmul(w.reshape(K, C * 9).astype(np.float32), cols.reshape(n, C * 9, SQ))
    return out.reshape(n, K, BOARD, BOARD)


def calibrate_batchnorm(raw, positions):
    """Give a random-init network the batch-norm statistics a trained one has.

    Leela Zero's batch norm has no learned scale, so a tower of He-normal
    convolutions whose BN variances are drawn independently of the data lets
    the activations grow geometrically with depth (about 1e4 after 20 blocks
    and 1e8 after 40, beyond fp16 range).  In a trained file the BN mean and
    variance of every layer are the statistics of that layer's own outputs.
    This pass runs the network in fp32 on ``positions`` and rewrites each
    layer's statistics as ``mean = mu + m * sigma`` and ``var = sigma^2 * v``,
    where ``mu, sigma`` are the measured per-channel moments and ``m ~ N(0,
    0.1)``, ``v ~ U(0.5, 1.5)`` are the values the raw network was drawn with.
    Activations then stay of order sqrt(depth).  Returns a new raw network.
    """
    out = dict(raw)
    out["bn_mean"], out["bn_var"] = [], []
    eps = np.float32(1e-5)

    def stats(y):  # y [n][K][...]
        k = y.shape[1]
        flat = np.moveaxis(y.reshape(y.shape[0], k, -1), 1, 0).reshape(k, -1)
        return flat.mean(1).astype(np.float32), flat.var(1).astype(np.float32)

    def bn_relu(y, mean, var, res=None):
        z = (y - mean[None, :, None, None]) / np.sqrt(var + eps)[None, :, None, None]
        if res is not None:
            z = z + res
        return np.maximum(z, 0).astype(np.float32)

    x = np.asarray(positions, np.float32).reshape(-1, INPUT_PLANES, BOARD, BOARD)
    res = None
    for l, w in enumerate(raw["conv_w"]):
        y = conv3x3_direct(x, w) + raw["conv_b"][l][None, :, None, None]
        mu, var = stats(y)
        var = np.maximum(var, np.float32(1e-6))
        mean = (mu + raw["bn_mean"][l] * np.sqrt(var)).astype(np.float32)
        v = (var * raw["bn_var"][l]).astype(np.float32)
        out["bn_mean"].append(mean)
        out["bn_var"].append(v)
        if l == 0:
            x = bn_relu(y, mean, v)
            res = x
        elif l % 2 == 1:
            x = bn_relu(y, mean, v)
        else:
            x = bn_relu(y, mean, v, res)
            res = x
    flat = x.reshape(x.shape[0], x.shape[1], SQ)
    for head in ("pol", "val"):
        y = np.matmul(raw[head + "_w"], flat) + raw[head + "_b"][None, :, None]
        mu, var = stats(y)
        var = np.maximum(var, np.float32(1e-6))
        out["bn_%s_mean" % head] = (mu + raw["bn_%s_mean" % head] * np.sqrt(var)).astype(np.float32)
        out["bn_%s_var" % head] = (var * raw["bn_%s_var" % head]).astype(np.float32)
    return out


def layer_activation_rms(raw, positions):
    """Root mean square of every 3x3 layer's output (after batch norm, residual
    and ReLU) of a raw network on ``positions``, fp32 on the CPU: one value per
    layer.  Used to check that a network calibrated on a few positions behaves
    the same on the positions it is then evaluated on."""
    eps = np.float32(1e-5)
    x = np.asarray(positions, np.float32).reshape(-1, INPUT_PLANES, BOARD, BOARD)
    res, rms = None, []
    for l, w in enumerate(raw["conv_w"]):
        y = conv3x3_direct(x, w) + raw["conv_b"][l][None, :, None, None]
        z = (y - raw["bn_mean"][l][None, :, None, None]) / np.sqrt(raw["bn_var"][l] + eps)[None, :, None, None]
        if l > 0 and l % 2 == 0:
            z = z + res
        x = np.maximum(z, 0).astype(np.float32)
        if l % 2 == 0:
            res = x
        rms.append(float(np.sqrt(np.mean(np.square(x, dtype=np.float64)))))
    return rms


def synthetic_network(blocks, channels, seed, calibrated=False, calibration_positions=4):
    """Seeded random-init network, prepared for a pipe.  ``calibrated`` applies
    :func:`calibrate_batchnorm` on synthetic positions drawn from seed + 1."""
    raw = synthetic_raw_network(blocks, channels, seed)
    if calibrated:
        raw = calibrate_batchnorm(raw, synthetic_positions(calibration_positions, seed + 1))
    return prepare(raw)


