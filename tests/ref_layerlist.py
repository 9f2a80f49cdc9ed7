"""Plain, slow float64 oracle of the layer-list family (Vamidra), one function per mechanism, written from the equations; it shares no
code with the product.  Whole sequences at once, position by position where a recurrence runs.

Notation: h [T, width] is a sublayer's input, W a dict name -> float64 array (matrices stored [out, in]), c the mixer's configuration.
"""
import json
import struct

import numpy as np


# ---- element-wise ----
def silu(v):
    return v / (1.0 + np.exp(-v))


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def softplus(v):
    return np.log1p(np.exp(-np.abs(v))) + np.maximum(v, 0.0)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * w, no bias."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_unit(x, eps):
    return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps)


# ---- mechanisms ----
def visible(i, j, size, keep_first):
    """Position i sees j: causal, and inside the window or among the kept first tokens.  size <= 0: no window."""
    return j <= i and (size <= 0 or i - j < size or j < keep_first)


def attention(h, W, pre, c):
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D)
    k = (h @ W[pre + "k"].T).reshape(T, G, D)
    v = (h @ W[pre + "v"].T).reshape(T, G, Dv)
    gate = sigmoid(h @ W[pre + "g"].T)                      # [T, H], from the same input as the projections
    size = c.get("mask", {}).get("size", 0)
    keep = c.get("mask", {}).get("keep_first", 0)
    cap = c.get("softcap", 0.0)
    out = np.zeros((T, H, Dv))
    for hh in range(H):
        kv = hh // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, size, keep)]
            s = np.array([q[i, hh] @ k[j, kv] for j in js]) * c["scale"]
            if cap and cap > 0:
                s = cap * np.tanh(s / cap)
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, hh] = sum(pj * v[j, kv] for pj, j in zip(p, js))
    out *= gate[:, :, None]
    return out.reshape(T, H * Dv) @ W[pre + "o"].T


def causal_conv(x, w, b):
    """x [T, C]; w [C, taps] with the last column on the current token, zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = np.zeros((T, C))
    for t in range(T):
        acc = b.copy()
        for d in range(taps):
            if t - d >= 0:
                acc = acc + w[:, taps - 1 - d] * x[t - d]
        y[t] = acc
    return y


def mamba2(h, W, pre, c, eps):
    T = h.shape[0]
    Hn, P, N, G, taps, ng = c["heads"], c["vdim"], c["state"], c["groups"], c["conv"], c["norm_groups"]
    inner = Hn * P
    u = h @ W[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[pre + "conv"], W[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hn, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[pre + "dt_bias"])
    A = -np.exp(W[pre + "A_log"])
    S = np.zeros((Hn, N, P))
    y = np.zeros((T, Hn, P))
    for t in range(T):
        for hh in range(Hn):
            g = hh // (Hn // G)
            S[hh] = np.exp(A[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * np.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ Cm[t, g] + W[pre + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)                        # the gate comes before the norm
    y = rms_unit(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[pre + "norm"]
    return y @ W[pre + "o"].T


def feed_forward(h, W, pre):
    return (gelu_tanh(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def run_order(cfg):
    """[(layer index, pass number or None)]: layers before the repeated block once, the block `times` times in a row, the rest once."""
    L, lp = len(cfg["layers"]), cfg.get("loop")
    order, i = [], 0
    while i < L:
        if lp and i == lp["start"]:
            for t in range(lp["times"]):
                for k in range(lp["start"], lp["stop"]):
                    order.append((k, t if k == lp["start"] else None))
            i = lp["stop"]
        else:
            order.append((i, None))
            i += 1
    return order


def forward(cfg, W, tokens):
    """Returns (logits [T, vocab], residual stream after every layer run [runs, T, width])."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    x0 = x.copy()
    taps = []
    for li, t in run_order(cfg):
        if t is not None:
            x = np.concatenate([x, x0], -1) @ W["loop.in"].T + W["loop.step"][t]
        layer, pre = cfg["layers"][li], "l%d." % li
        hin = layer_norm(x, W[pre + "norm1"], eps)
        if layer["type"] == "attention":
            mixed = attention(hin, W, pre + "mix.", layer["mixer"])
        else:
            mixed = mamba2(hin, W, pre + "mix.", layer["mixer"], eps)
        x = x + layer_norm(mixed, W[pre + "norm1b"], eps)
        if layer.get("mlp"):
            f = feed_forward(layer_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.")
            x = x + layer_norm(f, W[pre + "norm2b"], eps)
        taps.append(x.copy())
    x = layer_norm(x, W["final.norm"], eps)
    return (x @ W["head"].T) * cfg["logit_scale"], np.stack(taps)


# ---- test models: shapes from a configuration, random bf16-representable weights ----
def tensor_shapes(cfg):
    Wd = cfg["width"]
    sh = {"embed": (cfg["vocab"], Wd), "head": (cfg["vocab"], Wd), "final.norm": (Wd,)}
    if cfg.get("loop"):
        sh["loop.in"] = (Wd, 2 * Wd)
        sh["loop.step"] = (cfg["loop"]["times"], Wd)
    for i, l in enumerate(cfg["layers"]):
        p, c = "l%d." % i, l["mixer"]
        sh[p + "norm1"] = sh[p + "norm1b"] = (Wd,)
        if l["type"] == "attention":
            sh[p + "mix.q"] = (c["heads"] * c["dim"], Wd)
            sh[p + "mix.k"] = (c["kv_heads"] * c["dim"], Wd)
            sh[p + "mix.v"] = (c["kv_heads"] * c["vdim"], Wd)
            sh[p + "mix.g"] = (c["heads"], Wd)
            sh[p + "mix.o"] = (Wd, c["heads"] * c["vdim"])
        else:
            inner, ch = c["heads"] * c["vdim"], c["heads"] * c["vdim"] + 2 * c["groups"] * c["state"]
            sh[p + "mix.in"] = (inner + ch + c["heads"], Wd)
            sh[p + "mix.conv"] = (ch, c["conv"])
            sh[p + "mix.conv.b"] = (ch,)
            sh[p + "mix.dt_bias"] = sh[p + "mix.A_log"] = sh[p + "mix.D"] = (c["heads"],)
            sh[p + "mix.norm"] = (inner,)
            sh[p + "mix.o"] = (Wd, inner)
        if l.get("mlp"):
            sh[p + "norm2"] = sh[p + "norm2b"] = (Wd,)
            sh[p + "mlp.gate"] = sh[p + "mlp.up"] = (l["mlp"]["ff"], Wd)
            sh[p + "mlp.down"] = (Wd, l["mlp"]["ff"])
    return sh


def to_bf16_bits(a):
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return b.astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def random_weights(cfg, seed=0):
    """name -> (bf16 bit pattern uint16 array, float64 value array); values are exactly representable in bf16."""
    rng = np.random.default_rng(seed)
    bits, vals = {}, {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf.startswith("norm"):
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf == "A_log":
            a = rng.uniform(-1.0, 1.0, shape)
        elif leaf == "dt_bias":
            a = rng.uniform(-3.0, 0.5, shape)
        elif leaf == "D":
            a = rng.uniform(0.5, 1.5, shape)
        elif leaf == "b":
            a = 0.1 * rng.standard_normal(shape)
        elif leaf == "conv":
            a = 0.5 * rng.standard_normal(shape)
        elif leaf == "step":
            a = 0.1 * rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) / np.sqrt(shape[-1])
        bits[name] = to_bf16_bits(a)
        vals[name] = from_bf16_bits(bits[name])
    return bits, vals


def write_model_dir(path, cfg, bits):
    """config.json + model.safetensors (bf16) as a loader expects them."""
    import os
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, off, blobs = {}, 0, []
    for name, b in bits.items():
        raw = np.ascontiguousarray(b).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(b.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw)


def rel_err(got, want):
    """Per row: rms of the difference (mean taken off) over the rms of the wanted row (mean taken off)."""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.maximum(np.sqrt((w ** 2).mean(-1)), 1e-30)
