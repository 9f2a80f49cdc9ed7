"""Plain, slow float64 oracle of the Mumizen design (layer-list family), one function per mechanism, written from the equations; it
shares no code with the product.  Whole sequences at once, position by position where a recurrence runs.

Notation: h [T, width] is a sublayer's input, W a dict name -> float64 array (matrices stored [out, in]), c a mixer's configuration.

The design: every layer is  x <- x + mixer(shift(norm1 x)),  x <- x + ff(norm2 x)  with a grouped RMS norm, a per-channel blend of the
mixer's input with the previous token's (token shift), and after every layer a learned weighted sum over the embedding output and the
results of all layers so far (depth average).  Mixers: two linear-attention recurrences with a fixed decay per head ("lightning",
"retention") and a softmax attention over a low-rank latent with a shared rotated key part ("latent_attention", optionally reading an
earlier layer's latent cache).  Feed-forward: a clamped gated unit, dense or as a routed mixture of experts with a shared expert.
"""
import json
import math
import os
import struct

import numpy as np


# ---- element-wise ----
def silu(v):
    return v / (1.0 + np.exp(-v))


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def rms_unit(x, eps):
    return x / np.sqrt((x ** 2).mean(-1, keepdims=True) + eps)


def group_rms_norm(x, w, groups, eps):
    """The last axis is cut into `groups` equal consecutive parts; each part is divided by its own root mean square; then * w."""
    T, n = x.shape
    parts = x.reshape(T, groups, n // groups)
    return rms_unit(parts, eps).reshape(T, n) * w


def token_shift(h, mu, prev=None):
    """out[t] = h[t] + (h[t-1] - h[t]) * mu, with h[-1] = prev (zeros at the start of a sequence); returns (out, the last h)."""
    before = np.zeros_like(h)
    before[1:] = h[:-1]
    if prev is not None:
        before[0] = prev
    return h + (before - h) * mu, h[-1].copy()


def depth_average(history, coef):
    """history: [X_0 .. X_n] (X_0 the embedding output, X_j the result of layer j-1); sum_j coef[j] X_j."""
    assert len(history) == len(coef)
    return sum(cj * Xj for cj, Xj in zip(coef, history))


# ---- linear attention with a fixed decay per head ----
def decay_recurrence(q, k, v, decay, S0=None):
    """q, k [T, H, D], v [T, H, Dv], decay [H].  S_t = decay S_{t-1} + k_t v_t^T (S [H, D, Dv]), o_t = S_t^T q_t.  Returns (o, S_T)."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = np.zeros((H, D, Dv)) if S0 is None else S0.copy()
    o = np.zeros((T, H, Dv))
    for t in range(T):
        for hh in range(H):
            S[hh] = decay[hh] * S[hh] + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    return o, S


def lightning(h, W, pre, c, eps):
    T = h.shape[0]
    H, D, Dv = c["heads"], c["dim"], c["vdim"]
    q = silu(h @ W[pre + "q"].T).reshape(T, H, D)
    k = silu(h @ W[pre + "k"].T).reshape(T, H, D)
    v = silu(h @ W[pre + "v"].T).reshape(T, H, Dv)
    o, _ = decay_recurrence(q, k, v, np.asarray(c["decay"], dtype=np.float64))
    o = rms_unit(o.reshape(T, H * Dv), eps) * W[pre + "norm"]          # all heads normed together
    o = o * sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


def retention(h, W, pre, c, eps):
    T = h.shape[0]
    H, D, Dv = c["heads"], c["dim"], c["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D)
    k = (h @ W[pre + "k"].T).reshape(T, H, D) * D ** -0.5
    v = (h @ W[pre + "v"].T).reshape(T, H, Dv)
    o, _ = decay_recurrence(q, k, v, np.asarray(c["decay"], dtype=np.float64))
    o = rms_unit(o, eps).reshape(T, H * Dv)                             # every head by its own root mean square, no weight
    o = o * silu(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


# ---- rotary positions ----
def rotary_table(rot):
    """Frequencies [dims/2] and the factor on cos / sin, with the long-context blend of rot['scaling'] when it is there."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = sc["factor"], sc["original"]

    def turn_dim(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(turn_dim(sc["fast"])), 0)
    hi = min(math.ceil(turn_dim(sc["slow"])), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, pos, rot):
    """x [T, ..., n]: the first rot['dims'] entries of the last axis are rotated in pairs (i, i + dims/2), the rest pass."""
    dims = rot["dims"]
    half = dims // 2
    f, mag = rotary_table(rot)
    ang = np.asarray(pos, dtype=np.float64)[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    cs, sn = (np.cos(ang) * mag).reshape(shape), (np.sin(ang) * mag).reshape(shape)
    a, b = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = a * cs - b * sn
    out[..., half:dims] = b * cs + a * sn
    return out


# ---- attention over a latent ----
def latent_kv(h, W, pre, c, eps, pos):
    """What a layer with its own down-projection caches: the normed latent [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    R = c["kv_rank"]
    d = h @ W[pre + "dkv"].T
    lat = rms_unit(d[:, :R], eps) * W[pre + "dkv.norm"]
    kr = rotate(d[:, R:], pos, c["rot"])
    return lat, kr


def latent_attention(h, W, pre, c, eps, pos, lat, kr):
    """lat / kr: latent and rotated key part of positions 0 .. T-1 (this layer's own, or an earlier layer's)."""
    T = h.shape[0]
    H, D, Dr, Dv = c["heads"], c["dim"], c["rot_dim"], c["vdim"]
    cq = rms_unit(h @ W[pre + "dq"].T, eps) * W[pre + "dq.norm"]
    q = (cq @ W[pre + "uq"].T).reshape(T, H, D + Dr)
    qn, qr = q[..., :D], rotate(q[..., D:], pos, c["rot"])
    kn = (lat @ W[pre + "uk"].T).reshape(T, H, D)
    v = (lat @ W[pre + "uv"].T).reshape(T, H, Dv)
    out = np.zeros((T, H, Dv))
    for hh in range(H):
        for i in range(T):
            s = (kn[: i + 1, hh] @ qn[i, hh] + kr[: i + 1] @ qr[i, hh]) * c["scale"]
            p = np.exp(s - s.max())
            p /= p.sum()
            out[i, hh] = p @ v[: i + 1, hh]
    out = out.reshape(T, H * Dv) * sigmoid(h @ W[pre + "g"].T)
    return out @ W[pre + "o"].T


# ---- feed-forward ----
def clamped_glu(h, W, pre, limit):
    g = np.minimum(h @ W[pre + "gate"].T, limit)
    u = np.clip(h @ W[pre + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[pre + "down"].T


def route(h, W, pre, top):
    """Per token: the indices of the `top` largest router logits and the softmax over those logits only."""
    z = h @ W[pre + "router"].T + W[pre + "router.b"]
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zs = np.take_along_axis(z, idx, -1)
    p = np.exp(zs - zs.max(-1, keepdims=True))
    return idx, p / p.sum(-1, keepdims=True)


def mixture(h, W, pre, mlp):
    idx, wts = route(h, W, pre, mlp["router"]["top"])
    y = np.zeros((h.shape[0], W[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, wt in zip(idx[t], wts[t]):
            y[t] += wt * clamped_glu(h[t:t + 1], W, pre + "e%d." % e, mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        y += clamped_glu(h, W, pre + "shared.", mlp["shared"]["limit"])
    return y


def feed_forward(h, W, pre, mlp):
    if mlp["kind"] == "dense":
        return clamped_glu(h, W, pre, mlp["limit"])
    return mixture(h, W, pre, mlp)


# ---- the model ----
def forward(cfg, W, tokens):
    """logits [T, vocab] and the stream that leaves every layer [layers, T, width], for one sequence from position 0."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    T = len(tokens)
    pos = np.arange(T)
    x = W["embed"][np.asarray(tokens)]
    history, taps, latents = [x], [], {}
    for i, l in enumerate(cfg["layers"]):
        p, c = "l%d." % i, l["mixer"]
        h, _ = token_shift(group_rms_norm(x, W[p + "norm1"], groups, eps), W[p + "shift"])
        if l["type"] == "lightning":
            x = x + lightning(h, W, p + "mix.", c, eps)
        elif l["type"] == "retention":
            x = x + retention(h, W, p + "mix.", c, eps)
        elif l["type"] == "latent_attention":
            src = c.get("kv_from")
            if src is None:
                latents[i] = latent_kv(h, W, p + "mix.", c, eps, pos)
                src = i
            x = x + latent_attention(h, W, p + "mix.", c, eps, pos, *latents[src])
        else:
            raise ValueError(l["type"])
        if l.get("mlp"):
            x = x + feed_forward(group_rms_norm(x, W[p + "norm2"], groups, eps), W, p + "mlp.", l["mlp"])
        history.append(x)
        x = depth_average(history, W[p + "dwa"])
        taps.append(x)
    x = group_rms_norm(x, W["final.norm"], groups, eps)
    return x @ W["head"].T, np.stack(taps)


# ---- test models: shapes from a configuration, random bf16-representable weights ----
def glu_shapes(sh, pre, ff, Wd):
    sh[pre + "gate"] = sh[pre + "up"] = (ff, Wd)
    sh[pre + "down"] = (Wd, ff)


def tensor_shapes(cfg):
    Wd = cfg["width"]
    sh = {"embed": (cfg["vocab"], Wd), "head": (cfg["vocab"], Wd), "final.norm": (Wd,)}
    for i, l in enumerate(cfg["layers"]):
        p, c = "l%d." % i, l["mixer"]
        sh[p + "norm1"] = sh[p + "shift"] = (Wd,)
        sh[p + "dwa"] = (i + 2,)
        if l["type"] in ("lightning", "retention"):
            sh[p + "mix.q"] = sh[p + "mix.k"] = (c["heads"] * c["dim"], Wd)
            sh[p + "mix.v"] = sh[p + "mix.g"] = (c["heads"] * c["vdim"], Wd)
            sh[p + "mix.o"] = (Wd, c["heads"] * c["vdim"])
            if l["type"] == "lightning":
                sh[p + "mix.norm"] = (c["heads"] * c["vdim"],)
        else:
            H, D, Dr, Dv, R, Rq = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"], c["q_rank"]
            sh[p + "mix.dq"] = (Rq, Wd)
            sh[p + "mix.dq.norm"] = (Rq,)
            sh[p + "mix.uq"] = (H * (D + Dr), Rq)
            if c.get("kv_from") is None:
                sh[p + "mix.dkv"] = (R + Dr, Wd)
                sh[p + "mix.dkv.norm"] = (R,)
            sh[p + "mix.uk"] = (H * D, R)
            sh[p + "mix.uv"] = (H * Dv, R)
            sh[p + "mix.g"] = (H * Dv, Wd)
            sh[p + "mix.o"] = (Wd, H * Dv)
        m = l.get("mlp")
        if m:
            sh[p + "norm2"] = (Wd,)
            if m["kind"] == "dense":
                glu_shapes(sh, p + "mlp.", m["ff"], Wd)
            else:
                for e in range(m["router"]["experts"]):
                    glu_shapes(sh, p + "mlp.e%d." % e, m["expert"]["ff"], Wd)
                sh[p + "mlp.router"] = (m["router"]["experts"], Wd)
                sh[p + "mlp.router.b"] = (m["router"]["experts"],)
                if m.get("shared"):
                    glu_shapes(sh, p + "mlp.shared.", m["shared"]["ff"], Wd)
    return sh


def to_bf16_bits(a):
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return b.astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def random_weights(cfg, seed=0, gain=1.0):
    """name -> (bf16 bit pattern uint16 array, float64 value array); values are exactly representable in bf16."""
    rng = np.random.default_rng(seed)
    bits, vals = {}, {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf.startswith("norm"):
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif leaf == "shift":
            a = rng.uniform(0.0, 1.0, shape)
        elif leaf == "dwa":
            a = 0.3 * rng.standard_normal(shape)
            a[-1] += 1.0
        elif leaf == "b":
            a = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        elif leaf == "router":
            a = 4.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])      # spread logits: the choice of experts is no close call
        else:
            a = gain * rng.standard_normal(shape) / np.sqrt(shape[-1])
        bits[name] = to_bf16_bits(a)
        vals[name] = from_bf16_bits(bits[name])
    return bits, vals


def write_model_dir(path, cfg, bits):
    """config.json + model.safetensors (bf16) as a loader expects them."""
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
