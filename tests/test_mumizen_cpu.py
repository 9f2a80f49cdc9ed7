"""CPU-side tests of the Mumizen design: its place in the architecture table, configurations the reader refuses, and the float64
oracle's own invariants (the GPU tests compare the engine with that oracle)."""
import json

import numpy as np

import ref_mumizen as R


def tiny(layers, width=16, vocab=8, groups=2):
    return {"architecture": "Mumizen", "width": width, "vocab": vocab, "norm": {"eps": 1e-5, "groups": groups}, "layers": layers}


RET = {"type": "retention", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "decay": [0.9, 0.5]}, "mlp": None}
LAT = {"type": "latent_attention", "mlp": None,
       "mixer": {"heads": 2, "dim": 4, "rot_dim": 2, "vdim": 4, "kv_rank": 6, "q_rank": 6, "scale": 0.4, "rot": {"base": 100.0, "dims": 2}}}


def test_architecture_table(lib):
    names = [lib.c.pb200_arch_name(i).decode() for i in range(lib.c.pb200_arch_count())]
    assert "Mumizen" in names
    assert lib.c.pb200_arch_family(b"Mumizen") == 1


def test_bad_configurations_are_refused_before_any_device_work(lib):
    mk = lib.c.pb200_model_create_from_config

    def refused(cfg):
        return not mk(json.dumps(cfg).encode(), 30, 0, 64, 1)
    assert refused(tiny([]))
    assert refused(tiny([{"type": "attention", "mixer": {"heads": 2, "dim": 4}}]))                       # another design's mixer name
    assert refused(tiny([RET], groups=3))                                                               # 16 is no multiple of 3
    bad = json.loads(json.dumps(RET))
    bad["mixer"]["decay"] = [0.9]
    assert refused(tiny([bad]))                                                                         # one decay per head
    far = json.loads(json.dumps(LAT))
    far["mixer"]["kv_from"] = 1
    assert refused(tiny([LAT, far]))                                                                    # not an earlier layer
    assert refused(tiny([RET, dict(far, mixer=dict(far["mixer"], kv_from=0))]))                         # layer 0 has no latent cache
    other = json.loads(json.dumps(LAT))
    other["mixer"].update(kv_from=0, kv_rank=8)
    assert refused(tiny([LAT, other]))                                                                  # another latent size
    moe = dict(RET, mlp={"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 2, "top": 3}})
    assert refused(tiny([moe]))                                                                         # more choices than experts
    assert refused(tiny([dict(RET, mlp={"kind": "dense", "ff": 8})]))                                   # the clamp needs its limit


def test_recurrence_equals_the_unrolled_sum():
    rng = np.random.default_rng(0)
    T, H, D, Dv = 9, 2, 3, 4
    q, k, v = rng.standard_normal((T, H, D)), rng.standard_normal((T, H, D)), rng.standard_normal((T, H, Dv))
    decay = np.array([0.8, 1.0])
    o, S = R.decay_recurrence(q, k, v, decay)
    for t in range(T):
        for h in range(H):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert np.allclose(o[t, h], want)
    # a state carried over a cut equals the whole
    o1, S1 = R.decay_recurrence(q[:4], k[:4], v[:4], decay)
    o2, S2 = R.decay_recurrence(q[4:], k[4:], v[4:], decay, S1)
    assert np.allclose(np.concatenate([o1, o2]), o) and np.allclose(S2, S)


def test_group_norm_shift_and_depth_average():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((5, 12)) * 3
    y = R.group_rms_norm(x, np.ones(12), 3, 0.0)
    assert np.allclose((y.reshape(5, 3, 4) ** 2).mean(-1), 1.0)
    assert not np.allclose(y, R.group_rms_norm(x, np.ones(12), 1, 0.0))
    h = rng.standard_normal((4, 6))
    same, last = R.token_shift(h, np.zeros(6))
    assert np.allclose(same, h) and np.allclose(last, h[-1])
    prev, _ = R.token_shift(h, np.ones(6))
    assert np.allclose(prev[1:], h[:-1]) and np.allclose(prev[0], 0.0)
    a, la = R.token_shift(h[:2], np.full(6, 0.3))
    b, _ = R.token_shift(h[2:], np.full(6, 0.3), la)
    assert np.allclose(np.concatenate([a, b]), R.token_shift(h, np.full(6, 0.3))[0])
    hist = [rng.standard_normal((2, 3)) for _ in range(3)]
    assert np.allclose(R.depth_average(hist, [0.0, 0.0, 1.0]), hist[2])
    assert np.allclose(R.depth_average(hist, [0.5, 0.25, 2.0]), 0.5 * hist[0] + 0.25 * hist[1] + 2 * hist[2])


def test_rotary_table_and_rotation():
    f, mag = R.rotary_table({"base": 10000.0, "dims": 8})
    assert np.allclose(f, [1.0, 0.1, 0.01, 0.001]) and mag == 1.0
    rot = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    fs, mags = R.rotary_table(rot)
    assert np.isclose(mags, 0.1 * np.log(4.0) + 1.0)
    assert np.isclose(fs[0], f[0]) and np.isclose(fs[-1], f[-1] / 4.0)        # fast pairs keep their frequency, slow ones are stretched
    assert np.all(fs <= f + 1e-15) and np.all(fs >= f / 4.0 - 1e-15)
    # a rotated dot product depends on the distance of the two positions only; the untouched tail passes
    rng = np.random.default_rng(2)
    a, b = rng.standard_normal((1, 10)), rng.standard_normal((1, 10))
    d1 = R.rotate(a, [7], rot)[0] @ R.rotate(b, [3], rot)[0]
    d2 = R.rotate(a, [104], rot)[0] @ R.rotate(b, [100], rot)[0]
    assert np.isclose(d1, d2)
    assert np.allclose(R.rotate(a, [5], rot)[0, 8:], a[0, 8:])
    assert np.allclose(R.rotate(a, [0], rot)[0, :8], a[0, :8] * mags)


def test_router_and_clamp():
    rng = np.random.default_rng(3)
    W = {"r.router": rng.standard_normal((6, 5)), "r.router.b": rng.standard_normal(6)}
    h = rng.standard_normal((7, 5))
    idx, wts = R.route(h, W, "r.", 3)
    z = h @ W["r.router"].T + W["r.router.b"]
    assert np.allclose(wts.sum(-1), 1.0)
    for t in range(7):
        assert set(idx[t]) == set(np.argsort(-z[t])[:3])
        assert np.all(np.diff(wts[t]) <= 1e-12)                                # in the order of the choice
    G = {"f.gate": np.eye(3) * 10, "f.up": np.eye(3) * 10, "f.down": np.eye(3)}
    y = R.clamped_glu(np.array([[1.0, -1.0, 0.01]]), G, "f.", 2.0)[0]
    g = np.array([2.0, -10.0, 0.1])                                            # the gate is clipped from above only
    u = np.array([2.0, -2.0, 0.1])
    assert np.allclose(y, g * R.sigmoid(1.702 * g) * (u + 1.0))


def test_later_tokens_do_not_change_earlier_logits():
    cfg = tiny([RET, LAT, dict(LAT, mixer=dict(LAT["mixer"], kv_from=1),
                               mlp={"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 3, "top": 2}, "shared": {"ff": 4, "limit": 2.0}})])
    _, W = R.random_weights(cfg, seed=4)
    toks = [1, 5, 2, 7, 7, 0, 3]
    full, taps = R.forward(cfg, W, toks)
    part, _ = R.forward(cfg, W, toks[:4])
    assert np.allclose(full[:4], part)
    assert taps.shape == (3, 7, 16)
