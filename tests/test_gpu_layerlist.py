"""Layer-list family (Vamidra) on the GPU against the float64 oracle of tests/ref_layerlist.py: every mechanism alone, prompts against
token-by-token decoding, prompt portions, ragged batches, slot reuse, window / kept-token edges, long decoding, odd sizes, greedy
generation through the scheduler.  Small configurations made here; weights are random but exactly representable in bf16, so the
float32 engine and the oracle see the same numbers and the comparison is sharp."""
import copy

import numpy as np
import pytest

import ref_layerlist as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4     # relative rms error of a logits row, float32 engine vs float64 oracle
BF16_TOL = 6e-2


def attn_layer(heads=4, kv_heads=2, dim=24, vdim=40, size=7, keep=3, scale=0.3, softcap=5.0, ff=None):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
                      "mask": {"size": size, "keep_first": keep}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def ssm_layer(heads=6, vdim=20, state=12, groups=3, conv=3, norm_groups=2, ff=None):
    return {"type": "mamba2",
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, width=80, vocab=131, loop=None, logit_scale=0.7, eps=1e-5):
    c = {"architecture": "Vamidra", "width": width, "vocab": vocab, "logit_scale": logit_scale, "norm": {"eps": eps}, "layers": layers}
    if loop:
        c["loop"] = loop
    return c


def hybrid_config():
    return config([attn_layer(size=16, keep=4, ff=112), ssm_layer(ff=96), attn_layer(heads=3, kv_heads=3, dim=16, vdim=16, size=9, keep=0, ff=None),
                   ssm_layer(heads=4, vdim=24, state=16, groups=1, conv=4, norm_groups=1, ff=64)],
                  width=72, vocab=157, loop={"start": 0, "stop": 3, "times": 2})


def load(pkg, cfg, bits, dtype="float32", n_ctx=512, n_seq=8):
    m = pkg.Model.from_config(cfg, dtype=dtype, n_ctx=n_ctx, n_seq=n_seq)
    for name, b in bits.items():
        m.set_tensor(name, pkg.TYPES["bf16"], b)
    m.finalize()
    return m


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def run_whole(m, toks):
    s = m.seq_alloc()
    lg, _ = m.batch_step([(s, toks, list(range(len(toks))))])
    m.seq_free(s)
    return lg


def check(got, want, tol):
    e = R.rel_err(np.asarray(got, dtype=np.float64), want)
    assert e.max() < tol, f"worst row {int(e.argmax())}: {e.max():.3e} (tolerance {tol})"


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("which", ["attention", "mamba2", "feed_forward", "loop"])
def test_each_mechanism_alone(pkg, cuda, which, dtype, tol):
    if which == "attention":
        cfg = config([attn_layer()])
    elif which == "mamba2":
        cfg = config([ssm_layer()])
    elif which == "feed_forward":
        cfg = config([ssm_layer(heads=2, vdim=8, state=4, groups=1, conv=2, norm_groups=1, ff=136)])
    else:
        cfg = config([ssm_layer(ff=None), attn_layer(ff=48), ssm_layer(heads=2, vdim=16, state=8, groups=2, conv=2, norm_groups=1)],
                     loop={"start": 1, "stop": 3, "times": 3})
    bits, W = R.random_weights(cfg, seed=3)
    toks = tokens_for(cfg, 45, 1)
    want, taps = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits, dtype)
    m.tap_layers(True)
    got = run_whole(m, toks)
    got_taps = m.debug_read("layers", taps.size).reshape(taps.shape)
    m.close()
    check(got, want, tol)
    scale = np.abs(taps).max()
    assert np.abs(got_taps - taps).max() < (1e-4 if dtype == "float32" else 0.15) * scale


def test_prompt_against_token_by_token_decoding_past_the_ring(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=5)
    toks = tokens_for(cfg, 75, 2)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    check(run_whole(m, toks), want, F32_TOL)
    for cut in (1, 10):                                    # decoding runs far past keep_first + window rows: the ring wraps several times
        s = m.seq_alloc()
        rows = [m.batch_step([(s, toks[:cut], list(range(cut)))])[0]]
        for t in toks[cut:]:
            rows.append(m.batch_step([(s, [t], [0])])[0])
        m.seq_free(s)
        check(np.concatenate(rows), want, F32_TOL)
    m.close()


@pytest.mark.parametrize("portions", [[2] * 20, [1, 2, 3, 5, 8, 13, 8], [17, 2, 21], [39, 1]])
def test_prompt_in_portions(pkg, cuda, portions):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=6)
    toks = tokens_for(cfg, sum(portions), 3)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    s, at, rows = m.seq_alloc(), 0, []
    for n in portions:
        rows.append(m.batch_step([(s, toks[at:at + n], list(range(n)))])[0])
        at += n
        assert m.seq_length(s) == at
    m.close()
    check(np.concatenate(rows), want, F32_TOL)


def test_batch_of_unequal_requests_against_each_alone(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=7)
    lens, n_dec = [1, 7, 33, 64, 20], [25, 3, 12, 25, 0]
    reqs = [tokens_for(cfg, n + d, 10 + i) for i, (n, d) in enumerate(zip(lens, n_dec))]
    want = [R.forward(cfg, W, r)[0] for r in reqs]
    m = load(pkg, cfg, bits)
    slots = [m.seq_alloc() for _ in reqs]
    got = [[] for _ in reqs]
    lg, _ = m.batch_step([(s, r[:n], list(range(n))) for s, r, n in zip(slots, reqs, lens)])
    at = 0
    for i, n in enumerate(lens):
        got[i].append(lg[at:at + n])
        at += n
    for k in range(max(n_dec)):                            # shorter requests leave the batch earlier
        live = [i for i in range(len(reqs)) if k < n_dec[i]]
        lg, _ = m.batch_step([(slots[i], [reqs[i][lens[i] + k]], [0]) for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
    for s in slots:
        m.seq_free(s)
    alone = [run_whole(m, r) for r in reqs]
    m.close()
    for i in range(len(reqs)):
        g = np.concatenate(got[i])
        check(g, want[i], F32_TOL)
        check(g, alone[i].astype(np.float64), 5e-5)        # batch composition and prompt/decode split change rounding only


def test_slots_freed_and_used_again(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=8)
    m = load(pkg, cfg, bits, n_seq=3)
    a, b, c = (tokens_for(cfg, n, 20 + n) for n in (60, 9, 31))
    wa, wb, wc = (R.forward(cfg, W, t)[0] for t in (a, b, c))
    s0, s1, s2 = m.seq_alloc(), m.seq_alloc(), m.seq_alloc()
    with pytest.raises(pkg.host.Pb200Error):
        m.seq_alloc()                                       # every slot is taken
    m.batch_step([(s0, a, []), (s1, a[:40], []), (s2, b, [])])
    m.seq_free(s1)
    s3 = m.seq_alloc()
    assert s3 == s1                                         # the freed slot comes back, in the empty state
    lg, _ = m.batch_step([(s3, c, list(range(len(c))))])
    check(lg, wc, F32_TOL)
    m.seq_free(s0)
    m.seq_free(s2)
    s4 = m.seq_alloc()
    lg, _ = m.batch_step([(s4, b[:5], list(range(5)))])     # a short sequence in a slot that held a long one
    lg2 = np.concatenate([m.batch_step([(s4, [t], [0])])[0] for t in b[5:]])
    check(np.concatenate([lg, lg2]), wb, F32_TOL)
    with pytest.raises(pkg.host.Pb200Error):
        m.batch_step([(s2, [1], [0])])                      # a freed slot is not a sequence
    m.close()
    assert wa.shape[0] == 60


KEY_TOKEN, QUERY_TOKEN = 95, 96


def sharp_attention_model(size, keep, seed=9):
    """One attention layer made so that ONE visible position decides the output.  Queries and keys read only the first half of the
    width (same projection for both), values only the second half; KEY_TOKEN and QUERY_TOKEN share the first half of their embedding,
    so the query token scores the key token (and itself) far above every other position, while their values differ."""
    cfg = config([attn_layer(heads=2, kv_heads=2, dim=32, vdim=32, size=size, keep=keep, scale=1.5, softcap=30.0)], width=64, vocab=97)
    bits, W = R.random_weights(cfg, seed=seed)
    q = W["l0.mix.q"].copy()
    q[:, 32:] = 0.0
    v = W["l0.mix.v"].copy()
    v[:, :32] = 0.0
    e = W["embed"].copy()
    e[QUERY_TOKEN, :32] = e[KEY_TOKEN, :32]
    for name, a in (("l0.mix.q", q), ("l0.mix.k", q), ("l0.mix.v", v), ("embed", e)):
        bits[name] = R.to_bf16_bits(a)
        W[name] = R.from_bf16_bits(bits[name])
    return cfg, bits, W


@pytest.mark.parametrize("mode", ["prompt", "decode"])
def test_window_and_kept_token_edges(pkg, cuda, mode):
    size, keep = 12, 5
    cfg, bits, W = sharp_attention_model(size, keep)
    rng = np.random.default_rng(4)
    T, qpos = 70, 60
    cases = {"window_in": qpos - size + 1, "window_out": qpos - size, "kept_in": keep - 1, "kept_out": keep, "far": 20, "near": qpos - 1, "first": 0}
    m = load(pkg, cfg, bits)
    for name, j in cases.items():
        toks = rng.integers(0, 95, T).tolist()              # the two special tokens occur only where they are placed
        toks[j] = KEY_TOKEN
        toks[qpos] = QUERY_TOKEN
        want, _ = R.forward(cfg, W, toks)
        # the weights make the edge show: moving it by one position changes the oracle's answer at the query
        moved = copy.deepcopy(cfg)
        if name.startswith("window"):
            moved["layers"][0]["mixer"]["mask"]["size"] += 1 if name == "window_out" else -1
        elif name.startswith("kept"):
            moved["layers"][0]["mixer"]["mask"]["keep_first"] += 1 if name == "kept_out" else -1
        if moved != cfg:
            other, _ = R.forward(moved, W, toks)
            assert R.rel_err(other[qpos:qpos + 1], want[qpos:qpos + 1])[0] > 0.05, name
        s = m.seq_alloc()
        if mode == "prompt":
            got = m.batch_step([(s, toks, list(range(T)))])[0]
        else:
            cut = 3                                         # nearly everything is decoded: kept rows, ring wrap-around and the edges
            got = np.concatenate([m.batch_step([(s, toks[:cut], list(range(cut)))])[0]] + [m.batch_step([(s, [t], [0])])[0] for t in toks[cut:]])
        m.seq_free(s)
        check(got, want, F32_TOL)
    m.close()


def test_far_token_through_the_recurrent_state(pkg, cuda):
    cfg = config([ssm_layer(heads=4, vdim=16, state=16, groups=2, conv=4, norm_groups=2, ff=None)], width=64, vocab=61)
    bits, W = R.random_weights(cfg, seed=11)
    bits["l0.mix.A_log"] = R.to_bf16_bits(np.full(4, -6.0))            # slow decay: a token is still felt hundreds of steps later
    W["l0.mix.A_log"] = R.from_bf16_bits(bits["l0.mix.A_log"])
    toks = tokens_for(cfg, 400, 12)
    want, _ = R.forward(cfg, W, toks)
    changed = list(toks)
    changed[3] = (toks[3] + 1) % cfg["vocab"]
    want2, _ = R.forward(cfg, W, changed)
    assert R.rel_err(want2[-1:], want[-1:])[0] > 1e-3                   # position 3 matters at position 399
    m = load(pkg, cfg, bits)
    check(run_whole(m, toks), want, F32_TOL)
    s = m.seq_alloc()
    m.batch_step([(s, toks[:200], [])])
    got = np.concatenate([m.batch_step([(s, [t], [0])])[0] for t in toks[200:]])
    m.close()
    check(got, want[200:], F32_TOL)


@pytest.mark.parametrize("variant", ["no_kept_tokens", "window_longer_than_sequence", "window_of_one", "one_head_one_group_one_tap", "wide_values", "no_loop_no_softcap",
                                     "large_state_odd_dims"])
def test_other_sizes(pkg, cuda, variant):
    if variant == "no_kept_tokens":
        cfg = config([attn_layer(size=5, keep=0, ff=40), ssm_layer()], width=48)
    elif variant == "window_longer_than_sequence":
        cfg = config([attn_layer(size=1000, keep=2)], width=40)
    elif variant == "window_of_one":
        cfg = config([attn_layer(size=1, keep=6, heads=2, kv_heads=1, dim=8, vdim=8)], width=40)
    elif variant == "one_head_one_group_one_tap":
        cfg = config([ssm_layer(heads=1, vdim=36, state=7, groups=1, conv=1, norm_groups=1), attn_layer(heads=1, kv_heads=1, dim=20, vdim=12, size=4, keep=1)],
                     width=44, vocab=33, loop={"start": 0, "stop": 2, "times": 1})
    elif variant == "wide_values":
        cfg = config([attn_layer(heads=2, kv_heads=1, dim=16, vdim=200, size=6, keep=2), ssm_layer(heads=2, vdim=70, state=40, groups=2, conv=5, norm_groups=5)], width=56)
    elif variant == "large_state_odd_dims":              # a state too large for the register-resident scan; head sizes that are no multiple of 4
        cfg = config([ssm_layer(heads=2, vdim=10, state=136, groups=1, conv=3, norm_groups=2), attn_layer(heads=4, kv_heads=2, dim=18, vdim=6, size=8, keep=2)], width=52)
    else:
        cfg = config([attn_layer(softcap=0.0, ff=64), ssm_layer(ff=32)], width=64, logit_scale=1.0)
        del cfg["layers"][0]["mixer"]["softcap"]
    bits, W = R.random_weights(cfg, seed=13)
    toks = tokens_for(cfg, 37, 14)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits, n_ctx=64)
    check(run_whole(m, toks), want, F32_TOL)
    s = m.seq_alloc()
    got = np.concatenate([m.batch_step([(s, toks[:4], list(range(4)))])[0]] + [m.batch_step([(s, [t], [0])])[0] for t in toks[4:]])
    m.close()
    check(got, want, F32_TOL)


def test_greedy_generation_through_the_scheduler(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=15)
    prompts = [tokens_for(cfg, n, 30 + n) for n in (5, 19, 2, 11)]
    n_new = [9, 4, 9, 6]
    want = []
    for p, n in zip(prompts, n_new):                        # greedy decoding with the oracle: the whole sequence again for every token
        seq = list(p)
        for _ in range(n):
            seq.append(int(np.argmax(R.forward(cfg, W, seq)[0][-1])))
        want.append(seq[len(p):])
    m = load(pkg, cfg, bits, n_seq=3)                       # three slots for four requests: the last one waits for the next batch
    sched = pkg.BatchScheduler(m)
    reqs = [sched.submit(p, n) for p, n in zip(prompts, n_new)]
    sched.run()
    assert [r.out for r in reqs] == want
    assert all(r.done for r in reqs) and not sched.slots
    assert all(m.seq_length(s) < 0 for s in range(m.n_seq))  # every slot was given back
    m.close()


def test_model_directory_loader_and_missing_tensor(pkg, cuda, tmp_path):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=16)
    R.write_model_dir(tmp_path / "ok", cfg, bits)
    toks = tokens_for(cfg, 30, 17)
    want, _ = R.forward(cfg, W, toks)
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        m = pkg.Model.from_dir(tmp_path / "ok", dtype=dtype, n_ctx=64)
        assert (m.hp.n_vocab, m.hp.n_embd, m.hp.n_layer) == (cfg["vocab"], cfg["width"], len(cfg["layers"]))
        check(run_whole(m, toks), want, tol)
        m.close()
    less = {k: v for k, v in bits.items() if k != "l1.mix.D"}
    R.write_model_dir(tmp_path / "incomplete", cfg, less)
    with pytest.raises(pkg.host.Pb200Error):
        pkg.Model.from_dir(tmp_path / "incomplete", dtype="float32", n_ctx=64)
    bad = copy.deepcopy(cfg)
    bad["architecture"] = "NoSuchDesign"
    R.write_model_dir(tmp_path / "unknown", bad, bits)
    with pytest.raises(pkg.host.Pb200Error):
        pkg.Model.from_dir(tmp_path / "unknown", dtype="float32", n_ctx=64)


@pytest.mark.parametrize("T,N,K", [(1, 96, 64), (3, 130, 72), (5, 140, 80), (8, 257, 256), (9, 128, 64), (64, 300, 136), (100, 384, 200), (128, 129, 64), (200, 512, 384), (257, 129, 1032), (700, 904, 256)])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_dense_product_kernels(pkg, lib, cuda, T, N, K, dtype):
    """Every kernel behind the dense product (few-token rows, tiles, tensor cores) against a float64 product of the same operands."""
    import torch
    from gpu_util import ptr
    rng = np.random.default_rng(T * 7 + N)
    a = R.from_bf16_bits(R.to_bf16_bits(rng.standard_normal((T, K))))
    w = R.from_bf16_bits(R.to_bf16_bits(rng.standard_normal((N, K)) / np.sqrt(K)))
    bias, resid = rng.standard_normal(N), rng.standard_normal((T, N))
    want = 0.5 * (a @ w.T) + bias + resid
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    A, Wt = torch.tensor(a, dtype=tdt, device="cuda"), torch.tensor(w, dtype=tdt, device="cuda")
    Cd = torch.tensor(resid, dtype=torch.float32, device="cuda")            # the residual is added in place
    B = torch.tensor(bias, dtype=torch.float32, device="cuda")
    lib.check(lib.c.pb200_dense(pkg.TYPES[dtype], ptr(A), K, ptr(Wt), K, ptr(Cd), N, T, N, K, ptr(B), ptr(Cd), N, 0.5, None), "dense")
    torch.cuda.synchronize()
    assert lib.c.pb200_aborted() == 0
    got = Cd.cpu().numpy().astype(np.float64)
    assert np.abs(got - want).max() < 2e-5 * max(1.0, np.abs(want).max()) * np.sqrt(K / 64)
