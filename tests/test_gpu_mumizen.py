"""Mumizen (layer-list family) on the GPU against the float64 oracle of tests/ref_mumizen.py: every mechanism alone, prompts against
token-by-token decoding, prompt portions, ragged batches, slot reuse, far keys and far state, the edges of the kernels' tiles and
chunks, the first tokens, long decoding, odd sizes, greedy generation through the scheduler, the directory loader.  Small
configurations made here; weights are random but exactly representable in bf16, so the float32 engine and the oracle see the same
numbers and the comparison is sharp."""
import copy
import os
import subprocess
import sys

import numpy as np
import pytest

import ref_mumizen as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4     # relative rms error of a logits row, float32 engine vs float64 oracle
BF16_TOL = 6e-2

ROT = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}


def dense_ff(ff=88, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe_ff(experts=6, top=2, ff=40, limit=1.5, shared=56, shared_limit=2.5):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared, "limit": shared_limit}
    return m


def retention_layer(heads=3, dim=24, vdim=40, decay=(0.9, 0.97, 0.995), mlp=None):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def lightning_layer(heads=2, dim=16, vdim=24, decay=(0.8, 0.99), mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def latent_layer(heads=3, dim=20, rot_dim=8, vdim=28, kv_rank=36, q_rank=44, scale=0.25, rot=None, kv_from=None, mlp=None):
    mx = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
          "rot": copy.deepcopy(rot if rot is not None else ROT)}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def config(layers, width=72, vocab=149, groups=3, eps=1e-5):
    return {"architecture": "Mumizen", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": groups}, "layers": layers}


def hybrid_config():
    return config([retention_layer(mlp=dense_ff()), lightning_layer(mlp=moe_ff()), latent_layer(mlp=dense_ff(64, 2.0)),
                   latent_layer(heads=2, dim=12, vdim=20, q_rank=32, kv_from=2, mlp=moe_ff(experts=5, top=3, ff=32, shared=None)),
                   lightning_layer(heads=3, dim=8, vdim=8, decay=(0.5, 0.9, 1.0), mlp=None)])


def load(pkg, cfg, bits, dtype="float32", n_ctx=512, n_seq=8):
    m = pkg.Model.from_config(cfg, dtype=dtype, n_ctx=n_ctx, n_seq=n_seq)
    for name, b in bits.items():
        m.set_tensor(name, pkg.TYPES["bf16"], b)
    m.finalize()
    return m


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def run_whole(m, toks, want=None):
    s = m.seq_alloc()
    lg, _ = m.batch_step([(s, toks, list(range(len(toks))) if want is None else want)])
    m.seq_free(s)
    return lg


def run_decoded(m, toks, first):
    """The first `first` tokens as a prompt, the rest one by one; logits of every position."""
    s = m.seq_alloc()
    rows = [m.batch_step([(s, toks[:first], list(range(first)))])[0]]
    for t in toks[first:]:
        rows.append(m.batch_step([(s, [t], [0])])[0])
    m.seq_free(s)
    return np.concatenate(rows)


def check(got, want, tol):
    e = R.rel_err(np.asarray(got, dtype=np.float64), want)
    assert e.max() < tol, f"worst row {int(e.argmax())}: {e.max():.3e} (tolerance {tol})"


MECHANISMS = {
    "retention": lambda: config([retention_layer()]),
    "lightning": lambda: config([lightning_layer()]),
    "latent": lambda: config([latent_layer()]),
    "latent_shared_cache": lambda: config([latent_layer(), latent_layer(heads=2, dim=12, vdim=16, q_rank=24, kv_from=0)]),
    "dense_ff": lambda: config([lightning_layer(heads=1, dim=8, vdim=8, decay=(0.9,), mlp=dense_ff(136, 0.75))]),
    "moe": lambda: config([lightning_layer(heads=1, dim=8, vdim=8, decay=(0.9,), mlp=moe_ff())]),
    "depth_average": lambda: config([lightning_layer(heads=1, dim=8, vdim=8, decay=(0.9,)) for _ in range(4)]),
}


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("which", sorted(MECHANISMS))
def test_each_mechanism_alone(pkg, cuda, which, dtype, tol):
    cfg = MECHANISMS[which]()
    bits, W = R.random_weights(cfg, seed=3)
    toks = tokens_for(cfg, 37, 1)
    want, taps = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits, dtype)
    m.tap_layers(True)
    got = run_whole(m, toks)
    got_taps = m.debug_read("layers", taps.size).reshape(taps.shape)
    m.close()
    check(got, want, tol)
    scale = np.abs(taps).max()
    assert np.abs(got_taps - taps).max() < (1e-4 if dtype == "float32" else 8e-2) * scale


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_hybrid_prompt_and_decoding_agree_with_the_oracle(pkg, cuda, dtype, tol):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=5)
    toks = tokens_for(cfg, 90, 2)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits, dtype)
    check(run_whole(m, toks), want, tol)
    check(run_decoded(m, toks, 1), want, tol)          # everything after the first token through the decode path
    check(run_decoded(m, toks, 41), want, tol)
    m.close()


def test_prompt_portions_of_several_sizes(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=6)
    toks = tokens_for(cfg, 61, 3)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    for cuts in ([2, 2, 2, 55], [17, 16, 1, 27], [33, 2, 26], [60, 1]):
        s = m.seq_alloc()
        rows, at = [], 0
        for n in cuts:
            rows.append(m.batch_step([(s, toks[at:at + n], list(range(n)))])[0])
            at += n
        m.seq_free(s)
        check(np.concatenate(rows), want, F32_TOL)
    m.close()


def test_ragged_batch_equals_each_request_alone(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=7)
    m = load(pkg, cfg, bits, n_seq=6)
    lens = [1, 70, 9, 33, 18]
    reqs = [tokens_for(cfg, n + 6, 10 + i) for i, n in enumerate(lens)]
    alone = [run_decoded(m, r, n) for r, n in zip(reqs, lens)]
    slots = [m.seq_alloc() for _ in reqs]
    lg, _ = m.batch_step([(s, r[:n], list(range(n))) for s, r, n in zip(slots, reqs, lens)])
    got = [[] for _ in reqs]
    at = 0
    for i, n in enumerate(lens):
        got[i].append(lg[at:at + n])
        at += n
    live = list(range(len(reqs)))
    for k in range(6):
        if k == 3:
            live = live[:3]                                    # two requests end earlier
        lg, _ = m.batch_step([(slots[i], [reqs[i][lens[i] + k]], [0]) for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
    for i, r in enumerate(reqs):
        g = np.concatenate(got[i])
        assert np.abs(g - alone[i][:len(g)]).max() < 5e-5 * np.abs(alone[i]).max()
        want, _ = R.forward(cfg, W, r[:len(g)])
        check(g, want, F32_TOL)
    m.close()


def test_slots_are_clean_when_handed_out_again(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=8)
    m = load(pkg, cfg, bits, n_seq=2)
    a, b = tokens_for(cfg, 40, 20), tokens_for(cfg, 23, 21)
    wa, _ = R.forward(cfg, W, a)
    wb, _ = R.forward(cfg, W, b)
    for _ in range(3):                                          # the same two slots over and over, in changing roles
        s0, s1 = m.seq_alloc(), m.seq_alloc()
        lg, _ = m.batch_step([(s0, a, list(range(len(a)))), (s1, b, list(range(len(b))))])
        check(lg[:len(a)], wa, F32_TOL)
        check(lg[len(a):], wb, F32_TOL)
        m.seq_free(s0)
        s2 = m.seq_alloc()
        assert s2 == s0
        check(m.batch_step([(s2, b, list(range(len(b))))])[0], wb, F32_TOL)
        m.seq_free(s1)
        m.seq_free(s2)
        a, b, wa, wb = b, a, wb, wa
    m.close()


def one_token_matters(cfg, W, toks, where, other):
    """How much the last logits row of the oracle moves when only the token at `where` changes."""
    base, _ = R.forward(cfg, W, toks)
    t2 = list(toks)
    t2[where] = other
    moved, _ = R.forward(cfg, W, t2)
    return R.rel_err(moved[-1:], base[-1:])[0], base


def far_key_case():
    """One latent-attention layer whose last query puts nearly all its weight on position 5 of 300: queries are made the negated keys
    of their own token (so a token never looks at itself or its like), the last token A and the token B at position 5 are the pair of
    the vocabulary with the largest score, and the other positions hold tokens that score far below it against A."""
    cfg = config([latent_layer(heads=1, dim=24, rot_dim=4, vdim=16, kv_rank=32, q_rank=32, scale=3.0, rot={"base": 1e6, "dims": 4})],
                 width=48, vocab=97, groups=1)
    bits, W = R.random_weights(cfg, seed=11)
    W["l0.mix.dq"][:] = W["l0.mix.dkv"][:32]
    W["l0.mix.dq.norm"][:] = W["l0.mix.dkv.norm"]
    W["l0.mix.uq"][:24] = -W["l0.mix.uk"]
    W["l0.mix.uq"][24:] = 0.0                                   # the rotated part stays out of the score
    W["l0.shift"][:] = 0.0                                      # the mixer's input depends on the token alone
    for n in ("l0.mix.dq", "l0.mix.dq.norm", "l0.mix.uq", "l0.shift"):
        bits[n] = R.to_bf16_bits(W[n])
        W[n] = R.from_bf16_bits(bits[n])
    c, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    h = R.group_rms_norm(W["embed"], W["l0.norm1"], 1, eps)     # every token of the vocabulary at once
    lat, _ = R.latent_kv(h, W, "l0.mix.", c, eps, np.zeros(97))
    kn = lat @ W["l0.mix.uk"].T
    score = -(kn @ kn.T) * c["scale"]
    np.fill_diagonal(score, -np.inf)
    A, B = np.unravel_index(np.argmax(score), score.shape)
    quiet = [t for t in range(97) if t not in (A, B) and score[A, t] < score[A, B] - 14.0]
    assert len(quiet) >= 20
    rng = np.random.default_rng(4)
    toks = [quiet[i] for i in rng.integers(0, len(quiet), 300)]
    toks[5], toks[-1] = int(B), int(A)
    return cfg, bits, W, toks, quiet[0]


@pytest.mark.parametrize("decoded", [False, True])
def test_a_far_key_decides_the_output(pkg, cuda, decoded):
    cfg, bits, W, toks, other = far_key_case()
    moved, want = one_token_matters(cfg, W, toks, 5, other)
    assert moved > 0.05, moved                                  # the test is blind unless position 5 matters
    m = load(pkg, cfg, bits)
    got = run_decoded(m, toks, 280) if decoded else run_whole(m, toks)
    m.close()
    check(got, want, F32_TOL)


@pytest.mark.parametrize("decoded", [False, True])
def test_a_token_is_felt_far_later_through_the_state(pkg, cuda, decoded):
    cfg = config([retention_layer(heads=2, dim=16, vdim=16, decay=(0.999, 1.0)), lightning_layer(heads=1, dim=16, vdim=16, decay=(0.9995,))],
                 width=32, vocab=61, groups=2)
    bits, W = R.random_weights(cfg, seed=12)
    toks = tokens_for(cfg, 420, 5)
    moved, want = one_token_matters(cfg, W, toks, 3, (toks[3] + 7) % 61)
    assert moved > 25 * F32_TOL, moved                          # a lost or leaking state would show far above the tolerance
    m = load(pkg, cfg, bits)
    got = run_decoded(m, toks, 20) if decoded else run_whole(m, toks)
    m.close()
    check(got, want, F32_TOL)


@pytest.mark.parametrize("n", [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 130])
def test_lengths_around_the_edges_of_tiles_and_chunks(pkg, cuda, n):
    # the recurrence stages 16 tokens at a time, prompt attention walks 32 or 64 keys per tile and 4 or 64 queries per CTA, decode
    # attention 128 cache rows per pass: a prompt that ends just before, at and just after an edge, then two decoded tokens
    cfg = config([retention_layer(heads=2, dim=8, vdim=16, decay=(0.9, 0.99)), latent_layer(heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=16, q_rank=16,
                                                                                             rot={"base": 100.0, "dims": 4}, scale=1.5)],
                 width=32, vocab=53, groups=1)
    bits, W = R.random_weights(cfg, seed=13)
    toks = tokens_for(cfg, n + 2, n)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    check(run_decoded(m, toks, n), want, F32_TOL)
    m.close()


def test_first_tokens_of_a_sequence(pkg, cuda):
    # position 0 has no previous token to blend with, sees only itself and starts from the empty state
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=14)
    m = load(pkg, cfg, bits)
    for tok in (0, 7, cfg["vocab"] - 1):
        want, _ = R.forward(cfg, W, [tok])
        check(run_whole(m, [tok]), want, F32_TOL)
    toks = tokens_for(cfg, 3, 9)
    want, _ = R.forward(cfg, W, toks)
    check(run_decoded(m, toks, 1), want, F32_TOL)
    m.close()


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
def test_long_decoding(pkg, cuda, dtype, tol):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=15)
    toks = tokens_for(cfg, 260, 6)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits, dtype)
    check(run_decoded(m, toks, 4), want, tol)
    m.close()


ODD = {
    "one_of_everything": lambda: config([retention_layer(heads=1, dim=8, vdim=8, decay=(1.0,), mlp=moe_ff(experts=1, top=1, ff=8, shared=8)),
                                         latent_layer(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=4, q_rank=4, rot={"base": 10.0, "dims": 2})],
                                        width=16, vocab=11, groups=1),
    "every_expert_chosen": lambda: config([lightning_layer(mlp=moe_ff(experts=4, top=4, ff=24, shared=None))], groups=1),
    "odd_sizes": lambda: config([retention_layer(heads=3, dim=10, vdim=13, decay=(0.0, 0.5, 0.9), mlp=dense_ff(50)),
                                 latent_layer(heads=5, dim=6, rot_dim=6, vdim=9, kv_rank=21, q_rank=17, rot={"base": 500.0, "dims": 4}, mlp=moe_ff(7, 3, 18, 1.0, 10, 0.5)),
                                 lightning_layer(heads=2, dim=9, vdim=35, decay=(0.7, 0.95))], width=30, vocab=67, groups=5),
    "wide_recurrent_heads": lambda: config([lightning_layer(heads=1, dim=136, vdim=72, decay=(0.98,)), retention_layer(heads=2, dim=128, vdim=33, decay=(0.9, 0.99)),
                                            retention_layer(heads=1, dim=264, vdim=70, decay=(0.95,)), lightning_layer(heads=2, dim=40, vdim=17, decay=(0.9, 0.8))],
                                            width=64, vocab=31, groups=2),
    "wide_latent": lambda: config([latent_layer(heads=2, dim=40, rot_dim=16, vdim=136, kv_rank=260, q_rank=48,
                                                rot={"base": 10000.0, "dims": 16, "scaling": {"factor": 16.0, "original": 32, "fast": 4.0, "slow": 0.5}})],
                                   width=64, vocab=31, groups=4),
    "no_feed_forward_anywhere": lambda: config([latent_layer(), retention_layer(), latent_layer(kv_from=0)]),
}


@pytest.mark.parametrize("dtype,tol", [("float32", F32_TOL), ("bfloat16", BF16_TOL)])
@pytest.mark.parametrize("which", sorted(ODD))
def test_other_sizes(pkg, cuda, which, dtype, tol):
    cfg = ODD[which]()
    bits, W = R.random_weights(cfg, seed=16)
    toks = tokens_for(cfg, 45, 7)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits, dtype)
    check(run_whole(m, toks), want, tol)
    check(run_decoded(m, toks, 20), want, tol)
    m.close()


def test_many_tokens_take_the_sorted_expert_path(pkg, cuda):
    # a prompt long enough for the per-expert products, against the same tokens decoded one by one (the per-pair path)
    cfg = config([lightning_layer(mlp=moe_ff(experts=9, top=3, ff=48))])
    bits, W = R.random_weights(cfg, seed=17)
    toks = tokens_for(cfg, 150, 8)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits)
    whole = run_whole(m, toks)
    check(whole, want, F32_TOL)
    dec = run_decoded(m, toks, 1)
    assert np.abs(whole - dec).max() < 5e-5 * np.abs(whole).max()
    m.close()


@pytest.mark.parametrize("experts", [3, 12])
def test_expert_products_over_wide_token_tiles(pkg, cuda, experts):
    # 1200 (token, choice) pairs: 400 or 100 rows per expert on average, so the grouped product runs its 256- and 128-token tiles, with
    # experts whose rows end inside a tile
    cfg = config([lightning_layer(heads=1, dim=8, vdim=8, decay=(0.9,), mlp=moe_ff(experts=experts, top=2, ff=48, shared=None))], width=64, vocab=97, groups=2)
    bits, W = R.random_weights(cfg, seed=21)
    toks = tokens_for(cfg, 600, 9)
    want, _ = R.forward(cfg, W, toks)
    m = load(pkg, cfg, bits, "bfloat16", n_ctx=640, n_seq=2)
    check(run_whole(m, toks), want, BF16_TOL)
    m.close()


def test_greedy_generation_through_the_scheduler(pkg, cuda):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=18, gain=1.5)
    m = load(pkg, cfg, bits, n_seq=2)                           # fewer slots than requests: two batches
    prompts = [tokens_for(cfg, n, 30 + n) for n in (5, 19, 11)]
    outs = pkg.BatchScheduler(m).generate(prompts, 6)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg, _ = R.forward(cfg, W, seq)
            top2 = np.sort(lg[-1])[-2:]
            if top2[1] - top2[0] > 1e-3 * np.abs(lg[-1]).max():   # a clear winner must be the engine's choice
                assert int(np.argmax(lg[-1])) == tok
            seq.append(tok)
    m.close()


def test_directory_loader_and_trace_replay(pkg, cuda, tmp_path):
    cfg = hybrid_config()
    bits, W = R.random_weights(cfg, seed=19)
    d = tmp_path / "model"
    R.write_model_dir(str(d), cfg, bits)
    toks = tokens_for(cfg, 30, 4)
    want, _ = R.forward(cfg, W, toks)
    m = pkg.Model.from_dir(str(d), dtype="float32", n_ctx=64, n_seq=2)
    check(run_whole(m, toks), want, F32_TOL)
    m.close()
    del bits["l1.mlp.e3.up"]
    R.write_model_dir(str(d), cfg, bits)
    with pytest.raises(Exception):
        pkg.Model.from_dir(str(d), dtype="float32", n_ctx=64, n_seq=2)
    # the command-line replay: a prompt of two requests, then one decoded token each
    bits, W = R.random_weights(cfg, seed=19)
    R.write_model_dir(str(d), cfg, bits)
    import json
    a, b = toks[:20], tokens_for(cfg, 8, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:19], "want": [0, 18]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[19:], "want": [0]}, {"id": "b", "tokens": b[7:], "want": [0]}], "end": ["a", "b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out), "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "done 0" in p.stdout and "done 1" in p.stdout
    wa, _ = R.forward(cfg, W, a)
    wb, _ = R.forward(cfg, W, b)
    g0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1)
    g1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1)
    check(g0, np.stack([wa[0], wa[18], wb[6]]), F32_TOL)
    check(g1, np.stack([wa[19], wb[7]]), F32_TOL)
