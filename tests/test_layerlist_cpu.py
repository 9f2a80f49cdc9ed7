"""CPU-side tests of the layer-list family: the architecture table, the scheduler's batching rules over a stand-in model, and the
float64 oracle's own invariants (the GPU tests compare the engine with that oracle)."""
import numpy as np
import pytest

import ref_layerlist as R


def test_architecture_table(lib):
    names = [lib.c.pb200_arch_name(i).decode() for i in range(lib.c.pb200_arch_count())]
    assert {"llama", "qwen2", "Vamidra"} <= set(names)
    assert lib.c.pb200_arch_family(b"llama") == 0 and lib.c.pb200_arch_family(b"qwen2") == 0
    assert lib.c.pb200_arch_family(b"Vamidra") == 1
    assert lib.c.pb200_arch_family(b"vamidra") == -1 and lib.c.pb200_arch_family(b"") == -1


def test_bad_configurations_are_refused_before_any_device_work(lib):
    mk = lib.c.pb200_model_create_from_config
    assert not mk(b"{not json", 30, 0, 64, 1)
    assert not mk(b'{"architecture": "Nope", "width": 8, "vocab": 8, "layers": []}', 30, 0, 64, 1)
    assert not mk(b'{"architecture": "Vamidra", "width": 8, "vocab": 8, "layers": []}', 30, 0, 64, 1)
    assert not mk(b'{"architecture": "Vamidra", "width": 8, "vocab": 8, "layers": [{"type": "conv", "mixer": {}}]}', 30, 0, 64, 1)
    assert not mk(b'{"architecture": "Vamidra", "width": 8, "vocab": 8, "layers": [{"type": "attention", "mixer": {"heads": 3, "kv_heads": 2, "dim": 4}}]}', 30, 0, 64, 1)
    assert not mk(b'{"architecture": "Vamidra", "width": 8, "vocab": 8, "layers": [{"type": "attention", "mixer": {"heads": 2, "dim": 4}}]}', 12, 0, 64, 1)   # k-quant is not a compute type


class FakeModel:
    """Stands in for the engine: counts slots and records every batch step."""

    def __init__(self, n_seq):
        self.n_seq, self.len, self.steps = n_seq, {}, []

    def seq_alloc(self):
        for s in range(self.n_seq):
            if s not in self.len:
                self.len[s] = 0
                return s
        raise RuntimeError("no free slot")

    def seq_free(self, s):
        del self.len[s]

    def seq_length(self, s):
        return self.len.get(s, -1)

    def batch_step(self, entries, greedy=False):
        self.steps.append([(s, list(t)) for s, t, _ in entries])
        for s, t, _ in entries:
            self.len[s] += len(t)
        return None, [100 + s for s, _, _ in entries] if greedy else None


def test_scheduler_static_batches_and_slot_release(pkg):
    fm = FakeModel(2)
    sch = pkg.BatchScheduler(fm)
    a = sch.submit([1, 2, 3], 3)
    b = sch.submit([4], 1)
    c = sch.submit([5, 6], 2)              # waits: both slots are taken by the first batch
    sch.run()
    assert a.out == [100, 100, 100] and b.out == [101] and len(c.out) == 2
    assert fm.len == {} and not sch.slots
    first = fm.steps[0]
    assert sorted(len(t) for _, t in first) == [1, 3]          # a and b start together, whole prompts
    assert [len(s) for s in fm.steps[:3]] == [2, 1, 1]          # b leaves after its only token, nobody joins the running batch
    assert all(len(t) == 1 for st in fm.steps[1:3] for _, t in st)
    assert fm.steps[3] == [(0, [5, 6])]                         # then c starts, in a freed slot


def test_scheduler_step_primitive_maps_ids_to_slots(pkg):
    fm = FakeModel(4)
    sch = pkg.BatchScheduler(fm)
    sch.step([("x", [1, 2], [1]), ("y", [3], [0])])
    sch.step([("x", [4], [0]), ("y", [5], [0])], end=["y"])
    assert fm.len == {0: 3} and list(sch.slots) == ["x"]
    sch.step([("x", [6], [0]), ("z", [7, 8], [])], end=["x", "z"])
    assert fm.steps[-1] == [(0, [6]), (1, [7, 8])] and fm.len == {}
    assert sch.live_tokens() == 0


def test_oracle_mask_and_run_order():
    assert R.visible(10, 10, 3, 0) and R.visible(10, 8, 3, 0) and not R.visible(10, 7, 3, 0) and not R.visible(3, 4, 3, 0)
    assert R.visible(10, 1, 3, 2) and not R.visible(10, 2, 3, 2) and R.visible(10, 0, 0, 0)
    cfg = {"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}
    assert R.run_order(cfg) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None), (4, None)]
    assert R.run_order({"layers": [0, 0]}) == [(0, None), (1, None)]


def test_oracle_recurrence_equals_its_unrolled_sum():
    """The state recurrence of the oracle against the closed form y_t = sum_s (prod of decays after s) dt_s (C_t . B_s) x_s + D x_t."""
    rng = np.random.default_rng(0)
    c = {"heads": 2, "vdim": 3, "state": 4, "groups": 1, "conv": 1, "norm_groups": 1}
    inner, Wd, T = 6, 5, 9
    W = {"in": rng.standard_normal((2 * inner + 8 + 2, Wd)), "conv": np.ones((inner + 8, 1)), "conv.b": np.zeros(inner + 8),
         "dt_bias": rng.standard_normal(2), "A_log": rng.standard_normal(2), "D": rng.standard_normal(2), "norm": np.ones(inner), "o": np.eye(inner)}
    h = rng.standard_normal((T, Wd))
    got = R.mamba2(h, W, "", c, 0.0)
    u = h @ W["in"].T
    z, xbc, dt = u[:, :inner], R.silu(u[:, inner:2 * inner + 8]), R.softplus(u[:, 2 * inner + 8:] + W["dt_bias"])
    x, B, C = xbc[:, :inner].reshape(T, 2, 3), xbc[:, inner:inner + 4], xbc[:, inner + 4:]
    y = np.zeros((T, 2, 3))
    for t in range(T):
        for hh in range(2):
            a = -np.exp(W["A_log"][hh])
            for s in range(t + 1):
                y[t, hh] += np.exp(a * dt[s + 1:t + 1, hh].sum()) * dt[s, hh] * (C[t] @ B[s]) * x[s, hh]
            y[t, hh] += W["D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * R.silu(z)
    y = y / np.sqrt((y ** 2).mean(-1, keepdims=True))
    assert np.allclose(got, y, rtol=1e-9, atol=1e-12)


def test_bf16_bit_conversion_round_trip():
    a = np.array([1.0, -2.5, 3.1415926, 1e-3, 65504.0, 0.0])
    b = R.to_bf16_bits(a)
    assert np.array_equal(R.to_bf16_bits(R.from_bf16_bits(b)), b)
    assert abs(R.from_bf16_bits(b)[2] - 3.1415926) < 2 ** -7
