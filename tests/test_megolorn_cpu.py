"""Megolorn without a GPU: configuration checks, the registry entry, and closed-form self-checks of the plain oracle."""
import json

import numpy as np
import pytest

from tests import oracle_megolorn as O


def _cfg(layers):
    return {"architecture": "Megolorn", "vocab": 11, "width": 8, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5}, "layers": layers}


def _mixer(**kw):
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "diff": 0.25, "scale": 0.5, "mask": {"size": 3}}
    m.update(kw)
    return m


def test_config_checks():
    from krasis_b200.megolorn import MegolornConfig
    ok = _cfg([{"type": "attention", "mixer": _mixer(), "mlp": None}, {"type": "attention", "mixer": _mixer(kv_from=0), "mlp": None}])
    assert len(MegolornConfig.from_dict(ok).layers) == 2
    for bad in ([{"type": "delta", "mixer": _mixer(), "mlp": None}],
                [{"type": "attention", "mixer": _mixer(heads=3, kv_heads=2), "mlp": None}],
                [{"type": "attention", "mixer": _mixer(kv_from=0), "mlp": None}],
                [{"type": "attention", "mixer": _mixer(), "mlp": None}, {"type": "attention", "mixer": _mixer(kv_from=0, vdim=7), "mlp": None}],
                [{"type": "attention", "mixer": _mixer(), "mlp": None}, {"type": "attention", "mixer": _mixer(kv_from=0), "mlp": None},
                 {"type": "attention", "mixer": _mixer(kv_from=1), "mlp": None}],
                [{"type": "attention", "mixer": _mixer(), "mlp": {"kind": "conv"}}]):
        with pytest.raises(ValueError):
            MegolornConfig.from_dict(_cfg(bad))


def test_registry_knows_the_design(tmp_path):
    from krasis_b200.registry import architecture_of
    (tmp_path / "config.json").write_text(json.dumps(_cfg([])))
    assert architecture_of(str(tmp_path)) == "Megolorn"


def test_random_weights_have_the_designs_names():
    from krasis_b200.megolorn import MegolornConfig, random_weights
    mlp = {"kind": "moe", "expert": {"ff": 5}, "router": {"experts": 3, "identity": 1, "top": 2, "groups": {"count": 2, "keep": 1}}, "shared": {"ff": 7}}
    cfg = MegolornConfig.from_dict(_cfg([{"type": "attention", "mixer": _mixer(), "mlp": {"kind": "dense", "ff": 9, "limit": 1.0}},
                                         {"type": "attention", "mixer": _mixer(kv_from=0), "mlp": mlp}]))
    w = random_weights(cfg, 0)
    assert w["l0.mix.k"].shape == (1 * 2 * 4, 8) and w["l0.mix.q"].shape == (2 * 2 * 4, 8) and w["l0.mix.v.b"].shape == (6,)
    assert "l1.mix.k" not in w and "l1.mix.v" not in w and "l1.mix.k.norm" not in w
    assert w["l1.mlp.router"].shape == (4, 8) and w["l1.mlp.correction"].shape == (4,) and "l1.mlp.e3.gate" not in w
    assert w["l1.mlp.shared.down"].shape == (8, 7) and w["l0.mlp.down"].shape == (8, 9)


def test_oracle_mask_counts_chunks_from_position_zero():
    m = O.visible(7, chunk=3)
    want = np.array([[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0], [0, 0, 0, 1, 1, 0, 0],
                     [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1]], dtype=bool)
    assert np.array_equal(m, want)
    assert np.array_equal(O.visible(4), np.tril(np.ones((4, 4), dtype=bool)))


def test_oracle_rotation_is_relative_and_keeps_the_tail():
    rng = np.random.default_rng(0)
    f = O.rotary_frequencies(4, 100.0, 2.0)
    assert np.allclose(f, [0.5, 0.05])
    q, k = rng.normal(size=(1, 6)), rng.normal(size=(1, 6))
    dots = [float(O.rotate_pairs(q, [p + 5], f)[0] @ O.rotate_pairs(k, [p], f)[0]) for p in (0, 3, 40)]
    assert np.allclose(dots, dots[0])
    assert np.array_equal(O.rotate_pairs(q, [9], f)[0, 4:], q[0, 4:])
    u, v = q[0, 0], q[0, 1]
    a = 9 * 0.5
    assert np.allclose(O.rotate_pairs(q, [9], f)[0, :2], [u * np.cos(a) - v * np.sin(a), v * np.cos(a) + u * np.sin(a)])


def test_oracle_differential_head_of_one_visible_key():
    """With a chunk of one position every map returns the token's own value: o = (1 - lambda) v, so the unit norm leaves
    sign(1 - lambda) v / rms(v) * (1 - diff) whatever the queries are."""
    rng = np.random.default_rng(1)
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "diff": 0.25, "scale": 0.5, "mask": {"size": 1}}
    W = 5
    w = {"q": rng.normal(size=(16, W)), "q.b": rng.normal(size=16), "q.norm": np.ones(4), "k": rng.normal(size=(8, W)), "k.b": rng.normal(size=8),
         "k.norm": np.ones(4), "v": rng.normal(size=(6, W)), "v.b": rng.normal(size=6), "g": np.zeros((2, W)), "o": np.eye(12),
         "lq1": np.full(4, 0.1), "lk1": np.full(4, 0.2), "lq2": np.full(4, 0.3), "lk2": np.full(4, -0.1)}
    lam = O.differential_lambda(w, 0.25)
    assert np.isclose(lam, np.exp(0.08) - np.exp(-0.12) + 0.25)
    h = rng.normal(size=(3, W))
    out, (k, v) = O.differential_attention(h, w, m, 0.0)
    val = h @ w["v"].T + w["v.b"]
    want = np.sign(1 - lam) * val / np.sqrt((val ** 2).mean(-1, keepdims=True)) * 0.75 * 0.5          # gate sigmoid(0) = 1/2
    assert np.allclose(out[:, :6], want) and np.allclose(out[:, 6:], want)
    assert np.allclose(np.sqrt((k ** 2).mean(-1)), 1.0)


def test_oracle_router_groups_identity_and_weights():
    h = np.eye(6)[:1]                                            # logits = first column of the router
    z = np.array([2.0, 0.0, 1.0, 1.5, 3.0, 0.5])
    s = np.exp(z) / np.exp(z).sum()
    corr = np.array([0.0, 0.0, 0.0, 0.0, -1.0, 0.0])            # pushes the best score's choice below zero
    router = np.zeros((6, 6))
    router[:, 0] = z
    ids, wt = O.route(h, router, corr, 2, 3, 1)                  # groups {0,1} {2,3} {4,5}: best group by choice is {0,1}
    assert ids.tolist() == [[0, 1]] and np.allclose(wt, [[s[0], s[1]]])
    ids, wt = O.route(h, router, np.zeros(6), 2, 3, 2)           # groups {4,5} and {0,1} stay: 4, then 0
    assert ids.tolist() == [[4, 0]] and np.allclose(wt, [[s[4], s[0]]])
    w = {"router": router, "correction": np.zeros(6), "e0.gate": np.ones((2, 6)), "e0.up": np.ones((2, 6)), "e0.down": np.ones((6, 2))}
    mlp = {"router": {"experts": 1, "identity": 5, "top": 2, "groups": {"count": 3, "keep": 2}}}
    y = O.mixture(h, w, mlp)                                     # expert 0 and identity expert 4
    e0 = (O.silu(np.array([1.0, 1.0])) * 1.0).sum()
    assert np.allclose(y, s[4] * h + s[0] * e0)


def test_oracle_clamped_unit():
    w = {"gate": np.array([[3.0], [-3.0], [0.5]]), "up": np.array([[5.0], [-5.0], [0.25]]), "down": np.eye(3)}
    y = O.clamped_glu(np.array([[1.0]]), w, 1.0)
    g = np.array([1.0, -3.0, 0.5])
    u = np.array([1.0, -1.0, 0.25])
    assert np.allclose(y, g / (1 + np.exp(-1.702 * g)) * (u + 1))
