"""Host-side logic of ragged-batch serving, without a GPU: configuration and layer-run order, registry, step tables, page and slot
bookkeeping of the scheduler (with a stand-in model), the generation loop, sampling, and self-checks of the float64 oracle."""
import json

import numpy as np
import pytest
import torch

from tests import oracle_vofelix as O


def _cfg(loop=(1, 3, 3), n=5, side=4):
    layers = [{"type": "delta" if i % 2 == 0 else "latent_attention", "mixer": {}, "mlp": None} for i in range(n)]
    raw = {"architecture": "Vofelix", "vocab": 11, "width": 8, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5}, "layers": layers,
           "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}}
    if side:
        raw["token_side"] = {"dim": side}
    return raw


def test_layer_run_order_matches_oracle():
    from krasis_b200.vofelix import VofelixConfig
    for loop, n in [((1, 3, 3), 5), ((0, 5, 2), 5), ((2, 2, 4), 4), ((0, 1, 1), 3), ((3, 4, 2), 4)]:
        raw = _cfg(loop, n)
        assert VofelixConfig.from_dict(raw).runs() == O.layer_schedule(raw)
    runs = VofelixConfig.from_dict(_cfg((1, 3, 3), 5)).runs()
    assert [i for i, _ in runs] == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert [a for _, a in runs] == [False, False, False, True, False, True, False, False, False]


def test_config_rejects_unknown_parts():
    from krasis_b200.vofelix import VofelixConfig
    raw = _cfg()
    raw["layers"][0]["type"] = "convolution"
    with pytest.raises(ValueError):
        VofelixConfig.from_dict(raw)
    raw = _cfg()
    raw["layers"][1]["mlp"] = {"kind": "experts", "ff": 8}
    with pytest.raises(ValueError):
        VofelixConfig.from_dict(raw)
    raw = _cfg((4, 9, 2))
    with pytest.raises(ValueError):
        VofelixConfig.from_dict(raw)


def test_registry_chooses_by_config(tmp_path):
    from krasis_b200.registry import architecture_of
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Vofelix"}))
    assert architecture_of(str(tmp_path)) == "Vofelix"
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "qwen3_next", "architectures": ["Qwen3NextForCausalLM"]}))
    assert architecture_of(str(tmp_path)) == "qwen3_next"
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "unheard_of"}))
    with pytest.raises(ValueError):
        architecture_of(str(tmp_path))


def test_step_tables_layout():
    from krasis_b200.seqops import StepTables
    tb = StepTables([([5, 6, 7], 10, 2, [4, 9]), ([1], 0, 0, [3]), ([8, 8], 63, 1, [0, 1, 2])], "cpu")
    assert (tb.T, tb.S, tb.max_pages, tb.max_portion) == (6, 3, 3, 3)
    assert tb.tokens.tolist() == [5, 6, 7, 1, 8, 8]
    assert tb.positions.tolist() == [10, 11, 12, 0, 63, 64]
    assert tb.seq_of.tolist() == [0, 0, 0, 1, 2, 2]
    assert tb.cu.tolist() == [0, 3, 4, 6] and tb.slots.tolist() == [2, 0, 1]
    assert tb.pages.view(3, 3).tolist() == [[4, 9, 0], [3, 0, 0], [0, 1, 2]]


class FakeModel:
    """Stands in for a model: records the tables of every step; the logit of token v at a row is -|v - (token + position) % vocab|."""
    device, vocab, page_size = torch.device("cpu"), 13, 4

    def __init__(self):
        self.steps = []

    def make_caches(self, max_tokens, max_requests):
        from krasis_b200.attention import LatentKVCache, RecurrentStatePool
        self.kv = LatentKVCache([(2, 2)], "cpu", max_pages=(max_tokens + 3) // 4, dtype=torch.float32, page_size=4)
        self.pool = RecurrentStatePool(max_requests, "cpu")
        self.state = self.pool.register(3)
        return self.kv, self.pool

    def forward_step(self, tb, want_rows):
        self.steps.append(tb)
        for s in range(tb.S):
            self.state[tb.slots[s]] += 1.0
        if want_rows is None:
            return None
        tgt = (tb.tokens.long() + tb.positions.long())[want_rows] % self.vocab
        return -(torch.arange(self.vocab)[None, :] - tgt[:, None]).abs().float()


def test_scheduler_pages_slots_and_positions():
    from krasis_b200.scheduler import Scheduler
    m = FakeModel()
    s = Scheduler(m, max_tokens=32, max_requests=2)
    assert s.kv_cache.free_page_count == 8
    s.step([("a", [1, 2, 3, 4, 5], []), ("b", [7], [0])])
    assert s.kv_cache.free_page_count == 8 - 2 - 1
    s.step([("a", [6], [0])])                                     # b is left out of a step and goes on later
    tb = m.steps[-1]
    assert tb.positions.tolist() == [5] and tb.slots.tolist() == [s.live["a"].slot]
    s.step([("b", [8, 9, 10, 11], []), ("a", [1, 1, 1], [2])])
    tb = m.steps[-1]
    assert tb.positions.tolist() == [1, 2, 3, 4, 6, 7, 8] and tb.seq_of.tolist() == [0, 0, 0, 0, 1, 1, 1]
    assert len(s.live["b"].kv.pages) == 2 and len(s.live["a"].kv.pages) == 3
    with pytest.raises(RuntimeError):
        s.step([("c", [1], [])])                                  # both state slots are taken
    slot_b = s.live["b"].slot
    assert m.state[slot_b].tolist() == [2.0, 2.0, 2.0]
    s.finish("b")
    s.step([("c", [1], [])])
    assert s.live["c"].slot == slot_b and m.state[slot_b].tolist() == [1.0, 1.0, 1.0]      # the slot came back zeroed
    s.finish("a")
    s.finish("c")
    assert s.kv_cache.free_page_count == 8 and s.state_pool.free_slot_count == 2
    with pytest.raises(RuntimeError):
        s.step([("d", list(range(33)), [])])                      # more tokens than the pool was made for


def test_generate_continuous_batching_with_a_stand_in_model():
    from krasis_b200.scheduler import Scheduler
    m = FakeModel()
    s = Scheduler(m, max_tokens=64, max_requests=3)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [3], [2, 2], [5, 1, 5, 1, 5], [9]]
    outs = s.generate(prompts, max_new_tokens=5, step_tokens=4)

    def expect(p):
        seq, out = list(p), []
        for _ in range(5):
            out.append((seq[-1] + len(seq) - 1) % 13)
            seq.append(out[-1])
        return out
    assert outs == [expect(p) for p in prompts]
    assert not s.live and s.kv_cache.free_page_count == 16 and s.state_pool.free_slot_count == 3
    assert max(tb.T for tb in m.steps) <= 4 and max(tb.S for tb in m.steps) <= 3
    assert any(tb.S > 1 and tb.max_portion > 1 for tb in m.steps)          # a prompt portion ran beside decoded tokens


def test_sampler():
    from krasis_b200.sampling import Sampler, SamplingParams
    lg = torch.tensor([[0.1, 3.0, 2.9, -1.0], [5.0, 0.0, 0.0, 4.9]])
    assert Sampler()(lg).tolist() == [1, 0]
    assert Sampler(SamplingParams(temperature=1.0, top_k=1))(lg).tolist() == [1, 0]
    assert Sampler(SamplingParams(temperature=1.0, top_p=1e-6))(lg).tolist() == [1, 0]
    torch.manual_seed(0)
    picks = {tuple(Sampler(SamplingParams(temperature=1.0, top_k=2))(lg).tolist()) for _ in range(200)}
    assert picks <= {(1, 0), (2, 0), (1, 3), (2, 3)} and len(picks) > 1


def test_recurrent_state_pool_guards():
    from krasis_b200.attention import RecurrentStatePool
    p = RecurrentStatePool(2, "cpu")
    a, b = p.alloc(), p.alloc()
    with pytest.raises(RuntimeError):
        p.alloc()
    p.free(a)
    with pytest.raises(ValueError):
        p.free(a)
    assert p.alloc() == a and b != a


# ------------------------------------------------------------------------------------------------ the oracle's own consistency

def test_oracle_delta_rule_equals_its_closed_form_for_two_tokens():
    rng = np.random.default_rng(0)
    W, m = 6, {"heads": 1, "kv_heads": 1, "dim": 3, "vdim": 2, "conv": 1}
    w = {"q": rng.normal(size=(3, W)), "k": rng.normal(size=(3, W)), "v": rng.normal(size=(2, W)), "g": rng.normal(size=(2, W)),
         "a": rng.normal(size=(1, W)), "b": rng.normal(size=(1, W)), "q.conv": np.ones((3, 1)), "k.conv": np.ones((3, 1)), "v.conv": np.ones((2, 1)),
         "A_log": rng.normal(size=1), "dt_bias": rng.normal(size=1), "norm": np.ones(2), "o": np.eye(2)}
    h = rng.normal(size=(2, W))
    unit = lambda x: x / np.sqrt((x ** 2).sum() + 1e-6)
    q = [unit(O.silu(w["q"] @ h[t])) * 3 ** -0.5 for t in range(2)]
    k = [unit(O.silu(w["k"] @ h[t])) for t in range(2)]
    v = [O.silu(w["v"] @ h[t]) for t in range(2)]
    beta = [O.sigmoid(w["b"] @ h[t])[0] for t in range(2)]
    g = [np.exp(-np.exp(w["A_log"][0]) * O.softplus(w["a"] @ h[t] + w["dt_bias"])[0]) for t in range(2)]
    S1 = np.outer(k[0], beta[0] * v[0])
    S2 = g[1] * S1 + np.outer(k[1], beta[1] * (v[1] - (g[1] * S1).T @ k[1]))
    o = np.stack([S1.T @ q[0], S2.T @ q[1]])
    want = o / np.sqrt((o ** 2).mean(-1, keepdims=True) + 1e-5) * O.silu(h @ w["g"].T)
    np.testing.assert_allclose(O.delta_mixer(h, w, m, 1e-5), want, rtol=1e-12)


def test_oracle_window_and_sink():
    rng = np.random.default_rng(1)
    W, m = 8, {"heads": 2, "dim": 4, "rot_dim": 2, "vdim": 3, "kv_rank": 5, "scale": 0.7, "mask": {"size": 3},
               "rot": {"base": 100.0, "dims": 2}}
    w = {"q": rng.normal(size=(12, W)), "dkv": rng.normal(size=(7, W)), "dkv.norm": np.ones(5), "uk": rng.normal(size=(8, 5)),
         "uv": rng.normal(size=(6, 5)), "sink": np.array([0.3, -20.0]), "o": np.eye(6)}
    h = rng.normal(size=(6, W))
    full = O.latent_attention(h, w, None, m, 1e-5)
    # a change of the token three places back is not seen, two places back is
    h2 = h.copy()
    h2[2] += 1.0
    out2 = O.latent_attention(h2, w, None, m, 1e-5)
    assert np.allclose(out2[5], full[5]) and not np.allclose(out2[4], full[4])
    # position 0 attends itself only: weight 1 / (1 + exp(sink - s)); head 1's sink is negligible, head 0's is not
    c = O.rms_norm((h[:1] @ w["dkv"].T)[:, :5], w["dkv.norm"], 1e-5)
    v = (c @ w["uv"].T).reshape(2, 3)
    assert np.allclose(full[0, 3:], v[1], rtol=1e-6) and np.all(np.abs(full[0, :3]) < np.abs(v[0]))


def test_oracle_rotation_is_relative():
    f, amp = O.yarn_frequencies(8, 1000.0, None)
    rng = np.random.default_rng(2)
    q, k = rng.normal(size=(1, 8)), rng.normal(size=(1, 8))
    d = lambda pq, pk: (O.rotate_interleaved(q, np.array([pq], float), f, amp) @ O.rotate_interleaved(k, np.array([pk], float), f, amp).T).item()
    assert abs(d(5, 2) - d(105, 102)) < 1e-9 and abs(d(5, 2) - d(5, 3)) > 1e-6
