"""Megolorn on the GPU against the plain float64 oracle (tests/oracle_megolorn.py): each mechanism alone, then the whole model
through the scheduler — prefill against decoding, portions down to two tokens, unequal batches, reuse of pages and slots, chunk
and page edges with peaked scores, far keys, shared key/value layers, long decoding, odd sizes, and greedy generation through the
generation entry point.  Small random configurations made here; none of them is a shipped model's."""
import json
import struct

import numpy as np
import pytest
import torch

from tests import oracle_megolorn as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def seq():
    from krasis_b200.build import build_seq
    build_seq()
    from krasis_b200 import seqops
    seqops.load()
    return seqops


def attn_cfg(heads=6, kv_heads=3, dim=16, vdim=20, chunk=8, rot_dims=12, base=5000.0, factor=4.0, diff=0.3, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale if scale is not None else dim ** -0.5}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims, "scaling": {"factor": factor}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff=56, limit=0.75):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, identity=3, top=2, groups=3, keep=2, ff=24, shared=40):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top,
                                                          "groups": {"count": groups, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def L(mixer, mlp=None):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def model_cfg(layers, width=80, vocab=50, scale=2.0, eps=1e-5):
    return {"architecture": "Megolorn", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": layers}


def default_layers():
    return [L(attn_cfg(), dense()), L(attn_cfg(kv_from=0, chunk=5), moe()), L(attn_cfg(heads=2, kv_heads=1, dim=24, vdim=40, chunk=16, rot_dims=24)),
            L(attn_cfg(heads=4, kv_heads=4, dim=8, vdim=8, chunk=None, rot_dims=0), moe(experts=5, identity=0, top=3, groups=1, keep=1, shared=0)),
            L(attn_cfg(kv_from=2, heads=2, kv_heads=1, dim=24, vdim=40, chunk=7, rot_dims=24), dense(ff=33, limit=0.2))]


def build(raw, dtype=torch.float32, seed=0, page_size=None, tweak=None):
    from krasis_b200.megolorn import MegolornConfig, MegolornModel, random_weights
    cfg = MegolornConfig.from_dict(raw)
    w = random_weights(cfg, seed)
    if tweak:
        tweak(w)
    model = MegolornModel(cfg, w, dtype=dtype)
    if page_size:
        model.page_size = page_size
    return model, {k: v.numpy().astype(np.float64) for k, v in w.items()}


def sched(model, max_tokens=512, max_requests=4, **kw):
    from krasis_b200.scheduler import Scheduler
    return Scheduler(model, max_tokens=max_tokens, max_requests=max_requests, **kw)


def toks(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def close(got, want, rel, what=""):
    got = np.asarray(got, dtype=np.float64)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-9)
    assert err <= rel, f"{what}: relative error {err:.3e} > {rel:.1e}"


def run_portions(model, tokens, cuts, s=None, rid="a", finish=True):
    """Feed `tokens` in portions of the given sizes (the rest one by one); logits of every position."""
    s = s or sched(model)
    out, at = [], 0
    sizes = list(cuts) + [1] * (len(tokens) - sum(cuts))
    for n in sizes:
        out.append(s.step([(rid, tokens[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    if finish:
        s.finish(rid)
    return np.concatenate(out, 0)


def bf(x, g=None):
    return x.to(torch.bfloat16).float()


def rnd(*shape, seed=0, sd=1.0):
    return bf(torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * sd)


def f64(d):
    return {k: v.numpy().astype(np.float64) for k, v in d.items()}


def _peaky(names, factor):
    def tweak(w):
        for k in list(w):
            if any(k.endswith(n) for n in names):
                w[k] = (w[k] * factor).to(torch.bfloat16).float()
    return tweak


# ------------------------------------------------------------------------------------------------ mechanisms alone

def attn_weights(m, W, seed, own=True):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"q": rnd(H * 2 * d, W, seed=seed, sd=W ** -0.5 * 2), "q.b": rnd(H * 2 * d, seed=seed + 1, sd=0.2), "q.norm": 1 + rnd(d, seed=seed + 2, sd=0.2),
         "g": rnd(H, W, seed=seed + 3, sd=W ** -0.5 * 3), "o": rnd(W, H * dv, seed=seed + 4, sd=0.1)}
    for i, nm in enumerate(("lq1", "lk1", "lq2", "lk2")):
        w[nm] = rnd(d, seed=seed + 10 + i, sd=0.25)
    if own:
        w.update({"k": rnd(G * 2 * d, W, seed=seed + 5, sd=W ** -0.5 * 2), "k.b": rnd(G * 2 * d, seed=seed + 6, sd=0.2),
                  "k.norm": 1 + rnd(d, seed=seed + 7, sd=0.2), "v": rnd(G * dv, W, seed=seed + 8, sd=W ** -0.5), "v.b": rnd(G * dv, seed=seed + 9, sd=0.2)})
    return w


def make_mixer(m, w, dtype=torch.float32, own=True):
    from krasis_b200.megolorn import differential_lambda
    from krasis_b200.mixers import MultiMapAttention
    mw = {k.replace(".", "_"): v for k, v in w.items()}
    rot = m.get("rot") or {}
    return MultiMapAttention(mw, m["heads"], m["kv_heads"], 2, m["dim"], m["vdim"], m["scale"], 1e-5, dtype, torch.device("cuda", 0),
                             chunk=(m.get("mask") or {}).get("size"), rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 1e4),
                             rot_factor=(rot.get("scaling") or {}).get("factor", 1.0), map_coef=[1.0, -differential_lambda(mw, m["diff"])],
                             unit_norm=True, post_scale=1 - m["diff"], own_kv=own)


def run_mixer(seq, mixer, h, cuts, page_size=4, caches=None):
    """One sequence through a mixer in portions; returns the outputs of all positions and the cache pools."""
    from krasis_b200.attention import HeadKVCache, SequenceKVState
    T = h.shape[0]
    kv = caches or HeadKVCache([mixer.cache_dims()], "cuda:0", max_pages=(T + page_size - 1) // page_size + 2, dtype=mixer.dtype, page_size=page_size)
    st = SequenceKVState(kv)
    kc, vc = kv.get_layer_caches(0)
    out, at = [], 0
    for n in list(cuts) + [1] * (T - sum(cuts)):
        st.ensure_capacity(n)
        tb = seq.StepTables([([0] * n, st.seq_len, 0, st.pages)], torch.device("cuda", 0))
        out.append(mixer.forward(h[at:at + n].to("cuda", mixer.dtype).contiguous(), tb, kc, vc, page_size).cpu().numpy())
        st.advance(n)
        at += n
    return np.concatenate(out, 0), kv


@pytest.mark.parametrize("m", [attn_cfg(), attn_cfg(heads=2, kv_heads=2, dim=32, vdim=8, chunk=None, rot_dims=32, factor=1.0),
                               attn_cfg(heads=8, kv_heads=1, dim=6, vdim=70, chunk=3, rot_dims=2, diff=0.0),
                               attn_cfg(heads=3, kv_heads=3, dim=10, vdim=33, chunk=64, rot_dims=0, diff=0.8, scale=0.7)])
def test_differential_attention_alone(seq, m):
    W, T = 48, 41
    w = attn_weights(m, W, seed=3)
    h = rnd(T, W, seed=1)
    want, _ = O.differential_attention(h.numpy().astype(np.float64), f64(w), m, 1e-5)
    mixer = make_mixer(m, w)
    for cuts in ([T], [], [2, 2, 5, 17], [30, 2]):
        got, _ = run_mixer(seq, mixer, h, cuts)
        close(got, want, 3e-5, f"portions {cuts}")


def test_attention_on_another_layers_keys_and_values(seq):
    m = attn_cfg(heads=4, kv_heads=2, dim=12, vdim=24, chunk=9, rot_dims=8)
    W, T = 40, 30
    w0, w1 = attn_weights(m, W, seed=5), attn_weights(m, W, seed=50, own=False)
    h0, h1 = rnd(T, W, seed=2), rnd(T, W, seed=3)
    _, kv = O.differential_attention(h0.numpy().astype(np.float64), f64(w0), m, 1e-5)
    want, _ = O.differential_attention(h1.numpy().astype(np.float64), f64(w1), m, 1e-5, kv=kv)
    a, b = make_mixer(m, w0), make_mixer(m, w1, own=False)
    from krasis_b200.attention import HeadKVCache
    for cuts in ([T], [7, 2, 11]):
        pools = HeadKVCache([a.cache_dims()], "cuda:0", max_pages=12, dtype=torch.float32, page_size=4)
        outs = []
        from krasis_b200.attention import SequenceKVState
        st, at = SequenceKVState(pools), 0
        kc, vc = pools.get_layer_caches(0)
        for n in list(cuts) + [1] * (T - sum(cuts)):
            st.ensure_capacity(n)
            tb = seq.StepTables([([0] * n, st.seq_len, 0, st.pages)], torch.device("cuda", 0))
            a.forward(h0[at:at + n].cuda().contiguous(), tb, kc, vc, 4)
            outs.append(b.forward(h1[at:at + n].cuda().contiguous(), tb, kc, vc, 4).cpu().numpy())
            st.advance(n)
            at += n
        close(np.concatenate(outs, 0), want, 3e-5, f"shared keys and values, portions {cuts}")


def test_attention_decode_grid_cuts_the_key_range(seq):
    """A single decoded token over hundreds of keys runs as several blocks per token whose pieces are merged; bfloat16 cache."""
    m = attn_cfg(heads=4, kv_heads=2, dim=16, vdim=32, chunk=512, rot_dims=16)
    W, T = 32, 300
    w = attn_weights(m, W, seed=9)
    h = rnd(T, W, seed=4)
    want, _ = O.differential_attention(h.numpy().astype(np.float64), f64(w), m, 1e-5)
    got, _ = run_mixer(seq, make_mixer(m, w), h, [T - 3], page_size=64)
    close(got, want, 3e-5, "fp32, cut key range")
    got, _ = run_mixer(seq, make_mixer(m, w, dtype=torch.bfloat16), h, [T - 3], page_size=64)
    close(got, want, 3e-2, "bf16, cut key range")


def test_tensor_core_prefill_of_differential_attention(seq):
    """bfloat16 with 128 query / key dims per map and 128 or 256 value dims: portions of 128 tokens or more run the tcgen05 attention
    core, one call per chunk the portion touches.  Against the oracle and against the plain kernel on the same bf16 cache, with
    peaked scores, chunks that end inside, at and across KV tiles, portions that start in the middle of a chunk."""
    from krasis_b200.build import build as build_core
    build_core()
    for chunk, vdim, heads, kv_heads in ((100, 128, 2, 1), (64, 256, 4, 2), (333, 128, 2, 2), (None, 256, 2, 1)):
        raw = model_cfg([L(attn_cfg(heads=heads, kv_heads=kv_heads, dim=128, vdim=vdim, chunk=chunk, rot_dims=64, scale=0.02), dense(ff=64))], width=64)
        model, w = build(raw, dtype=torch.bfloat16, seed=31, tweak=_peaky(["q.norm", "k.norm"], 2.0))
        mixer = model.layers[0]["mixer"]
        assert mixer.tc_shape
        tk = toks(700, raw["vocab"], 16)
        want = O.forward(raw, w, tk)
        if chunk:                                   # the chunk's edge must move the logits by far more than the tolerances below
            wide = json.loads(json.dumps(raw))
            wide["layers"][0]["mixer"]["mask"]["size"] = chunk + 1
            assert np.abs(O.forward(wide, w, tk) - want).max() > 0.15 * np.abs(want).max()
        fast_whole = run_portions(model, tk, [700], s=sched(model, 1024))
        fast_parts = run_portions(model, tk, [130, 257, 128, 150], s=sched(model, 1024))          # then 35 single tokens through the plain kernel
        mixer.tc_min_portion = 1 << 30
        plain = run_portions(model, tk, [700], s=sched(model, 1024))
        mixer.tc_min_portion = 128
        close(plain, want, 5e-2, f"chunk {chunk}: plain kernel against the oracle")
        close(fast_whole, want, 5e-2, f"chunk {chunk}: tensor-core prefill against the oracle")
        close(fast_whole, plain, 3e-2, f"chunk {chunk}: tensor-core prefill against the plain kernel")
        close(fast_parts, plain, 3e-2, f"chunk {chunk}: tensor-core portions against the plain kernel")


def test_clamped_swish_and_silu_units(seq):
    from krasis_b200.mixers import GatedMLP
    W, F, T = 40, 72, 19
    w = {"gate": rnd(F, W, seed=1, sd=0.5), "up": rnd(F, W, seed=2, sd=0.5), "down": rnd(W, F, seed=3, sd=0.2)}
    h = rnd(T, W, seed=4)
    pre = h.numpy().astype(np.float64) @ w["gate"].numpy().astype(np.float64).T
    assert (pre > 0.6).mean() > 0.1 and (pre < -0.6).mean() > 0.1        # the clamps are in play on both sides
    mlp = GatedMLP(w, torch.float32, "cuda:0", act="clamped_swish", limit=0.6, alpha=1.702)
    close(mlp.forward(h.cuda()).cpu().numpy(), O.clamped_glu(h.numpy().astype(np.float64), f64(w), 0.6), 2e-5, "clamped swish")
    mlp = GatedMLP(w, torch.float32, "cuda:0", act="silu")
    hw = f64(w)
    close(mlp.forward(h.cuda()).cpu().numpy(), O.silu_glu(h.numpy().astype(np.float64), hw["gate"], hw["up"], hw["down"]), 2e-5, "silu")


@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 4, 2), (15, 2, 3, 1), (7, 7, 1, 1), (64, 5, 8, 3), (9, 1, 3, 3)])
def test_router_choice_groups_and_weights(seq, E, top, groups, keep):
    T, W = 37, 24
    rw, h = rnd(E, W, seed=E, sd=0.6), rnd(T, W, seed=E + 1)
    corr = rnd(E, seed=E + 2, sd=0.3) - 0.4                               # mostly negative choice scores: a masked group must not win as 0
    z = (h @ rw.T).cuda().contiguous()
    ids, wt = seq.route(z, corr.cuda(), top, groups, keep)
    want_ids, want_w = O.route(h.numpy().astype(np.float64), rw.numpy().astype(np.float64), corr.numpy().astype(np.float64), top, groups, keep)
    if top > 1:
        assert (want_w + np.take_along_axis(np.tile(corr.numpy(), (T, 1)), want_ids, 1) < 0).any()
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    close(wt.cpu().numpy(), want_w, 1e-5, "router weights")


@pytest.mark.parametrize("T", [1, 5, 8, 9, 70, 200])
def test_routed_experts_alone(seq, T):
    """Few tokens take the GEMV form, more the binned tile form; identity experts, a shared expert, experts that get no token."""
    from krasis_b200.mixers import RoutedExperts
    W, F, E, ident = 32, 20, 7, 2
    mlp = moe(experts=E, identity=ident, top=3, groups=3, keep=2, ff=F, shared=28)
    w = {"router": rnd(E + ident, W, seed=1, sd=0.8), "correction": rnd(E + ident, seed=2, sd=0.1)}
    for e in range(E):
        w.update({f"e{e}.gate": rnd(F, W, seed=10 + e, sd=0.3), f"e{e}.up": rnd(F, W, seed=30 + e, sd=0.3), f"e{e}.down": rnd(W, F, seed=50 + e, sd=0.3)})
    w.update({"shared.gate": rnd(28, W, seed=70, sd=0.3), "shared.up": rnd(28, W, seed=71, sd=0.3), "shared.down": rnd(W, 28, seed=72, sd=0.3)})
    h = rnd(T, W, seed=T)
    want = O.mixture(h.numpy().astype(np.float64), f64(w), mlp)
    mod = RoutedExperts({k.replace(".", "_"): v for k, v in w.items()}, E, ident, 3, torch.float32, "cuda:0", groups=3, keep=2)
    got = mod.forward(h.cuda())
    close(got.cpu().numpy(), want, 3e-5, f"{T} tokens")
    if T > 1:                                                            # a row does not depend on the rest of the batch beyond rounding
        alone = mod.forward(h[T - 1:].cuda())
        close(alone.cpu().numpy(), got[T - 1:].cpu().numpy().astype(np.float64), 1e-5, "last row alone")


def test_routed_experts_on_the_tensor_core_gemm(seq):
    """bfloat16 steps with many rows per expert gather the rows in binned order and run one grouped tcgen05 GEMM per projection:
    against the oracle and against the binned tile kernels, with one expert that gets no token at all."""
    from krasis_b200.build import build as build_core
    from krasis_b200.mixers import RoutedExperts
    build_core()
    W, F, E, ident, T = 64, 128, 5, 1, 700
    mlp = moe(experts=E, identity=ident, top=2, groups=3, keep=2, ff=F, shared=0)
    w = {"router": rnd(E + ident, W, seed=1, sd=0.8), "correction": rnd(E + ident, seed=2, sd=0.02)}
    w["correction"][3] = -10.0                                           # expert 3 is never chosen
    for e in range(E):
        w.update({f"e{e}.gate": rnd(F, W, seed=10 + e, sd=0.2), f"e{e}.up": rnd(F, W, seed=30 + e, sd=0.2), f"e{e}.down": rnd(W, F, seed=50 + e, sd=0.2)})
    h = rnd(T, W, seed=7)
    want = O.mixture(h.numpy().astype(np.float64), f64(w), mlp)
    mod = RoutedExperts({k.replace(".", "_"): v for k, v in w.items()}, E, ident, 2, torch.bfloat16, "cuda:0", groups=3, keep=2)
    hb = h.cuda().to(torch.bfloat16)
    assert mod._tensor_core_ok(hb, T * 2)
    fast = mod.forward(hb).cpu().numpy()
    mod.tc_min_rows_per_expert = 1 << 30
    plain = mod.forward(hb).cpu().numpy()
    close(plain, want, 2e-2, "tile kernels against the oracle")
    close(fast, want, 2e-2, "tensor-core GEMMs against the oracle")
    close(fast, plain.astype(np.float64), 1e-2, "tensor-core GEMMs against the tile kernels")


def test_residual_sum_and_norm_without_bias(seq):
    T, W = 5, 77
    x, y, y2, wn = rnd(T, W, seed=1), rnd(T, W, seed=2), rnd(T, W, seed=3), 1 + rnd(W, seed=4, sd=0.1)
    xd = x.cuda().clone()
    h = seq.residual_add_norm(xd, y.cuda(), y2.cuda(), out_norm=(wn.cuda(), None), eps=1e-5)
    xs = x.numpy().astype(np.float64) + (y.numpy().astype(np.float64) + y2.numpy())
    close(xd.cpu().numpy(), xs, 1e-6, "sum")
    close(h.cpu().numpy(), O.layer_norm_nobias(xs, wn.numpy().astype(np.float64), 1e-5), 1e-5, "norm")
    xd = x.cuda().clone()
    assert seq.residual_add_norm(xd, y.cuda()) is None
    close(xd.cpu().numpy(), x.numpy().astype(np.float64) + y.numpy(), 1e-6, "one addend, no norm")


# ------------------------------------------------------------------------------------------------ the whole model

def test_layer_trace_matches_oracle(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=1, page_size=4)
    tk = toks(29, raw["vocab"], 5)
    col = []
    want = O.forward(raw, w, tk, col)
    model.layer_trace = []
    got = run_portions(model, tk, [29])
    trace, model.layer_trace = model.layer_trace, None
    assert len(trace) == len(col) == len(raw["layers"])
    for i, (a, b) in enumerate(zip(trace, col)):
        close(a.cpu().numpy(), b, 2e-5, f"residual stream after layer {i}")
    close(got, want, 4e-5, "logits")


def test_prefill_vs_decode_vs_portions(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=2, page_size=4)
    tk = toks(61, raw["vocab"], 9)
    want = O.forward(raw, w, tk)
    close(run_portions(model, tk, [61]), want, 4e-5, "whole prompt")
    close(run_portions(model, tk, []), want, 4e-5, "token by token")
    for cuts in ([2, 2, 2, 2], [3, 5, 7, 11, 13], [1, 4, 4, 4, 30], [59, 2], [31], [8, 8, 8], [7, 2, 7, 2]):
        close(run_portions(model, tk, cuts), want, 4e-5, f"portions {cuts}")


def test_unequal_batch_equals_each_alone(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=3, page_size=4)
    reqs = {"a": toks(37, 50, 1), "b": toks(5, 50, 2), "c": toks(22, 50, 3), "d": toks(1, 50, 4)}
    want = {k: O.forward(raw, w, v) for k, v in reqs.items()}
    s = sched(model, max_tokens=256)
    plan = [[("a", 9), ("b", 2), ("c", 22)], [("a", 1), ("b", 1), ("d", 1)], [("a", 20), ("b", 2)], [("a", 7)]]
    at, got = {k: 0 for k in reqs}, {k: [] for k in reqs}
    for step in plan:
        lg = s.step([(k, reqs[k][at[k]:at[k] + n], list(range(n))) for k, n in step]).cpu().numpy()
        o = 0
        for k, n in step:
            got[k].append(lg[o:o + n])
            o += n
            at[k] += n
    for k in reqs:
        assert at[k] == len(reqs[k])
        close(np.concatenate(got[k], 0), want[k], 4e-5, f"request {k} in a mixed batch")


def test_pages_and_slots_are_reused(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=4, page_size=4)
    s = sched(model, max_tokens=48, max_requests=2)             # 12 pages, 2 slots: every later request runs on used ones
    free0 = s.kv_cache.free_page_count
    for i in range(5):
        a, b = toks(23 + i, 50, 10 + i), toks(9 + 2 * i, 50, 20 + i)
        la = s.step([("a", a[:10], list(range(10))), ("b", b, list(range(len(b))))]).cpu().numpy()
        s.finish("b")
        lb = s.step([("a", a[10:], list(range(len(a) - 10)))]).cpu().numpy()
        s.finish("a")
        close(np.concatenate([la[:10], lb], 0), O.forward(raw, w, a), 4e-5, f"pass {i}, request a")
        close(la[10:], O.forward(raw, w, b), 4e-5, f"pass {i}, request b")
        assert s.kv_cache.free_page_count == free0 and s.state_pool.free_slot_count == 2
    with pytest.raises(RuntimeError):
        s.step([("x", toks(60, 50, 1), [])])                    # more pages than the pool has


def test_chunk_edges_and_page_borders_with_peaked_scores(seq):
    """Query and key norm weights scaled up so that single keys carry the softmax: a key one off a chunk's edge or a lost page moves
    the logits by far more than the tolerance (checked on the oracle itself first).  Chunks of 6 and 10 on pages of 4: every chunk
    edge falls somewhere else in a page."""
    layers = [L(attn_cfg(heads=2, kv_heads=1, dim=16, vdim=16, chunk=6, rot_dims=8), dense(ff=48)),
              L(attn_cfg(heads=3, kv_heads=3, dim=8, vdim=8, chunk=10, rot_dims=8))]
    raw = model_cfg(layers)
    model, w = build(raw, seed=6, page_size=4, tweak=_peaky(["q.norm", "k.norm"], 3.0))
    tk = toks(45, raw["vocab"], 3)
    want = O.forward(raw, w, tk)
    for delta in (1, -1):
        other = json.loads(json.dumps(raw))
        other["layers"][0]["mixer"]["mask"]["size"] += delta
        moved = np.abs(O.forward(other, w, tk) - want).max(-1) / np.abs(want).max()
        assert (moved > 1e-2).sum() > 10, "the oracle must be sensitive to the chunk size"
    for cuts in ([45], [], [6, 6, 6], [5, 2, 5, 2, 5], [7, 7, 7, 7], [13, 2, 19]):
        close(run_portions(model, tk, cuts), want, 5e-5, f"portions {cuts}")


def test_far_key_stands_out_among_hundreds(seq):
    """The second layer's keys use its query projection, with peaked scores: a token that appears once, far back, and again near the
    end is found there across 300 positions (its value differs, because the first layer mixed other neighbours into it).  The oracle
    is checked to move by far more than the tolerance when that far token is replaced."""
    layers = [L(attn_cfg(heads=2, kv_heads=1, dim=8, vdim=8, chunk=4, rot_dims=4), dense(ff=32)),
              L(attn_cfg(heads=2, kv_heads=1, dim=16, vdim=24, chunk=512, rot_dims=0, diff=0.2, scale=1.0), dense(ff=32))]
    raw = model_cfg(layers, vocab=40)

    def tweak(w):
        w["l1.mix.q.norm"] = (w["l1.mix.q.norm"] * 2.5).to(torch.bfloat16).float()
        w["l1.mix.k.norm"] = w["l1.mix.q.norm"].clone()
        w["l1.mix.k"], w["l1.mix.k.b"] = w["l1.mix.q"][:32].clone(), w["l1.mix.q.b"][:32].clone()   # head 0's queries look for their own token
    model, w = build(raw, seed=8, page_size=64, tweak=tweak)
    tk = toks(330, 39, 4)
    marks = (-12, -7, -1)
    tk[5] = 39
    for i in marks:
        tk[i] = 39
    want = O.forward(raw, w, tk)
    gone = list(tk)
    gone[5] = 0
    moved = np.abs(O.forward(raw, w, gone) - want).max(-1) / np.abs(want).max()
    assert all(moved[i] > 1e-2 for i in marks)
    close(run_portions(model, tk, [330]), want, 5e-5, "whole prompt")
    close(run_portions(model, tk, [300]), want, 5e-5, "decoded over a far key")
    close(run_portions(model, tk, [128, 2, 100, 64]), want, 5e-5, "portions")


def test_first_tokens_and_single_token_requests(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=11, page_size=4)
    for n in (1, 2, 3):
        tk = toks(n, 50, n)
        close(run_portions(model, tk, [n]), O.forward(raw, w, tk), 4e-5, f"{n}-token request")
    s = sched(model)
    lg = s.step([("p", [7], [0]), ("q", [7], [0]), ("r", [3, 7], [1])]).cpu().numpy()
    close(lg[0], O.forward(raw, w, [7])[0], 4e-5, "one token")
    assert np.allclose(lg[0], lg[1], rtol=0, atol=1e-6)
    close(lg[2], O.forward(raw, w, [3, 7])[1], 4e-5, "second token")


def test_long_decoding_over_many_chunks(seq):
    raw = model_cfg([L(attn_cfg(chunk=16), dense()), L(attn_cfg(kv_from=0, chunk=48), moe())])
    model, w = build(raw, seed=12, page_size=8)
    tk = toks(170, 50, 6)
    close(run_portions(model, tk, [3]), O.forward(raw, w, tk), 5e-5, "167 decoded tokens")


@pytest.mark.parametrize("layers", [
    [L(attn_cfg(heads=1, kv_heads=1, dim=2, vdim=1, chunk=1, rot_dims=2, diff=0.0)), L(attn_cfg(heads=1, kv_heads=1, dim=2, vdim=1, chunk=2, rot_dims=2, kv_from=0), moe(experts=1, identity=0, top=1, groups=1, keep=1, ff=3, shared=0))],
    [L(attn_cfg(heads=5, kv_heads=5, dim=20, vdim=20, chunk=1000, rot_dims=20, factor=1.0, base=100.0), moe(experts=2, identity=6, top=4, groups=4, keep=3, ff=8, shared=8)),
     L(attn_cfg(heads=10, kv_heads=5, dim=20, vdim=20, chunk=3, rot_dims=4, kv_from=0), moe(experts=9, identity=1, top=2, groups=2, keep=2, ff=130, shared=0)),
     L(attn_cfg(heads=2, kv_heads=2, dim=34, vdim=130, chunk=11, rot_dims=6), dense(ff=7, limit=5.0))],
])
def test_other_sizes_and_degenerate_values(seq, layers):
    raw = model_cfg(layers, width=36, vocab=23, scale=1.0, eps=1e-3)
    model, w = build(raw, seed=13, page_size=2)
    tk = toks(27, 23, 8)
    want = O.forward(raw, w, tk)
    close(run_portions(model, tk, [27]), want, 5e-5, "whole")
    close(run_portions(model, tk, [4, 2, 9]), want, 5e-5, "portions")


def test_bfloat16_serving_close_to_oracle(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, dtype=torch.bfloat16, seed=14, page_size=4)
    tk = toks(40, 50, 2)
    want = O.forward(raw, w, tk)
    a, b = run_portions(model, tk, [40]), run_portions(model, tk, [9, 2, 13])
    close(a, want, 6e-2, "bf16 whole")
    close(b, want, 6e-2, "bf16 portions")
    close(b, a.astype(np.float64), 6e-2, "bf16: portions against whole")


def test_greedy_generation_through_the_entry_point(seq):
    """Scheduler.generate (admission, portions under a token budget, decode beside prefill, slot and page reuse) against greedy
    decoding with the oracle.  Steps whose two best logits are closer than the comparison tolerance end the comparison of a prompt."""
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=9, page_size=4)
    prompts = [toks(n, 50, 50 + n) for n in (19, 3, 33, 8, 1, 12)]
    s = sched(model, max_tokens=160, max_requests=3)
    outs = s.generate(prompts, max_new_tokens=12, step_tokens=16)
    assert s.kv_cache.free_page_count == 40 and s.state_pool.free_slot_count == 3 and not s.live
    checked = 0
    for p, out in zip(prompts, outs):
        assert len(out) == 12
        seqn = list(p)
        for tok in out:
            lg = O.forward(raw, w, seqn)[-1]
            top = np.sort(lg)[-2:]
            if top[1] - top[0] < 1e-3 * np.abs(lg).max():
                break
            assert tok == int(np.argmax(lg))
            seqn.append(tok)
            checked += 1
    assert checked >= 40


def test_decode_steps_replayed_from_cuda_graphs_equal_eager_steps(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=17, page_size=4)
    a, b = toks(70, 50, 1), toks(60, 50, 2)
    outs = []
    for graphs in (False, True):
        s = sched(model, max_tokens=512, max_requests=3, cuda_graphs=graphs)
        got = [s.step([("a", a[:20], [19]), ("b", b[:5], [4])])]
        for i in range(40):
            got.append(s.step([("a", [a[20 + i]], [0]), ("b", [b[5 + i]], [0])]))
        s.finish("b")
        for i in range(8):
            got.append(s.step([("a", [a[60 + i]], [0])]))
        outs.append([g.clone() for g in got])
        if graphs:
            assert sum(1 for v in s._graphs.values() if v) >= 2
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    close(outs[1][-1][0].cpu().numpy(), O.forward(raw, w, a[:68])[67], 5e-5, "last decoded token of request a")


def test_registry_loads_a_checkpoint_directory_and_the_trace_runner_replays_it(seq, tmp_path, monkeypatch, capsys):
    import io
    import sys
    from krasis_b200 import trace_runner
    from krasis_b200.megolorn import MegolornConfig, random_weights
    from krasis_b200.registry import architecture_of, load_model
    raw = model_cfg(default_layers())
    w = random_weights(MegolornConfig.from_dict(raw), 10)
    header, blobs, off = {}, [], 0
    for k, v in w.items():
        b = v.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert architecture_of(str(tmp_path)) == "Megolorn"
    tk = toks(25, 50, 14)
    want = O.forward(raw, {k: v.numpy().astype(np.float64) for k, v in w.items()}, tk)
    close(run_portions(load_model(str(tmp_path), dtype=torch.float32), tk, [25]), want, 4e-5, "loaded checkpoint")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tk[:10], "want": [0, 9]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": tk[10:12], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": tk[12:], "want": [12]}, {"id": "y", "tokens": tk[:3], "want": [2]}], "end": ["x", "y"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out = tmp_path / "out"
    assert trace_runner.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    assert [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    close(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), want[[0, 9]], 4e-5, "step 0")
    close(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1), want[[24, 2]], 4e-5, "step 2")
