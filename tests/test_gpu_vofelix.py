"""Vofelix on the GPU against the plain float64 oracle (tests/oracle_vofelix.py): each mechanism alone, then the whole model
through the scheduler — prefill against decoding, portions down to one token, unequal batches, reuse of pages and state slots,
window and page edges, sinks, long decoding, odd sizes, and greedy generation through the generation entry point.
Small random configurations made here; none of them is a shipped model's."""
import numpy as np
import pytest
import torch

from tests import oracle_vofelix as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def seq():
    from krasis_b200.build import build_seq
    build_seq()
    from krasis_b200 import seqops
    seqops.load()
    return seqops


def latent_cfg(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, window=7, scale=None, rot_dims=None, scaling=True):
    rot = {"base": 5000.0, "dims": rot_dim if rot_dims is None else rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": rot,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window:
        m["mask"] = {"size": window}
    return m


def delta_cfg(heads=4, kv_heads=2, dim=24, vdim=40, conv=4):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def model_cfg(layers, width=96, vocab=50, side=6, loop=(1, 2, 2), scale=3.0, eps=1e-5):
    raw = {"architecture": "Vofelix", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
           "layers": layers, "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}}
    if side:
        raw["token_side"] = {"dim": side}
    return raw


def L(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def default_layers():
    return [L("delta", delta_cfg()), L("latent_attention", latent_cfg(), ff=80), L("delta", delta_cfg(heads=2, kv_heads=2, dim=16, vdim=16, conv=2), ff=40),
            L("latent_attention", latent_cfg(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=24, window=5, rot_dims=8))]


def build(raw, dtype=torch.float32, seed=0, page_size=None, tweak=None):
    from krasis_b200.vofelix import VofelixConfig, VofelixModel, random_weights
    cfg = VofelixConfig.from_dict(raw)
    w = random_weights(cfg, seed)
    if tweak:
        tweak(w)
    model = VofelixModel(cfg, w, dtype=dtype)
    if page_size:
        model.page_size = page_size
    return model, {k: v.numpy().astype(np.float64) for k, v in w.items()}


def sched(model, max_tokens=512, max_requests=4):
    from krasis_b200.scheduler import Scheduler
    return Scheduler(model, max_tokens=max_tokens, max_requests=max_requests)


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
        lg = s.step([(rid, tokens[at:at + n], list(range(n)))])
        out.append(lg.cpu().numpy())
        at += n
    if finish:
        s.finish(rid)
    return np.concatenate(out, 0)


# ------------------------------------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("M,N,K", [(1, 5, 7), (3, 33, 64), (8, 130, 200), (9, 64, 16), (70, 65, 33), (200, 96, 257)])
def test_gemm_any_shape_and_dtype(seq, M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N)
    for da in (torch.float32, torch.bfloat16):
        for dw in (torch.float32, torch.bfloat16):
            a = torch.randn(M, K, generator=g).to(da).cuda()
            w = torch.randn(N, K, generator=g).to(dw).cuda()
            want = a.double().cpu().numpy() @ w.double().cpu().numpy().T
            close(seq.gemm(a, w, torch.float32).cpu().numpy(), want, 2e-6, f"gemm {da} {dw}")
            close(seq.gemm(a, w, torch.bfloat16).float().cpu().numpy(), want, 5e-3, "gemm bf16 out")


def test_gemm_rows_do_not_depend_on_batch(seq):
    g = torch.Generator().manual_seed(1)
    a, w = torch.randn(100, 72, generator=g).cuda(), torch.randn(50, 72, generator=g).cuda()
    full = seq.gemm(a, w)
    part = seq.gemm(a[10:30].contiguous(), w)
    assert torch.equal(full[10:30], part)          # same K order per output whatever else is in the launch


def test_gemm_heads_strided(seq):
    g = torch.Generator().manual_seed(2)
    T, H, K, N = 11, 3, 10, 7
    big = torch.randn(T, H * (K + 4) + 5, generator=g).cuda()
    a = big[:, :H * (K + 4)].view(T, H, K + 4)[:, :, :K]
    w = torch.randn(H, N, K, generator=g).cuda()
    out = torch.empty(T, H, N, device="cuda")
    seq.gemm_heads(a, w, out)
    want = np.einsum("thk,hnk->thn", a.double().cpu().numpy(), w.double().cpu().numpy())
    close(out.cpu().numpy(), want, 2e-6, "gemm_heads")


@pytest.mark.parametrize("W", [8, 96, 250, 1030])
def test_residual_norm(seq, W):
    g = torch.Generator().manual_seed(W)
    T, eps = 5, 1e-5
    r = lambda *s: torch.randn(*s, generator=g).cuda()
    x, y, x0, wa, ba, wb, bb = r(T, W) * 3 + 1, r(T, W) * 2 + 0.5, r(T, W), r(W), r(W), r(W), r(W)
    n = lambda t: t.double().cpu().numpy()
    for mode in ("layer", "rms"):
        xx = x.clone()
        h = seq.residual_norm(xx, y, (mode, wa, ba) if mode == "layer" else (mode, wa), x0=x0, out_norm=(wb, bb), eps=eps)
        add = O.layer_norm(n(y), n(wa), n(ba), eps) if mode == "layer" else O.rms_norm(n(y), n(wa), eps)
        want_x = n(x) + add + n(x0)
        close(xx.cpu().numpy(), want_x, 2e-6, "x " + mode)
        close(h.cpu().numpy(), O.layer_norm(want_x, n(wb), n(bb), eps), 5e-6, "h " + mode)
    xx = x.clone()
    h = seq.residual_norm(xx, out_norm=(wb, bb), eps=eps)
    assert torch.equal(xx, x)
    close(h.cpu().numpy(), O.layer_norm(n(x), n(wb), n(bb), eps), 5e-6, "norm only")


def test_act_mul_and_side_gate(seq):
    g = torch.Generator().manual_seed(3)
    T, F, dim = 7, 13, 5
    gu = (torch.randn(T, 2 * F, generator=g) * 2).cuda()
    out = seq.act_mul(gu, torch.float32).cpu().numpy()
    a = gu.double().cpu().numpy()
    close(out, O.gelu_tanh(a[:, :F]) * a[:, F:], 2e-6, "act_mul")
    table = torch.randn(9, 4 * dim, generator=g).cuda()
    tok = torch.tensor([0, 8, 3, 3, 1, 7, 2], dtype=torch.int32).cuda()
    gg = torch.randn(T, dim, generator=g).cuda()
    got = seq.side_gate(gg, table, tok, 2 * dim, torch.float32).cpu().numpy()
    want = O.gelu_tanh(gg.double().cpu().numpy()) * table.double().cpu().numpy()[tok.cpu().numpy()][:, 2 * dim:3 * dim]
    close(got, want, 2e-6, "side_gate")


def test_yarn_table_matches_oracle(seq):
    from krasis_b200.mixers import yarn_table
    for dims, base, sc in [(8, 5000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}), (32, 1e5, None),
                           (16, 100.0, {"factor": 1.5, "original": 16, "fast": 2.0, "slow": 0.5})]:
        f, amp = yarn_table(dims, base, sc)
        fo, ao = O.yarn_frequencies(dims, base, sc)
        np.testing.assert_allclose(f.numpy(), fo, rtol=1e-13)
        assert abs(amp - ao) < 1e-15


def _one_layer(kind, mixer, ff=None, side=0, **kw):
    return model_cfg([L(kind, mixer, ff)], side=side, loop=(0, 0, 1), **kw)


@pytest.mark.parametrize("mixer", [latent_cfg(), latent_cfg(window=None), latent_cfg(heads=1, dim=8, rot_dim=0, vdim=8, kv_rank=8, window=3, scaling=False),
                                   latent_cfg(heads=9, dim=16, rot_dim=12, vdim=8, kv_rank=200, window=70, rot_dims=4),
                                   latent_cfg(scale=1.5, window=6)])
def test_latent_attention_alone(seq, mixer):
    raw = _one_layer("latent_attention", mixer)
    model, w = build(raw, seed=11)
    T = 90
    tk = toks(T, raw["vocab"], 5)
    got = run_portions(model, tk, [T])
    close(got, O.forward(raw, w, tk), 3e-5, "latent attention, whole prompt")
    got = run_portions(model, tk, [37, 2, 1, 20])
    close(got, O.forward(raw, w, tk), 3e-5, "latent attention, portions and decoding")


@pytest.mark.parametrize("mixer", [delta_cfg(), delta_cfg(heads=1, kv_heads=1, dim=8, vdim=8, conv=1), delta_cfg(heads=6, kv_heads=2, dim=40, vdim=24, conv=3),
                                   delta_cfg(heads=2, kv_heads=2, dim=16, vdim=72, conv=5),
                                   # key sizes 32 / 64 / 128 with value sizes in multiples of 32 run the register-state kernels
                                   delta_cfg(heads=2, kv_heads=1, dim=32, vdim=32, conv=3), delta_cfg(heads=3, kv_heads=3, dim=64, vdim=64, conv=4),
                                   delta_cfg(heads=2, kv_heads=2, dim=128, vdim=96, conv=2),
                                   delta_cfg(heads=66, kv_heads=2, dim=32, vdim=32, conv=2)])      # 33 heads share a key head
def test_delta_mixer_alone(seq, mixer):
    raw = _one_layer("delta", mixer)
    model, w = build(raw, seed=12)
    T = 70
    tk = toks(T, raw["vocab"], 6)
    want = O.forward(raw, w, tk)
    close(run_portions(model, tk, [T]), want, 3e-5, "delta, whole prompt")
    close(run_portions(model, tk, [17, 2, 3, 1, 30]), want, 3e-5, "delta, portions and decoding")
    close(run_portions(model, tk, []), want, 3e-5, "delta, token by token")


def test_latent_attention_bfloat16_cache_and_decode_grids(seq):
    """bf16 cache rows read 8 values at a time (latent and rotated sizes in multiples of 8); a step of few tokens runs one head per
    block with the dot products cut into pieces, a long portion runs 8 heads per block: both against the oracle and each other."""
    raw = _one_layer("latent_attention", latent_cfg(heads=16, dim=16, rot_dim=8, vdim=16, kv_rank=64, window=40), width=64)
    tk = toks(120, raw["vocab"], 15)
    for dtype, tol in ((torch.float32, 3e-5), (torch.bfloat16, 4e-2)):
        model, w = build(raw, dtype=dtype, seed=14)
        want = O.forward(raw, w, tk)
        a = run_portions(model, tk, [120])
        b = run_portions(model, tk, [100])           # 100 at once (8 heads per block), then 20 single tokens (1 head per block)
        close(a, want, tol, f"{dtype} whole")
        close(b, want, tol, f"{dtype} portion + decoding")


def test_tensor_core_prefill_of_latent_attention(seq):
    """bfloat16, 128 + 64 query / key dims, 128 value dims: portions of 128 tokens or more run the tcgen05 attention core on keys and
    values up-projected from the cached latents.  Against the oracle, and against the plain kernel on the same bf16 cache, with peaked
    scores and heavy sinks, windows that end inside, at and across KV tiles, portions that start in the middle of a window."""
    from krasis_b200.build import build as build_core
    build_core()
    for window, sink_shift, scale in ((100, 2.0, 0.25), (64, 0.0, 0.15), (333, 3.0, 0.3), (None, 1.0, 0.2)):
        raw = _one_layer("latent_attention", latent_cfg(heads=2, dim=128, rot_dim=64, vdim=128, kv_rank=64, window=window, scale=scale), width=64)

        def tweak(w):
            for k in w:
                if k.endswith("mix.sink"):
                    w[k] = w[k] + sink_shift
        model, w = build(raw, dtype=torch.bfloat16, seed=31, tweak=tweak)
        mixer = model.layers[0]["mixer"]
        assert mixer.tc_shape
        tk = toks(700, raw["vocab"], 16)
        want = O.forward(raw, w, tk)
        if window:                                  # the window's edge must move the logits by far more than the tolerances below
            wide = {**raw, "layers": [{**raw["layers"][0], "mixer": {**raw["layers"][0]["mixer"], "mask": {"size": window + 1}}}]}
            assert np.abs(O.forward(wide, w, tk) - want).max() > 0.15 * np.abs(want).max()
        fast_whole = run_portions(model, tk, [700], s=sched(model, 1024))
        fast_parts = run_portions(model, tk, [130, 257, 128, 150], s=sched(model, 1024))          # then 35 single tokens through the plain kernel
        mixer.tc_min_portion = 1 << 30
        plain = run_portions(model, tk, [700], s=sched(model, 1024))
        mixer.tc_min_portion = 128
        close(plain, want, 5e-2, f"window {window}: plain kernel against the oracle")
        close(fast_whole, want, 5e-2, f"window {window}: tensor-core prefill against the oracle")
        close(fast_whole, plain, 3e-2, f"window {window}: tensor-core prefill against the plain kernel")
        close(fast_parts, plain, 3e-2, f"window {window}: tensor-core portions against the plain kernel")


def test_mlp_and_side_alone(seq):
    raw = _one_layer("delta", delta_cfg(), ff=72, side=10)
    model, w = build(raw, seed=13)
    tk = toks(20, raw["vocab"], 7)
    close(run_portions(model, tk, [20]), O.forward(raw, w, tk), 3e-5, "feed-forward + token side input")


def test_layer_trace_matches_oracle(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=1)
    tk = toks(33, raw["vocab"], 8)
    model.layer_trace = []
    s = sched(model)
    s.step([("a", tk, [])])
    _, trace = O.forward(raw, w, tk, return_layers=True)
    assert len(model.layer_trace) == trace.shape[0] == 5          # the looped layer runs twice
    for i, x in enumerate(model.layer_trace):
        want = trace[i]
        if i + 1 < trace.shape[0] and model.runs[i + 1][1]:          # the fused kernel has already added the embedding for the next pass
            want = want + w["embed"][tk] * raw["embedding"]["scale"]
        close(x.cpu().numpy(), want, 3e-5, f"residual stream after layer run {i}")


# ------------------------------------------------------------------------------------------------ whole model through the scheduler

def test_prefill_vs_decode_vs_portions(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=2, page_size=4)
    tk = toks(61, raw["vocab"], 9)
    want = O.forward(raw, w, tk)
    close(run_portions(model, tk, [61]), want, 4e-5, "whole prompt")
    close(run_portions(model, tk, []), want, 4e-5, "token by token")
    for cuts in ([2, 2, 2, 2], [3, 5, 7, 11, 13], [1, 4, 4, 4, 30], [59, 2], [31]):
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
        ents = [(k, reqs[k][at[k]:at[k] + n], list(range(n))) for k, n in step]
        lg = s.step(ents).cpu().numpy()
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
        close(np.concatenate([la[:10], lb], 0), O.forward(raw, w, a), 4e-5, f"round {i}, request a")
        close(la[10:], O.forward(raw, w, b), 4e-5, f"round {i}, request b")
        assert s.kv_cache.free_page_count == free0 and s.state_pool.free_slot_count == 2
    with pytest.raises(RuntimeError):
        s.step([("x", toks(60, 50, 1), [])])                    # more pages than the pool has


def _peaky(names, factor):
    def tweak(w):
        for k in list(w):
            if any(k.endswith(n) for n in names):
                w[k] = (w[k] * factor).to(torch.bfloat16).float()
    return tweak


def test_window_edges_pages_and_sink_with_peaked_scores(seq):
    """Scores scaled up so single keys carry the softmax: a key one off the window's edge, a lost page or a missing sink moves the
    logits by far more than the tolerance.  Sinks are made large enough to hold a visible share of every softmax."""
    layers = [L("latent_attention", latent_cfg(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=32, window=9, scale=2.0), ff=48),
              L("latent_attention", latent_cfg(heads=3, dim=8, rot_dim=8, vdim=8, kv_rank=16, window=16, scale=3.0))]
    raw = model_cfg(layers, side=0, loop=(0, 1, 2))

    def tweak(w):
        for k in w:
            if k.endswith("mix.sink"):
                w[k] = w[k] + 2.0
    model, w = build(raw, seed=5, page_size=4, tweak=tweak)
    tk = toks(45, 50, 11)
    want = O.forward(raw, w, tk)
    # the oracle itself must feel the window edge and the sink here, else the test shows nothing
    wide = {**raw, "layers": [{**l, "mixer": {**l["mixer"], "mask": {"size": l["mixer"]["mask"]["size"] + 1}}} for l in layers]}
    assert np.abs(O.forward(wide, w, tk) - want).max() > 1e-2 * np.abs(want).max()
    no_sink = {k: (v - 50.0 if k.endswith("mix.sink") else v) for k, v in w.items()}
    assert np.abs(O.forward(raw, no_sink, tk) - want).max() > 1e-2 * np.abs(want).max()
    close(run_portions(model, tk, [45]), want, 6e-5, "whole prompt")
    close(run_portions(model, tk, [8, 1, 1, 7, 2, 16]), want, 6e-5, "portions that end at window and page edges, then decoding")
    close(run_portions(model, tk, []), want, 6e-5, "decoding across window and page edges")


def test_far_key_through_recurrent_state(seq):
    """A delta-rule model must carry what the first tokens wrote over hundreds of steps: slow decay, long prompt, decoding tail."""
    layers = [L("delta", delta_cfg(heads=2, kv_heads=1, dim=16, vdim=16, conv=3)), L("delta", delta_cfg(heads=2, kv_heads=2, dim=16, vdim=16, conv=2), ff=32)]
    raw = model_cfg(layers, width=64, side=4, loop=(0, 0, 1))

    def tweak(w):
        for k in w:
            if k.endswith("A_log"):
                w[k] = w[k] - 6.0          # decay close to 1: the state remembers
    model, w = build(raw, seed=6, tweak=tweak)
    tk = toks(420, 50, 12)
    want = O.forward(raw, w, tk)
    other = list(tk)
    other[0] = (tk[0] + 1) % 50
    assert np.abs(O.forward(raw, w, other)[-1] - want[-1]).max() > 5e-4 * np.abs(want).max()      # the last logits still feel token 0
    got = run_portions(model, tk, [130, 2, 127, 11])                                             # then 150 tokens one by one
    close(got, want, 1e-4, "long prompt in portions + long decoding")


def test_first_tokens_and_single_token_requests(seq):
    raw = model_cfg(default_layers(), loop=(0, 4, 2))
    model, w = build(raw, seed=7, page_size=4)
    s = sched(model)
    for n in (1, 2, 3):
        tk = toks(n, 50, 30 + n)
        close(run_portions(model, tk, [n], s=s, rid=n), O.forward(raw, w, tk), 4e-5, f"{n}-token request")


def test_other_sizes_and_degenerate_values(seq):
    """Sizes the usual configurations make equal or 1: one head, kv_heads == heads, dk != dv, one tap, no loop, scale 1, no side input,
    a loop over the whole model, rotation on a part of the rotated dims."""
    variants = [
        model_cfg([L("latent_attention", latent_cfg(heads=1, dim=8, rot_dim=4, vdim=12, kv_rank=8, window=1), ff=8)], width=32, side=0, loop=(0, 0, 1), scale=1.0),
        model_cfg([L("delta", delta_cfg(heads=1, kv_heads=1, dim=8, vdim=24, conv=1)), L("delta", delta_cfg(heads=4, kv_heads=4, dim=32, vdim=8, conv=2))],
                  width=40, side=3, loop=(0, 2, 3)),
        model_cfg([L("latent_attention", latent_cfg(heads=5, dim=12, rot_dim=20, vdim=4, kv_rank=36, window=64, rot_dims=10), ff=100),
                   L("delta", delta_cfg(heads=3, kv_heads=1, dim=20, vdim=20, conv=4), ff=24)], width=72, vocab=31, side=7, loop=(1, 2, 4), eps=1e-3),
    ]
    for i, raw in enumerate(variants):
        model, w = build(raw, seed=20 + i, page_size=8)
        tk = toks(75, raw["vocab"], 40 + i)
        want = O.forward(raw, w, tk)
        close(run_portions(model, tk, [75]), want, 5e-5, f"variant {i}, whole")
        close(run_portions(model, tk, [5, 2, 40]), want, 5e-5, f"variant {i}, portions + decoding")


def test_bfloat16_serving_close_to_oracle(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, dtype=torch.bfloat16, seed=8, page_size=4)
    tk = toks(50, raw["vocab"], 13)
    want = O.forward(raw, w, tk)
    a = run_portions(model, tk, [50])
    b = run_portions(model, tk, [7, 2, 20])
    close(a, want, 6e-2, "bf16 whole")
    close(b, want, 6e-2, "bf16 portions")
    close(a, b, 4e-2, "bf16 whole against portions")


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
    """Decode steps captured per (live requests, page-list width) and replayed: bit-identical logits, over page borders (new
    page-list widths re-capture), with a request joining and one leaving, and a prompt portion in between (eager)."""
    from krasis_b200.scheduler import Scheduler
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=17, page_size=4)
    a, b, c = toks(90, 50, 1), toks(70, 50, 2), toks(40, 50, 3)
    outs = []
    for graphs in (False, True):
        s = Scheduler(model, max_tokens=512, max_requests=3, cuda_graphs=graphs)
        got = [s.step([("a", a[:20], [19]), ("b", b[:5], [4])])]
        for i in range(40):
            got.append(s.step([("a", [a[20 + i]], [0]), ("b", [b[5 + i]], [0])]))
        got.append(s.step([("c", c[:30], [29]), ("a", [a[60]], [0])]))
        for i in range(10):
            got.append(s.step([("a", [a[61 + i]], [0]), ("b", [b[45 + i]], []), ("c", [c[30 + i]], [0])]))
        s.finish("b")
        for i in range(10):
            got.append(s.step([("c", [c[30 + i]], [0]), ("a", [a[71 + i]], [0])]))
        outs.append([g.clone() for g in got])
        if graphs:
            assert sum(1 for v in s._graphs.values() if v) >= 3
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    want = O.forward(raw, w, a[:81])
    close(outs[1][-1][1].cpu().numpy(), want[80], 5e-5, "last decoded token of request a")


def test_registry_loads_a_checkpoint_directory(seq, tmp_path):
    """config.json + model.safetensors on disk -> registry -> model -> same logits as the oracle."""
    import json
    import struct
    from krasis_b200.registry import architecture_of, load_model
    from krasis_b200.vofelix import VofelixConfig, random_weights
    raw = model_cfg(default_layers())
    w = random_weights(VofelixConfig.from_dict(raw), 10)
    header, blobs, off = {}, [], 0
    for k, v in w.items():
        b = v.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert architecture_of(str(tmp_path)) == "Vofelix"
    model = load_model(str(tmp_path), dtype=torch.float32)
    tk = toks(25, 50, 14)
    w64 = {k: v.numpy().astype(np.float64) for k, v in w.items()}
    want = O.forward(raw, w64, tk)
    close(run_portions(model, tk, [25]), want, 4e-5, "loaded checkpoint")

    # the trace runner on the same directory: steps from standard input, logits of the wanted places to <step>.f32, "done <step>" lines
    import io
    import sys
    from krasis_b200 import trace_runner
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tk[:10], "want": [0, 9]}, {"id": "y", "tokens": tk[:3], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "y", "tokens": tk[3:4], "want": []}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": tk[10:25], "want": [14]}, {"id": "z", "tokens": tk[:2], "want": [1]}], "end": ["x", "z"]}]
    out_dir = tmp_path / "out"
    stdin, stdout = sys.stdin, sys.stdout
    sys.stdin, sys.stdout = io.StringIO("".join(json.dumps(x) + "\n" for x in steps)), io.StringIO()
    try:
        rc = trace_runner.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(out_dir), "--max-tokens", "128"])
        printed = sys.stdout.getvalue()
    finally:
        sys.stdin, sys.stdout = stdin, stdout
    assert rc == 0 and [l for l in printed.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out_dir / "1.f32").exists()
    got0 = np.fromfile(out_dir / "0.f32", dtype="<f4").reshape(2, -1)
    got2 = np.fromfile(out_dir / "2.f32", dtype="<f4").reshape(2, -1)
    close(got0, want[[0, 9]], 4e-5, "trace step 0")
    close(got2, np.stack([want[24], want[1]]), 4e-5, "trace step 2")

    # the generation command line: greedy ids for two prompts, one JSON line each
    from krasis_b200.__main__ import main as cli
    sys.stdout = io.StringIO()
    try:
        rc = cli(["generate", "--model", str(tmp_path), "--dtype", "float32", "--prompt-ids", ",".join(map(str, tk[:7])), "--prompt-ids", "3,4",
                  "--max-new-tokens", "3", "--max-tokens", "256"])
        lines = [json.loads(l) for l in sys.stdout.getvalue().splitlines() if l.startswith("{")]
    finally:
        sys.stdout = stdout
    assert rc == 0 and [x["prompt_tokens"] for x in lines] == [7, 2] and all(len(x["generated"]) == 3 for x in lines)
    first = O.forward(raw, w64, tk[:7])[-1]
    if np.sort(first)[-1] - np.sort(first)[-2] > 1e-3 * np.abs(first).max():
        assert lines[0]["generated"][0] == int(np.argmax(first))
