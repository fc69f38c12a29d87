"""Vofelix: a decoder-only design of pre/post-normed layers whose mixers are either windowed latent attention with a softmax sink
or a gated delta rule, with an optional gated feed-forward, a per-layer token input, and a span of layers that is run several
times with the same weights (each run with a cache or state of its own; the embedding is added back before every later run).

config.json keys: architecture, vocab, width, embedding.scale, norm.eps, token_side.dim, loop {start, stop, times},
layers [{type: "latent_attention" | "delta", mixer: {...}, mlp: {kind: "dense", ff} | null}].
Tensor names: embed, side.embed, l<i>.norm1[.b], norm1b, norm2, norm2b, l<i>.mix.*, l<i>.mlp.{gate,up,down},
l<i>.side.{gate,proj,norm}, final.norm[.b], head.

The model exposes the step interface of `krasis_b200.scheduler`: `make_caches`, `forward_step(tables, want_rows)`.
The residual stream and every norm are fp32; `dtype` (bfloat16 or float32) is the type of weights, GEMM inputs and the cache.
"""
import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import seqops as ops
from .attention import LatentKVCache, RecurrentStatePool
from .mixers import GatedDeltaMixer, GatedMLP, TokenSideInput, WindowLatentAttention, lin


@dataclass
class VofelixConfig:
    vocab: int
    width: int
    embed_scale: float
    eps: float
    layers: List[dict]
    side_dim: int = 0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    raw: dict = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "VofelixConfig":
        loop = raw.get("loop") or {}
        side = raw.get("token_side") or {}
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), embed_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                  eps=float(raw["norm"]["eps"]), layers=list(raw["layers"]), side_dim=int(side.get("dim", 0)),
                  loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)), raw=raw)
        for L in cfg.layers:
            if L["type"] not in ("latent_attention", "delta"):
                raise ValueError(f"unknown mixer type {L['type']!r}")
            if L.get("mlp") and L["mlp"].get("kind", "dense") != "dense":
                raise ValueError(f"unknown feed-forward kind {L['mlp'].get('kind')!r}")
        n = len(cfg.layers)
        if not (0 <= cfg.loop_start <= cfg.loop_stop <= n):
            raise ValueError("loop span outside the layer list")
        return cfg

    def runs(self):
        """[(layer index, True if the embedding is added back right before this run)] in execution order."""
        n = len(self.layers)
        if self.loop_times <= 1 or self.loop_stop <= self.loop_start:
            return [(i, False) for i in range(n)]
        out = [(i, False) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            out += [(i, t > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, False) for i in range(self.loop_stop, n)]


def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):].replace(".", "_"): v for k, v in weights.items() if k.startswith(prefix)}


def random_weights(cfg: VofelixConfig, seed: int = 0, std: float = 0.05) -> dict:
    """Random tensors of the design's names and shapes (bf16-representable fp32 on the CPU): tests and benchmarks."""
    g = torch.Generator().manual_seed(seed)
    W = cfg.width
    r = lambda *s, sd=std: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16).float()
    nw = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).float()
    w = {"embed": r(cfg.vocab, W, sd=1.0 / max(cfg.embed_scale, 1e-6)), "head": r(cfg.vocab, W, sd=W ** -0.5),
         "final.norm": nw(W), "final.norm.b": r(W)}
    if cfg.side_dim:
        w["side.embed"] = r(cfg.vocab, cfg.side_dim * len(cfg.layers), sd=1.0)
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L["mixer"]
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if L.get("mlp") else [])
        for nm in names:
            w[p + nm], w[p + nm + ".b"] = nw(W), r(W)
        if L["type"] == "latent_attention":
            H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w.update({p + "mix.q": r(H * (dn + dr), W, sd=W ** -0.5 * 2), p + "mix.dkv": r(rk + dr, W, sd=W ** -0.5 * 2),
                      p + "mix.dkv.norm": nw(rk), p + "mix.uk": r(H * dn, rk, sd=rk ** -0.5 * 2), p + "mix.uv": r(H * dv, rk, sd=rk ** -0.5),
                      p + "mix.sink": r(H, sd=1.0), p + "mix.o": r(W, H * dv, sd=(H * dv) ** -0.5)})
        else:
            H, Hk, dk, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for nm, rows in (("q", Hk * dk), ("k", Hk * dk), ("v", H * dv)):
                w[p + "mix." + nm] = r(rows, W, sd=W ** -0.5 * 2)
                w[p + f"mix.{nm}.conv"] = r(rows, K, sd=0.5)
            w.update({p + "mix.g": r(H * dv, W, sd=W ** -0.5), p + "mix.a": r(H, W, sd=W ** -0.5), p + "mix.b": r(H, W, sd=W ** -0.5),
                      p + "mix.A_log": r(H, sd=0.5), p + "mix.dt_bias": r(H, sd=0.5), p + "mix.norm": nw(dv),
                      p + "mix.o": r(W, H * dv, sd=(H * dv) ** -0.5)})
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            w.update({p + "mlp.gate": r(F, W, sd=W ** -0.5), p + "mlp.up": r(F, W, sd=W ** -0.5), p + "mlp.down": r(W, F, sd=F ** -0.5)})
        if cfg.side_dim:
            w.update({p + "side.gate": r(cfg.side_dim, W, sd=W ** -0.5), p + "side.proj": r(W, cfg.side_dim, sd=cfg.side_dim ** -0.5),
                      p + "side.norm": nw(W)})
    return w


class VofelixModel:
    """Weights on the device plus the step function; caches and state slots are made by `make_caches` for a serving session."""

    architecture = "Vofelix"
    page_size = 64

    def __init__(self, cfg: VofelixConfig, weights: dict, dtype=torch.bfloat16, device=0):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype: bfloat16 or float32")
        if not torch.cuda.is_available():
            raise RuntimeError("VofelixModel needs a CUDA device (krasis_b200 has no CPU path)")
        ops.load()
        self.cfg, self.dtype = cfg, dtype
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        dev, W, eps = self.device, cfg.width, cfg.eps
        d = lambda t: t.to(device=dev, dtype=dtype).contiguous()
        f = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()
        self.embed, self.head = d(weights["embed"]), d(weights["head"])
        self.final_norm = (f(weights["final.norm"]), f(weights["final.norm.b"]))
        self.side_table = d(weights["side.embed"]) if cfg.side_dim else None
        self.layers = []
        for i, L in enumerate(cfg.layers):
            p, m = f"l{i}.", L["mixer"]
            lay = {"type": L["type"]}
            for nm in ("norm1", "norm1b", "norm2", "norm2b"):
                if p + nm in weights:
                    lay[nm] = (f(weights[p + nm]), f(weights[p + nm + ".b"]))
            mw = _sub(weights, p + "mix.")
            if L["type"] == "latent_attention":
                rot = m.get("rot") or {}
                lay["mixer"] = WindowLatentAttention(mw, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"],
                                                     (m.get("mask") or {}).get("size"), rot.get("dims", 0 if not rot else m["rot_dim"]),
                                                     rot.get("base", 10000.0), rot.get("scaling"), eps, dtype, dev)
            else:
                lay["mixer"] = GatedDeltaMixer(mw, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], eps, dtype, dev)
            lay["mlp"] = GatedMLP(_sub(weights, p + "mlp."), dtype, dev) if L.get("mlp") else None
            lay["side"] = TokenSideInput(_sub(weights, p + "side."), self.side_table, i * cfg.side_dim, cfg.side_dim, dtype, dev) \
                if cfg.side_dim else None
            self.layers.append(lay)
        self.runs = cfg.runs()

    # ------------------------------------------------------------------------------------------- construction
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype=torch.bfloat16, device=0, **_):
        from . import loader
        raw = json.load(open(os.path.join(model_dir, "config.json")))
        cfg = VofelixConfig.from_dict(raw)
        weights = loader.read_named_tensors(model_dir)
        return cls(cfg, weights, dtype=dtype, device=device)

    @classmethod
    def random(cls, cfg: VofelixConfig, seed: int = 0, dtype=torch.bfloat16, device=0):
        return cls(cfg, random_weights(cfg, seed), dtype=dtype, device=device)

    # ------------------------------------------------------------------------------------------- serving interface
    def make_caches(self, max_tokens: int, max_requests: int):
        """(paged cache, state pool) for a session that holds at most max_tokens tokens (each request rounded up to whole pages)
        in at most max_requests live requests.  Every run of a layer gets its own cache pool / state tensors."""
        pages = (max_tokens + self.page_size - 1) // self.page_size
        dims, self._run_cache, self._run_state = [], {}, {}
        pool = RecurrentStatePool(max_requests, self.device)
        for ri, (li, _) in enumerate(self.runs):
            mixer = self.layers[li]["mixer"]
            if isinstance(mixer, WindowLatentAttention):
                self._run_cache[ri] = len(dims)
                dims.append(mixer.cache_dims())
            else:
                self._run_state[ri] = mixer.register_state(pool)
        kv = LatentKVCache(dims, self.device, max_pages=max(pages, 1), dtype=self.dtype, page_size=self.page_size)
        self.kv_cache, self.state_pool = kv, pool
        return kv, pool

    def forward_step(self, tb: ops.StepTables, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every layer run; returns fp32 logits [len(want_rows), vocab] (None if nothing is wanted)."""
        cfg, eps, dt = self.cfg, self.cfg.eps, self.dtype
        x0 = ops.embed(self.embed, tb.tokens, cfg.embed_scale)
        x = x0.clone() if any(again for _, again in self.runs) else x0
        first = self.layers[self.runs[0][0]]
        h = ops.residual_norm(x, out_norm=first["norm1"], out_dtype=dt, eps=eps)
        for ri, (li, _) in enumerate(self.runs):
            lay = self.layers[li]
            nxt = self.runs[ri + 1] if ri + 1 < len(self.runs) else None
            nxt_norm = self.layers[nxt[0]]["norm1"] if nxt else self.final_norm
            nxt_x0 = x0 if (nxt and nxt[1]) else None
            nxt_dt = dt if nxt else torch.float32
            if lay["type"] == "latent_attention":
                ckv, kr = self.kv_cache.get_layer_caches(self._run_cache[ri])
                y = lay["mixer"].forward(h, tb, ckv, kr, self.kv_cache.page_size)
            else:
                tail, state = self._run_state[ri]
                y = lay["mixer"].forward(h, tb, tail, state)
            last_sub = lay["mlp"] is None and lay["side"] is None
            if lay["mlp"] is not None:
                h = ops.residual_norm(x, y, ("layer",) + lay["norm1b"], out_norm=lay["norm2"], out_dtype=dt, eps=eps)
                y = lay["mlp"].forward(h)
                if lay["side"] is None:
                    h = ops.residual_norm(x, y, ("layer",) + lay["norm2b"], x0=nxt_x0, out_norm=nxt_norm, out_dtype=nxt_dt, eps=eps)
                else:
                    ops.residual_norm(x, y, ("layer",) + lay["norm2b"], eps=eps)
            elif last_sub:
                h = ops.residual_norm(x, y, ("layer",) + lay["norm1b"], x0=nxt_x0, out_norm=nxt_norm, out_dtype=nxt_dt, eps=eps)
            else:
                ops.residual_norm(x, y, ("layer",) + lay["norm1b"], eps=eps)
            if lay["side"] is not None:
                y = lay["side"].forward(x, tb)
                h = ops.residual_norm(x, y, ("rms", lay["side"].norm), x0=nxt_x0, out_norm=nxt_norm, out_dtype=nxt_dt, eps=eps)
            if self.layer_trace is not None:
                self.layer_trace.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        hw = h.index_select(0, want_rows)            # fp32 rows of the final norm
        return lin(hw, self.head, torch.float32)

    layer_trace = None      # tests: set to a list to collect the residual stream after every layer run
