"""Megolorn: a decoder-only design of parallel layers — one layer norm (weight, no bias) whose output feeds both the mixer and the
feed-forward, x <- x + (mixer(h) + ff(h)).  The mixer is differential attention: every query head carries two attention maps with
keys of their own over shared values, combined as a1 - lambda a2 with one lambda per layer, unit-normed per head and gated per
head; grouped key/value heads with biases, RMS norm on queries and keys, interleaved rotary positions on part of the dimensions with
linear scaling, a causal mask cut into chunks counted from position 0; a layer may read an earlier layer's cached keys and values
instead of projecting its own.  The feed-forward is dense (clamped swish form) or a mixture of SiLU experts with a softmax router,
a choice correction, expert groups, identity experts and a shared expert.

config.json keys: architecture, vocab, width, embedding.scale, norm.eps,
layers [{type: "attention", mixer: {heads, kv_heads, dim, vdim, scale, diff, mask.size, rot {base, dims, scaling.factor}, kv_from},
         mlp: null | {kind: "dense", ff, limit} | {kind: "moe", expert.ff, router {experts, identity, top, groups {count, keep}},
                      shared.ff}}].
Tensor names: embed, l<i>.norm1, l<i>.mix.{q, k, v}[.b], l<i>.mix.{q, k}.norm, l<i>.mix.{lq1, lk1, lq2, lk2, g, o},
l<i>.mlp.{gate, up, down} | l<i>.mlp.{router, correction, e<j>.{gate, up, down}, shared.{gate, up, down}}, final.norm, head.

The model exposes the step interface of `krasis_b200.scheduler`: `make_caches`, `forward_step(tables, want_rows)`.
The residual stream and every norm are fp32; `dtype` (bfloat16 or float32) is the type of weights, GEMM inputs and the cache.
"""
import json
import math
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import seqops as ops
from .attention import HeadKVCache, RecurrentStatePool
from .mixers import GatedMLP, MultiMapAttention, RoutedExperts, lin

SWISH_ALPHA = 1.702      # slope inside the sigmoid of the dense feed-forward's activation
MAPS = 2                 # attention maps per head


@dataclass
class MegolornConfig:
    vocab: int
    width: int
    embed_scale: float
    eps: float
    layers: List[dict]
    raw: dict = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "MegolornConfig":
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), embed_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                  eps=float(raw["norm"]["eps"]), layers=list(raw["layers"]), raw=raw)
        for i, L in enumerate(cfg.layers):
            if L["type"] != "attention":
                raise ValueError(f"unknown mixer type {L['type']!r}")
            m = L["mixer"]
            if m["heads"] % m["kv_heads"]:
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            src = m.get("kv_from")
            if src is not None:
                if not 0 <= src < i or cfg.layers[src]["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer that projects its own keys and values")
                sm = cfg.layers[src]["mixer"]
                if (sm["kv_heads"], sm["dim"], sm["vdim"]) != (m["kv_heads"], m["dim"], m["vdim"]):
                    raise ValueError(f"layer {i}: key/value sizes differ from layer {src}'s")
            mlp = L.get("mlp")
            if mlp and mlp.get("kind", "dense") not in ("dense", "moe"):
                raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        return cfg


def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):].replace(".", "_"): v for k, v in weights.items() if k.startswith(prefix)}


def random_weights(cfg: MegolornConfig, seed: int = 0) -> dict:
    """Random tensors of the design's names and shapes (bf16-representable fp32 on the CPU): tests and benchmarks."""
    g = torch.Generator().manual_seed(seed)
    W = cfg.width
    r = lambda *s, sd=1.0: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16).float()
    nw = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).float()
    w = {"embed": r(cfg.vocab, W, sd=1.0 / max(cfg.embed_scale, 1e-6)), "head": r(cfg.vocab, W, sd=W ** -0.5), "final.norm": nw(W)}
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w[p + "norm1"] = nw(W)
        names = [("q", H * MAPS * d)] + ([("k", G * MAPS * d), ("v", G * dv)] if m.get("kv_from") is None else [])
        for nm, rows in names:
            w[p + "mix." + nm] = r(rows, W, sd=W ** -0.5 * (1.0 if nm == "v" else 2.0))
            w[p + f"mix.{nm}.b"] = r(rows, sd=0.1)
            if nm != "v":
                w[p + f"mix.{nm}.norm"] = nw(d)
        for nm in ("lq1", "lk1", "lq2", "lk2"):
            w[p + "mix." + nm] = r(d, sd=0.1)
        w[p + "mix.g"] = r(H, W, sd=W ** -0.5)
        w[p + "mix.o"] = r(W, H * dv, sd=(H * dv) ** -0.5)
        mlp = L.get("mlp")
        if mlp and mlp.get("kind", "dense") == "dense":
            F = mlp["ff"]
            w.update({p + "mlp.gate": r(F, W, sd=W ** -0.5), p + "mlp.up": r(F, W, sd=W ** -0.5), p + "mlp.down": r(W, F, sd=F ** -0.5)})
        elif mlp:
            rt, F = mlp["router"], mlp["expert"]["ff"]
            n = rt["experts"] + rt.get("identity", 0)
            w[p + "mlp.router"] = r(n, W, sd=W ** -0.5 * 2)
            w[p + "mlp.correction"] = r(n, sd=0.05)
            for e in range(rt["experts"]):
                w.update({p + f"mlp.e{e}.gate": r(F, W, sd=W ** -0.5), p + f"mlp.e{e}.up": r(F, W, sd=W ** -0.5),
                          p + f"mlp.e{e}.down": r(W, F, sd=F ** -0.5)})
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                w.update({p + "mlp.shared.gate": r(Fs, W, sd=W ** -0.5), p + "mlp.shared.up": r(Fs, W, sd=W ** -0.5),
                          p + "mlp.shared.down": r(W, Fs, sd=Fs ** -0.5)})
    return w


def differential_lambda(mix: dict, diff: float) -> float:
    """exp(lq1 . lk1) - exp(lq2 . lk2) + diff, evaluated once per layer in fp64."""
    dot = lambda a, b: float((mix[a].double() * mix[b].double()).sum())
    return math.exp(dot("lq1", "lk1")) - math.exp(dot("lq2", "lk2")) + float(diff)


class MegolornModel:
    """Weights on the device plus the step function; the cache pools are made by `make_caches` for a serving session."""

    architecture = "Megolorn"
    page_size = 64

    def __init__(self, cfg: MegolornConfig, weights: dict, dtype=torch.bfloat16, device=0):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype: bfloat16 or float32")
        if not torch.cuda.is_available():
            raise RuntimeError("MegolornModel needs a CUDA device (krasis_b200 has no CPU path)")
        ops.load()
        self.cfg, self.dtype = cfg, dtype
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        dev, eps = self.device, cfg.eps
        d = lambda t: t.to(device=dev, dtype=dtype).contiguous()
        f = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()
        self.embed, self.head = d(weights["embed"]), d(weights["head"])
        self.final_norm = f(weights["final.norm"])
        self.layers = []
        for i, L in enumerate(cfg.layers):
            p, m = f"l{i}.", L["mixer"]
            mw = _sub(weights, p + "mix.")
            rot = m.get("rot") or {}
            diff = float(m.get("diff", 0.0))
            lay = {"norm1": f(weights[p + "norm1"]), "kv_from": m.get("kv_from")}
            lay["mixer"] = MultiMapAttention(
                mw, m["heads"], m["kv_heads"], MAPS, m["dim"], m["vdim"], m["scale"], eps, dtype, dev,
                chunk=(m.get("mask") or {}).get("size"), rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 10000.0),
                rot_factor=(rot.get("scaling") or {}).get("factor", 1.0), map_coef=[1.0, -differential_lambda(mw, diff)],
                unit_norm=True, post_scale=1.0 - diff, own_kv=m.get("kv_from") is None)
            mlp = L.get("mlp")
            if not mlp:
                lay["mlp"] = None
            elif mlp.get("kind", "dense") == "dense":
                lay["mlp"] = GatedMLP(_sub(weights, p + "mlp."), dtype, dev, act="clamped_swish", limit=mlp["limit"], alpha=SWISH_ALPHA)
            else:
                rt = mlp["router"]
                grp = rt.get("groups") or {}
                lay["mlp"] = RoutedExperts(_sub(weights, p + "mlp."), rt["experts"], rt.get("identity", 0), rt["top"], dtype, dev,
                                           groups=grp.get("count", 1), keep=grp.get("keep", 1))
            self.layers.append(lay)

    # ------------------------------------------------------------------------------------------- construction
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype=torch.bfloat16, device=0, **_):
        from . import loader
        cfg = MegolornConfig.from_dict(json.load(open(os.path.join(model_dir, "config.json"))))
        return cls(cfg, loader.read_named_tensors(model_dir), dtype=dtype, device=device)

    @classmethod
    def random(cls, cfg: MegolornConfig, seed: int = 0, dtype=torch.bfloat16, device=0):
        return cls(cfg, random_weights(cfg, seed), dtype=dtype, device=device)

    # ------------------------------------------------------------------------------------------- serving interface
    def make_caches(self, max_tokens: int, max_requests: int):
        """(paged cache, state pool) for a session that holds at most max_tokens tokens (each request rounded up to whole pages)
        in at most max_requests live requests.  A layer that projects keys and values owns a pool pair; a layer that reads another
        layer's is pointed at that pair.  The design has no recurrent state: the state pool only hands out request slots."""
        pages = (max_tokens + self.page_size - 1) // self.page_size
        dims, self._layer_cache = [], {}
        for i, lay in enumerate(self.layers):
            if lay["kv_from"] is None:
                self._layer_cache[i] = len(dims)
                dims.append(lay["mixer"].cache_dims())
        for i, lay in enumerate(self.layers):
            if lay["kv_from"] is not None:
                self._layer_cache[i] = self._layer_cache[lay["kv_from"]]
        self.kv_cache = HeadKVCache(dims, self.device, max_pages=max(pages, 1), dtype=self.dtype, page_size=self.page_size)
        self.state_pool = RecurrentStatePool(max_requests, self.device)
        return self.kv_cache, self.state_pool

    def forward_step(self, tb: ops.StepTables, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every layer; returns fp32 logits [len(want_rows), vocab] (None if nothing is wanted)."""
        cfg, eps, dt = self.cfg, self.cfg.eps, self.dtype
        x = ops.embed(self.embed, tb.tokens, cfg.embed_scale)
        h = ops.residual_add_norm(x, out_norm=(self.layers[0]["norm1"], None), out_dtype=dt, eps=eps)
        n = len(self.layers)
        for i, lay in enumerate(self.layers):
            kc, vc = self.kv_cache.get_layer_caches(self._layer_cache[i])
            y_mix = lay["mixer"].forward(h, tb, kc, vc, self.kv_cache.page_size)
            y_ff = lay["mlp"].forward(h) if lay["mlp"] is not None else None
            nxt = (self.layers[i + 1]["norm1"], dt) if i + 1 < n else (self.final_norm, torch.float32)
            h = ops.residual_add_norm(x, y_mix, y_ff, out_norm=(nxt[0], None), out_dtype=nxt[1], eps=eps)
            if self.layer_trace is not None:
                self.layer_trace.append(x.clone())
        if want_rows is None or want_rows.numel() == 0:
            return None
        return lin(h.index_select(0, want_rows), self.head, torch.float32)

    layer_trace = None      # tests: set to a list to collect the residual stream after every layer
