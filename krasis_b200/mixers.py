"""Token mixers and sublayers for ragged-batch serving (prefill portions and decoded tokens in one step).

Each class owns its weights on the device, takes its constants as constructor arguments and runs on the kernels of
libkrasis_b200_seq (`krasis_b200.seqops`): a model composes them (krasis_b200/vofelix.py).

  WindowLatentAttention   attention over a cached low-rank latent with one shared rotated key part, interleaved rotary positions
                          with YaRN frequency blending, a sliding window and a per-head softmax sink
  GatedDeltaMixer         short causal convolutions on q / k / v, unit-norm q and k, gated delta-rule state per head in fp32
                          slots, per-head RMS norm of the read-out with a SiLU gate
  GatedMLP                down(act(gate h) * (up h)) with the tanh form of GELU
  TokenSideInput          per-layer token table slice, gated by a projection of the residual stream, RMS-normed
`lin(a, w, out_dtype)` picks the GEMM: the tcgen05 kernel of the core library for large aligned bf16 products, the generic
kernel of the sequence library otherwise (any shape, fp32 or bf16).
"""
import math
import os

import torch

from . import seqops as ops


_core = None


def _core_lib():
    """The core library's tcgen05 GEMM, if that library has been built (it is optional for models that run on seqops alone)."""
    global _core
    if _core is None:
        _core = False
        if os.environ.get("KB2_SEQ_TCGEN05", "1") != "0":
            try:
                from . import capi
                if os.path.exists(capi.LIB_PATH):
                    _core = capi.load()
            except Exception:       # noqa: BLE001 — optional accelerator; the generic kernel computes the same product
                _core = False
    return _core


def lin(a: torch.Tensor, w: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """a [M, K] @ w [N, K]^T with fp32 accumulation."""
    M, K = a.shape
    N = w.shape[0]
    if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M >= 256 and K % 64 == 0 and N % 16 == 0 and N >= 256
            and a.is_contiguous() and w.is_contiguous()):
        core = _core_lib()
        if core:
            from . import capi
            out = torch.empty((M, N), dtype=out_dtype, device=a.device)
            capi.check(core.kb2_linear_bf16(a.data_ptr(), w.data_ptr(), None, out.data_ptr(), M, N, K, int(out_dtype == torch.float32),
                                            a.device.index or 0, torch.cuda.current_stream(a.device).cuda_stream))
            return out
    return ops.gemm(a, w, out_dtype)


def yarn_table(dims: int, base: float, scaling):
    """Angular frequency of each rotated pair (fp64) and the amplitude both sin and cos carry.
    scaling = {factor, original, fast, slow} or None: pairs that turn more than `fast` times over `original` positions keep their
    frequency, pairs that turn less than `slow` times are slowed by `factor`, a linear ramp in between."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class WindowLatentAttention:
    """weights: q [H (dn + dr), W], dkv [r + dr, W], dkv_norm [r], uk [H dn, r], uv [H dv, r], sink [H], o [W, H dv]."""

    def __init__(self, weights: dict, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float, window,
                 rot_dims: int, rot_base: float, rot_scaling, eps: float, dtype, device):
        self.H, self.dn, self.dr, self.dv, self.r = heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.dtype, self.device = float(scale), float(eps), dtype, device
        self.window = int(window) if window else 1 << 30
        self.rot_dims = int(rot_dims)
        if self.rot_dims > rot_dim or self.rot_dims % 2:
            raise ValueError("rotated dimensions must be even and at most rot_dim")
        freq, amp = yarn_table(self.rot_dims, rot_base, rot_scaling) if self.rot_dims else (torch.zeros(1, dtype=torch.float64), 1.0)
        self.freq, self.amp = freq.to(device), float(amp)
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.w_in = d(torch.cat([weights["q"], weights["dkv"]], 0))                # one projection: [q | latent | rotated key]
        self.dkv_norm, self.sink = f(weights["dkv_norm"]), f(weights["sink"])
        # absorbed key up-projection: q_abs[h] = q_nope[h] @ uk[h]  ->  stored [H, r, dn] for an A B^T product
        self.uk_t = d(weights["uk"].reshape(heads, dim, kv_rank).transpose(1, 2))
        self.uv = d(weights["uv"].reshape(heads, vdim, kv_rank))
        self.w_o = d(weights["o"])
        # long prompt portions in bfloat16 with 128 + 64 query / key dims and 128 value dims run the tcgen05 attention core of the MoE
        # prefill models (non-absorbed form: keys and values of the window are up-projected from the cached latents by one GEMM)
        self.tc_min_portion = 128
        self.tc_shape = dtype == torch.bfloat16 and dim == 128 and rot_dim == 64 and vdim == 128 and kv_rank % 64 == 0
        self.w_kv_up = d(torch.cat([weights["uk"], weights["uv"]], 0)) if self.tc_shape else None

    def cache_dims(self):
        return self.r, self.dr

    def forward(self, h: torch.Tensor, tb: ops.StepTables, ckv: torch.Tensor, kr: torch.Tensor, page_size: int) -> torch.Tensor:
        lib, T, H = ops.load(), h.shape[0], self.H
        proj = lin(h, self.w_in, torch.float32)
        ldp = proj.stride(0)
        s = torch.cuda.current_stream(h.device).cuda_stream
        dtc = ops.dt_code(ckv.dtype)
        ops.check(lib.kb2_seq_latent_prep(proj.data_ptr(), ldp, T, H, self.dn, self.dr, self.r, self.dkv_norm.data_ptr(), self.eps,
                                          self.freq.data_ptr(), self.rot_dims, self.amp, tb.positions.data_ptr(), tb.seq_of.data_ptr(),
                                          tb.pages.data_ptr(), tb.max_pages, page_size, ckv.data_ptr(), kr.data_ptr(), dtc, s))
        q = proj[:, :H * (self.dn + self.dr)].view(T, H, self.dn + self.dr)
        o = torch.empty((T, H, self.dv), dtype=self.dtype, device=h.device)
        core = _core_lib() if self.tc_shape else False
        fast = [i for i, (_, n, _, _) in enumerate(tb.layout) if n >= self.tc_min_portion] if core else []
        if len(fast) < tb.S:
            q_abs = torch.empty((T, H, self.r), dtype=torch.float32, device=h.device)
            ops.gemm_heads(q[:, :, :self.dn], self.uk_t, q_abs)
            o_lat = torch.empty((T, H, self.r), dtype=torch.float32, device=h.device)
            # a step of few tokens (decoding) cuts each token's keys into pieces so that the whole GPU works on them
            blocks = T * ((H + 7) // 8)
            max_keys = max(min(self.window, start + n) for _, n, start, _ in tb.layout)
            nsplit = max(1, min(296 // max(blocks, 1), (max_keys + 31) // 32, 64))
            part_acc = torch.empty((T, nsplit, H, self.r), dtype=torch.float32, device=h.device) if nsplit > 1 else None
            part_ml = torch.empty((T, nsplit, H, 2), dtype=torch.float32, device=h.device) if nsplit > 1 else None
            ops.check(lib.kb2_seq_latent_window_attn(q_abs.data_ptr(), proj.data_ptr(), ldp, T, H, self.dn, self.dr, self.r, ckv.data_ptr(),
                                                     kr.data_ptr(), dtc, tb.positions.data_ptr(), tb.seq_of.data_ptr(), tb.pages.data_ptr(),
                                                     tb.max_pages, page_size, self.sink.data_ptr(), self.scale, self.window,
                                                     o_lat.data_ptr(), tb.cu.data_ptr() if fast else None, self.tc_min_portion, nsplit,
                                                     part_acc.data_ptr() if nsplit > 1 else None,
                                                     part_ml.data_ptr() if nsplit > 1 else None, s))
            ops.gemm_heads(o_lat, self.uv, o)
        for i in fast:
            from . import capi
            row0, n, start, _ = tb.layout[i]
            lo, rows = ops.key_rows(tb, i, self.window, page_size)
            kv_up = lin(ckv.view(-1, self.r).index_select(0, rows), self.w_kv_up, torch.bfloat16)     # [keys, H * (128 + 128)]
            kpe = kr.view(-1, self.dr).index_select(0, rows)
            q_bf = proj[row0:row0 + n, :H * (self.dn + self.dr)].to(torch.bfloat16).contiguous()
            capi.check(core.kb2_fmha_latent(q_bf.data_ptr(), kv_up.data_ptr(), kpe.data_ptr(), o[row0:row0 + n].data_ptr(), n, start - lo,
                                            start - lo + n, H, self.scale, min(self.window, 1 << 30), self.sink.data_ptr(),
                                            h.device.index or 0, s))
        return lin(o.view(T, H * self.dv), self.w_o, torch.float32)


class GatedDeltaMixer:
    """weights: q, k [Hk dk, W], v, g [H dv, W], a, b [H, W], q_conv, k_conv, v_conv [channels, taps], A_log, dt_bias [H],
    norm [dv], o [W, H dv]."""

    def __init__(self, weights: dict, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float, dtype, device):
        self.H, self.Hk, self.dk, self.dv, self.K = heads, kv_heads, dim, vdim, int(taps)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.eps, self.dtype, self.device = float(eps), dtype, device
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        f = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.C = 2 * kv_heads * dim + heads * vdim                                  # convolved channels: q | k | v
        self.g_off, self.a_off, self.b_off = self.C, self.C + heads * vdim, self.C + heads * vdim + heads
        self.w_in = d(torch.cat([weights[k] for k in ("q", "k", "v", "g", "a", "b")], 0))
        self.taps = f(torch.cat([weights["q_conv"], weights["k_conv"], weights["v_conv"]], 0))
        self.A_log, self.dt_bias, self.norm = f(weights["A_log"]), f(weights["dt_bias"]), f(weights["norm"])
        self.w_o = d(weights["o"])
        # key sizes 32 / 64 / 128 with value sizes that are multiples of 32 keep the state in registers; others in shared memory
        self.register_state_kernel = dim in (32, 64, 128) and vdim % 32 == 0

    def register_state(self, pool):
        """(conv tail [slots, C, taps - 1], recurrent state [slots, H, dk, dv]) in a RecurrentStatePool."""
        return pool.register(self.C, max(self.K - 1, 1)), pool.register(self.H, self.dk, self.dv)

    def forward(self, h: torch.Tensor, tb: ops.StepTables, tail: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        lib, T = ops.load(), h.shape[0]
        proj = lin(h, self.w_in, torch.float32)
        s = torch.cuda.current_stream(h.device).cuda_stream
        conv = torch.empty((T, self.C), dtype=torch.float32, device=h.device)
        ops.check(lib.kb2_seq_conv_silu(proj.data_ptr(), proj.stride(0), T, tb.S, self.C, self.K, self.taps.data_ptr(), tail.data_ptr(),
                                        tb.seq_of.data_ptr(), tb.cu.data_ptr(), tb.slots.data_ptr(), conv.data_ptr(), s))
        o = torch.empty((T, self.H * self.dv), dtype=self.dtype, device=h.device)
        scratch = None
        if self.register_state_kernel:
            scratch = torch.empty(2 * T * self.Hk * self.dk + 2 * T * self.H + T * self.H * self.dv + 4, dtype=torch.float32, device=h.device)
        ops.check(lib.kb2_seq_delta_rule(conv.data_ptr(), self.C, proj.data_ptr(), proj.stride(0), self.g_off, self.a_off, self.b_off, T,
                                         tb.S, self.H, self.Hk, self.dk, self.dv, self.A_log.data_ptr(), self.dt_bias.data_ptr(),
                                         self.norm.data_ptr(), self.eps, state.data_ptr(), tb.cu.data_ptr(), tb.slots.data_ptr(),
                                         scratch.data_ptr() if scratch is not None else None, o.data_ptr(), ops.dt_code(self.dtype), s))
        return lin(o, self.w_o, torch.float32)


class GatedMLP:
    """weights: gate, up [F, W], down [W, F]."""

    def __init__(self, weights: dict, dtype, device):
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        self.w_gu, self.w_down, self.dtype = d(torch.cat([weights["gate"], weights["up"]], 0)), d(weights["down"]), dtype

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return lin(ops.act_mul(lin(h, self.w_gu, self.dtype), self.dtype), self.w_down, torch.float32)


class TokenSideInput:
    """weights: gate [dim, W], proj [W, dim], norm [W]; `table` [vocab, layers * dim] is shared by the layers, this one reads the
    columns [col0, col0 + dim).  forward returns y = proj(gelu(gate x) * table[token]); the caller adds rms_norm(y) * norm."""

    def __init__(self, weights: dict, table: torch.Tensor, col0: int, dim: int, dtype, device):
        d = lambda t: t.to(device=device, dtype=dtype).contiguous()
        self.w_gate, self.w_proj = d(weights["gate"]), d(weights["proj"])
        self.norm = weights["norm"].to(device=device, dtype=torch.float32).contiguous()
        self.table, self.col0, self.dim, self.dtype = table, col0, dim, dtype

    def forward(self, x: torch.Tensor, tb: ops.StepTables) -> torch.Tensor:
        # x is the fp32 residual stream itself; a long bfloat16 step rounds it once so that the projection runs on the tensor cores
        a = x.to(torch.bfloat16) if (self.dtype == torch.bfloat16 and x.shape[0] >= 256 and _core_lib()) else x
        g = lin(a, self.w_gate, torch.float32)
        return lin(ops.side_gate(g, self.table, tb.tokens, self.col0, self.dtype), self.w_proj, torch.float32)
