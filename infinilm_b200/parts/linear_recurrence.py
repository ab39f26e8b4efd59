"""Mixers that keep a matrix per head instead of keys: a decayed sum of outer products ("lightning" linear attention)
and the gated delta rule. Both run their recurrence token by token in float32, from a float32 state per request.

DecayLinearAttention:
    q = silu(W_q h), k = silu(W_k h), v = silu(W_v h);  per head  S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t
    y = W_o ( rms_norm(o over all heads) * w * sigmoid(W_g h) )
GatedDeltaRule:
    q, k, v = silu(short_conv(W_q h)), silu(short_conv(W_k h)), silu(short_conv(W_v h));  q, k unit vectors per head, q / sqrt(dim)
    beta = sigmoid(W_b h),  g = exp(-exp(A_log) softplus(W_a h + dt_bias))
    per head  S = g S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q      (the read-out sees the token's own write)
    y = W_o ( rms_norm(o per head) * w * silu(W_g h) )
MatrixLSTM (the matrix memory of an xLSTM block, with exponential gates kept in log space under a running maximum m):
    q = W_q h / sqrt(dim), k = W_k h, v = W_v h;  i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))
    m_t = max(f + m_(t-1), i);  S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;  n_t the same with k alone
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6);  y = W_o ( rms_norm(o per head) * w * sigmoid(W_g h) )
    (S, n and m start at zero; the state is S with n as one more column, and m)
ChannelDecayMixer (time mixing in the manner of RWKV's later versions: a decay per head and key channel that depends on the token):
    every projection reads its own blend of the token's input and its predecessor's, x_s = h + (h_prev - h) * mu_s, s in r, k, v, g, w
    r, k, v = W_r x_r, W_k x_k, W_v x_v (heads x dim);  gate = silu(W_g x_g);  w = exp(-exp(w0 + W_w2 tanh(W_w1 x_w)))
    per head  o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;  S_t = diag(w_t) S_(t-1) + k_t v_t^T      (u: a bonus for the token itself)
    y = W_o ( rms_norm(o per head) * w_norm * gate )
    (S starts at zero; the state is S and the last token's h)
The projections leave float32 on both paths (what enters a recurrence, its gates and decays stay 32-bit).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from .base import Mixer, register_part
from .linear import Linear
from .short_conv import ShortConv
from .spec import CacheNeed, WeightSpec


class _FusableEnds:
    """What both mixers of this file share at their two ends in a decode step of a few bfloat16 rows: the first product takes
    rows whose norm is only half done (and leaves float32), the output product adds into the residual and prepares the next norm."""

    def accepts_normed(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_ok(T, self.hidden)

    def fuses_tail(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_resid_ok(T, self.nv, self.hidden)

    def _project(self, x, out):
        if isinstance(x, ops.NormedInput):
            ops.gemm_skinny(x.xw, self.proj.weight, out, 1.0, None, norm_in=x)
            return out
        return self.proj(x, out, out_f32=True)

    def _output(self, gated, ctx, tail, tag):
        T = gated.shape[0]
        if tail is not None:
            return ops.gemm_skinny_resid(gated, self.o_proj.weight, self.o_proj.alpha, None, tail.resid, tail.scale, tail.norm.weight,
                                         tail.norm.eps, ctx.ws.rows("xw_mixer", T, self.hidden, self.dtype),
                                         ctx.ws.rows("sumsq_mixer", T, (self.hidden + 15) // 16, torch.float32))
        return self.o_proj(gated, ctx.ws.rows(tag, T, self.hidden, self.dtype))


class DecayLinearAttention(_FusableEnds, Mixer):
    """params: hidden, n_heads, qk_dim, v_dim, decay (one number per head), eps (of the output norm).
    Tensors: q, k, v, g, o [out, in]; norm [heads * v_dim]."""
    graph_safe = True
    ACT_PASS_ROWS = 64

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh, self.dk, self.dv = int(p["hidden"]), int(p["n_heads"]), int(p["qk_dim"]), int(p["v_dim"])
        self.eps = float(p["eps"])
        self.decay_list = [float(x) for x in p["decay"]]
        if len(self.decay_list) != self.nh:
            raise ValueError(f"linear attention: {len(self.decay_list)} decays for {self.nh} heads")
        self.nqk, self.nv = self.nh * self.dk, self.nh * self.dv
        self.proj = Linear(self.hidden, 2 * self.nqk + 2 * self.nv, dtype)          # [q | k | v | g]
        self.o_proj = Linear(self.nv, self.hidden, dtype)
        self.decay = self.norm_w = None

    def weight_specs(self) -> List[WeightSpec]:
        H = self.hidden
        return [WeightSpec("q", (self.nqk, H)), WeightSpec("k", (self.nqk, H)), WeightSpec("v", (self.nv, H)), WeightSpec("g", (self.nv, H)),
                WeightSpec("o", (H, self.nv)), WeightSpec("norm", (self.nv,), "vector", ("ones_normal", 0.05))]

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        self.proj.set(torch.cat([t["q"], t["k"], t["v"], t["g"]], dim=0))
        self.o_proj.set(t["o"])
        self.norm_w = t["norm"].contiguous()
        self.decay = torch.tensor(self.decay_list, dtype=torch.float64).to(torch.float32).to(t["q"].device)

    def cache_need(self):
        return CacheNeed("state", shape=(self.nh, self.dv, self.dk), dtype="float32")

    def forward(self, x, ctx, cache, tail=None):
        T, nqk, nv = x.shape[0], self.nqk, self.nv
        proj = self._project(x, ctx.ws.rows("dla_proj", T, 2 * nqk + 2 * nv, torch.float32))
        o = ctx.ws.rows("dla_o", T, nv, torch.float32)
        in_act = 1
        if T > self.ACT_PASS_ROWS:                # many rows: the activation as a pass of its own (the same function), not in the token loop
            ops.silu_cols(proj, 2 * nqk + nv)
            in_act = 0
        ops.matrix_state_scan_step(ctx, ops.SCAN_DECAY, proj[:, :nqk], proj[:, nqk: 2 * nqk], proj[:, 2 * nqk: 2 * nqk + nv], self.nh, self.nh,
                                   self.dk, self.dv, in_act, self.decay, None, None, cache.storage, cache.read_slots,
                                   cache.write_slots if cache.writable else cache.read_slots, ctx.entry_qstart, out=o)
        gated = ctx.ws.rows("dla_gated", T, nv, self.dtype)
        ops.group_norm_gate(o, self.norm_w, self.eps, proj, 2 * nqk + nv, ops.GATE_SIGMOID, gated, nv)
        return self._output(gated, ctx, tail, "dla_branch")


class GatedDeltaRule(_FusableEnds, Mixer):
    """params: hidden, n_heads (value heads), n_qk_heads, qk_dim, v_dim, conv_taps, eps (of the output norm), unit_eps (inside
    the root that makes q and k unit vectors, default 1e-6).
    Tensors: q, k [n_qk_heads * qk_dim, in], v, g [n_heads * v_dim, in], b, a [n_heads, in], o; q.conv, k.conv, v.conv
    [channels, taps]; A_log, dt_bias [n_heads]; norm [v_dim]."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh, self.ng = int(p["hidden"]), int(p["n_heads"]), int(p["n_qk_heads"])
        self.dk, self.dv = int(p["qk_dim"]), int(p["v_dim"])
        self.has_conv, self.taps = p.get("conv_taps") is not None, int(p.get("conv_taps") or 1)
        if self.nh <= 0 or self.ng <= 0 or self.nh % self.ng:
            raise ValueError(f"delta rule: {self.nh} value heads are not a multiple of {self.ng} q/k heads")
        self.eps, self.unit_eps = float(p["eps"]), float(p.get("unit_eps", 1e-6))
        self.nqk, self.nv = self.ng * self.dk, self.nh * self.dv
        self.n_conv = 2 * self.nqk + self.nv
        self.n_proj = self.n_conv + 2 * self.nh + self.nv                          # [q | k | v | b | a | g]
        self.n_proj_pad = (self.n_proj + 7) // 8 * 8
        self.proj = Linear(self.hidden, self.n_proj_pad, dtype)
        self.o_proj = Linear(self.nv, self.hidden, dtype)
        self.conv = ShortConv(self.n_conv, self.taps)
        self.a_log = self.dt_bias = self.norm_w = None

    def weight_specs(self) -> List[WeightSpec]:
        H = self.hidden
        specs = [WeightSpec("q", (self.nqk, H)), WeightSpec("k", (self.nqk, H)), WeightSpec("v", (self.nv, H)),
                 WeightSpec("b", (self.nh, H)), WeightSpec("a", (self.nh, H)), WeightSpec("g", (self.nv, H)), WeightSpec("o", (H, self.nv)),
                 WeightSpec("A_log", (self.nh,), "vector", ("normal", 0.5)), WeightSpec("dt_bias", (self.nh,), "vector", ("normal", 0.5)),
                 WeightSpec("norm", (self.dv,), "vector", ("ones_normal", 0.05))]
        if self.has_conv:
            specs += [WeightSpec(n + ".conv", (c, self.taps), "vector", ("normal", 0.5)) for n, c in (("q", self.nqk), ("k", self.nqk), ("v", self.nv))]
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        ws = [t["q"], t["k"], t["v"], t["b"], t["a"], t["g"]]
        if self.n_proj_pad != self.n_proj:
            ws.append(torch.zeros((self.n_proj_pad - self.n_proj, self.hidden), dtype=ws[0].dtype, device=ws[0].device))
        self.proj.set(torch.cat(ws, dim=0))
        self.o_proj.set(t["o"])
        if self.has_conv:
            self.conv.set([t["q.conv"], t["k.conv"], t["v.conv"]])
        else:
            self.conv.set([torch.ones((self.n_conv, 1), dtype=torch.float32, device=t["q"].device)])
        self.a_log, self.dt_bias = t["A_log"].to(torch.float32).contiguous(), t["dt_bias"].to(torch.float32).contiguous()
        self.norm_w = t["norm"].contiguous()

    def cache_need(self):
        return (CacheNeed("state", shape=(self.nh, self.dv, self.dk), dtype="float32"), self.conv.state_need())

    def forward(self, x, ctx, cache, tail=None):
        S, conv_state = cache
        T, nqk, nv, nh = x.shape[0], self.nqk, self.nv, self.nh
        proj = self._project(x, ctx.ws.rows("gdr_proj", T, self.n_proj_pad, torch.float32))
        qkv = ctx.ws.rows("gdr_qkv", T, self.n_conv, torch.float32)
        self.conv.run(proj, 0, ctx, conv_state, qkv, (1, self.n_conv, self.n_conv), act=1)
        beta = ctx.ws.rows("gdr_beta", T, nh, torch.float32)
        gdec = ctx.ws.rows("gdr_decay", T, nh, torch.float32)
        ops.delta_prep(qkv, 0, nqk, self.ng, self.dk, self.dk ** -0.5, self.unit_eps, proj, self.n_conv, self.n_conv + nh,
                       self.a_log, self.dt_bias, beta, gdec, nh)
        o = ctx.ws.rows("gdr_o", T, nv, torch.float32)
        ops.matrix_state_scan_step(ctx, ops.SCAN_DELTA, qkv[:, :nqk], qkv[:, nqk: 2 * nqk], qkv[:, 2 * nqk:], nh, self.ng, self.dk, self.dv, 0,
                                   None, beta, gdec, S.storage, S.read_slots, S.write_slots if S.writable else S.read_slots,
                                   ctx.entry_qstart, out=o)
        gated = ctx.ws.rows("gdr_gated", T, nv, self.dtype)
        ops.group_norm_gate(o, self.norm_w, self.eps, proj, self.n_conv + 2 * nh, ops.GATE_SILU, gated, self.dv)
        return self._output(gated, ctx, tail, "gdr_branch")


class MatrixLSTM(Mixer):
    """params: hidden, n_heads, qk_dim, v_dim, gate_cap (None or 0: the gates' pre-activations are not capped), eps (of the
    output norm), den_eps (added to the read-out's denominator, default 1e-6).
    Tensors: q, k [heads * qk_dim, in], v, g [heads * v_dim, in], i, f [heads, in], i.b, f.b [heads], o, norm [heads * v_dim]."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh, self.dk, self.dv = int(p["hidden"]), int(p["n_heads"]), int(p["qk_dim"]), int(p["v_dim"])
        if min(self.hidden, self.nh, self.dk, self.dv) <= 0:
            raise ValueError("matrix memory: sizes must be positive")
        self.cap = float(p.get("gate_cap") or 0.0)
        self.eps, self.den_eps = float(p["eps"]), float(p.get("den_eps", 1e-6))
        self.nqk, self.nv = self.nh * self.dk, self.nh * self.dv
        self.i_off = 2 * self.nqk + 2 * self.nv                                   # [q | k | v | g | i | f]
        self.n_proj = self.i_off + 2 * self.nh
        self.n_proj_pad = (self.n_proj + 7) // 8 * 8
        self.proj = Linear(self.hidden, self.n_proj_pad, dtype)
        self.o_proj = Linear(self.nv, self.hidden, dtype)
        self.norm_w = None

    def weight_specs(self) -> List[WeightSpec]:
        H = self.hidden
        return [WeightSpec("q", (self.nqk, H)), WeightSpec("k", (self.nqk, H)), WeightSpec("v", (self.nv, H)), WeightSpec("g", (self.nv, H)),
                WeightSpec("i", (self.nh, H)), WeightSpec("f", (self.nh, H)), WeightSpec("i.b", (self.nh,), "vector", ("normal", 0.5)),
                WeightSpec("f.b", (self.nh,), "vector", ("normal", 0.5)), WeightSpec("o", (H, self.nv)),
                WeightSpec("norm", (self.nv,), "vector", ("ones_normal", 0.05))]

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        dev = t["q"].device
        ws = [t["q"], t["k"], t["v"], t["g"], t["i"], t["f"]]
        if self.n_proj_pad != self.n_proj:
            ws.append(torch.zeros((self.n_proj_pad - self.n_proj, self.hidden), dtype=ws[0].dtype, device=dev))
        b = torch.zeros(self.n_proj_pad, dtype=torch.float32, device=dev)
        b[self.i_off: self.i_off + self.nh] = t["i.b"].float()
        b[self.i_off + self.nh: self.i_off + 2 * self.nh] = t["f.b"].float()
        self.proj.set(torch.cat(ws, dim=0), b)
        self.o_proj.set(t["o"])
        self.norm_w = t["norm"].to(torch.float32).contiguous()

    def cache_need(self):
        # S [heads, v_dim + 1, dim] (column by column; the last column is the normaliser n) and the running maximum m [heads]
        return (CacheNeed("state", shape=(self.nh, self.dv + 1, self.dk), dtype="float32"),
                CacheNeed("state", shape=(self.nh,), dtype="float32"))

    def forward(self, x, ctx, cache):
        S, M = cache
        T, nqk, nv, nh = x.shape[0], self.nqk, self.nv, self.nh
        proj = self.proj(x, ctx.ws.rows("mlstm_proj", T, self.n_proj_pad, torch.float32), out_f32=True)
        dec = ctx.ws.rows("mlstm_decay", T, nh, torch.float32)
        inw = ctx.ws.rows("mlstm_inw", T, nh, torch.float32)
        floor = ctx.ws.rows("mlstm_floor", T, nh, torch.float32)
        ops.stabilized_gates(proj, self.i_off, self.i_off + nh, self.cap, M.storage, M.read_slots,
                             M.write_slots if M.writable else M.read_slots, ctx.entry_qstart, ctx.n_entries, dec, inw, floor, nh)
        o = ctx.ws.rows("mlstm_o", T, nh * (self.dv + 1), torch.float32)
        ops.matrix_state_scan_step(ctx, ops.SCAN_GATED, proj[:, :nqk], proj[:, nqk: 2 * nqk], proj[:, 2 * nqk: 2 * nqk + nv], nh, nh,
                                   self.dk, self.dv + 1, 0, None, inw, dec, S.storage, S.read_slots,
                                   S.write_slots if S.writable else S.read_slots, ctx.entry_qstart, out=o)
        gated = ctx.ws.rows("mlstm_gated", T, nv, self.dtype)
        ops.group_norm_gate(o, self.norm_w, self.eps, proj, 2 * nqk + nv, ops.GATE_SIGMOID, gated, self.dv, den_floor=floor,
                            x_scale=self.dk ** -0.5, den_eps=self.den_eps)
        return self.o_proj(gated, ctx.ws.rows("mlstm_branch", T, self.hidden, self.dtype))


class ChannelDecayMixer(Mixer):
    """params: hidden, n_heads, dim (key, value and receptance size of a head), decay_rank (rows of w1; None: the stored tensor's),
    eps (of the output norm).
    Tensors: mu.r, mu.k, mu.v, mu.g, mu.w [hidden]; r, k, v, g [heads * dim, hidden]; w1 [rank, hidden], w2 [heads * dim, rank],
    w0 [heads * dim]; u [heads, dim]; norm [heads * dim]; o [hidden, heads * dim]."""
    graph_safe = True
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh, self.d = int(p["hidden"]), int(p["n_heads"]), int(p["dim"])
        if min(self.hidden, self.nh, self.d) <= 0:
            raise ValueError("channel-decay mixer: sizes must be positive")
        self.rank = None if p.get("decay_rank") is None else int(p["decay_rank"])
        self.eps = float(p["eps"])
        self.n = self.nh * self.d
        self.rkv = [Linear(self.hidden, self.n, dtype) for _ in range(3)]
        self.g_proj = Linear(self.hidden, self.n, dtype)
        self.o_proj = Linear(self.n, self.hidden, dtype)
        self.w1 = self.w2 = self.mu = self.u = self.norm_w = None

    def weight_specs(self) -> List[WeightSpec]:
        H, n = self.hidden, self.n
        r = -1 if self.rank is None else self.rank
        return ([WeightSpec("mu." + m, (H,), "vector", ("normal", 0.3)) for m in self.MIXES]
                + [WeightSpec(x, (n, H)) for x in ("r", "k", "v", "g")]
                + [WeightSpec("w1", (r, H), free=16), WeightSpec("w2", (n, r), init=("normal", 0.1), free=16),
                   WeightSpec("w0", (n,), "vector", ("normal", 0.5)), WeightSpec("u", (self.nh, self.d), "vector", ("normal", 0.5)),
                   WeightSpec("norm", (n,), "vector", ("ones_normal", 0.05)), WeightSpec("o", (H, n))])

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        for lin, name in zip(self.rkv, ("r", "k", "v")):
            lin.set(t[name])
        self.g_proj.set(t["g"])
        self.o_proj.set(t["o"])
        rank = int(t["w1"].shape[0])
        if tuple(t["w2"].shape) != (self.n, rank):
            raise ValueError(f"channel-decay mixer: w2 {tuple(t['w2'].shape)} does not follow w1's {rank} rows")
        self.w1, self.w2 = Linear(self.hidden, rank, self.dtype), Linear(rank, self.n, self.dtype)
        self.w1.set(t["w1"])
        self.w2.set(t["w2"], t["w0"].to(torch.float32))          # w0 joins the product as its bias, in float32
        self.mu = torch.stack([t["mu." + m].to(torch.float32) for m in self.MIXES]).contiguous()
        self.u = t["u"].to(torch.float32).contiguous()
        self.norm_w = t["norm"].to(torch.float32).contiguous()

    def cache_need(self):
        # S [heads, dim, dim] (column by column) and the last token's input row
        return (CacheNeed("state", shape=(self.nh, self.d, self.d), dtype="float32"),
                CacheNeed("state", shape=(self.hidden,), dtype="float32"))

    def forward(self, x, ctx, cache):
        S, prev = cache
        T, W, n, dt = x.shape[0], self.hidden, self.n, self.dtype
        ws = ctx.ws
        mix = ws.rows("cdm_mix", T, len(self.MIXES) * W, dt)
        ops.token_shift_mix(x, self.mu, prev.storage, prev.read_slots, prev.write_slots if prev.writable else None, ctx.tok_entry,
                            ctx.entry_qstart, mix)
        rkv = ws.rows("cdm_rkv", T, 3 * n, torch.float32)
        for i, lin in enumerate(self.rkv):
            lin(mix[:, i * W:(i + 1) * W], rkv[:, i * n:(i + 1) * n], out_f32=True)
        gate = self.g_proj(mix[:, 3 * W:4 * W], ws.rows("cdm_gate", T, n, dt))
        rank = self.w1.out_features
        low = self.w1(mix[:, 4 * W:5 * W], ws.rows("cdm_low", T, rank, torch.float32), out_f32=True)
        low_t = ws.rows("cdm_low_t", T, rank, dt)
        ops.tanh_rows(low, low_t)
        decay = self.w2(low_t, ws.rows("cdm_decay", T, n, torch.float32), out_f32=True)
        ops.double_exp_decay(decay, None, n)
        o = ws.rows("cdm_o", T, n, torch.float32)
        ops.matrix_state_scan_step(ctx, ops.SCAN_CHANNEL_DECAY, rkv[:, :n], rkv[:, n:2 * n], rkv[:, 2 * n:], self.nh, self.nh, self.d, self.d, 0,
                                   self.u, None, decay, S.storage, S.read_slots, S.write_slots if S.writable else S.read_slots,
                                   ctx.entry_qstart, out=o)
        gated = ws.rows("cdm_gated", T, n, dt)
        ops.group_norm_gate(o, self.norm_w, self.eps, gate, 0, ops.GATE_SILU, gated, self.d)
        return self.o_proj(gated, ws.rows("cdm_branch", T, self.hidden, dt))


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
register_part("mixer", "channel_decay", ChannelDecayMixer)
register_part("mixer", "matrix_lstm", MatrixLSTM)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
