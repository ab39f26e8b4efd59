"""Softmax attention over the paged cache whose queries and keys are normed. In its first form the norm is per head and
positions rotate nothing: they enter, if at all, as a learned bias by distance on the scores or as a temperature on the
queries. In its second form (`norm_over` "projection") the norm runs over a token's whole query projection (all heads at
once; the keys' likewise) with a weight of that many entries, a rotary encoding (`position`) may turn part of every head
afterwards, and the mask may be runs of `chunk` positions or a sliding `window`.

    [q | k | v | g] = W h (+ b)
    q_h <- rms_norm(q_h) * w_q * temp(pos),  k_g <- rms_norm(k_g) * w_k        (one weight vector each, shared by the heads)
    score(i, j) = scale * q_i . k_j + bias[bucket(i - j), h]                      (the bias table is optional)
    o_h = softmax over j <= i (optionally with a sink of score 0 in the denominator) of the scores, times v
    y = W_o ([o_1 .. o_H] * sigmoid(g))                                           (the gate, one per column, is optional)

Options: the values may be the keys as projected, before their norm (no v tensor); a mixer may read the keys and values that
another run-order entry cached (no k, v tensors, no cache of its own); key size and value size may differ - heads are laid
out at hd = max of the two rounded up to 16, the surplus columns zero, as `conv_attention` does.

The bias: table [rows, heads]; distances below rows/2 have a row each, the others share the remaining rows on a logarithmic
scale that reaches the last row at distance `far`: bucket(n) = n for n < rows/2, else
min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2))). At load it is unrolled into a float32
table [far + 1, heads] by distance, constant from `far` on, which is what the attention kernels index.
Tensors (under the part's prefix): q, k, v, g, o [out, in]; q.b, k.b, v.b; q.norm, k.norm [dim]; rel [rows, heads].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import ops
from .attention import PagedAttend
from .base import Mixer, build_part, register_part
from .linear import Linear
from .spec import CacheNeed, PartSpec, WeightSpec


def distance_buckets(rows: int, far: int) -> List[int]:
    """bucket(n) for n = 0 .. far (every distance beyond `far` shares the last entry's row)."""
    half = rows // 2
    if rows < 2 or far <= half:
        raise ValueError(f"distance bias: a table of {rows} rows needs far > rows/2 (got {far})")
    out = []
    for n in range(far + 1):
        if n < half:
            out.append(n)
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


class QKNormAttention(Mixer):
    """params: hidden, n_heads, n_kv_heads, qk_dim, v_dim, scale, eps (of the query and key norms), qkv_bias,
    value_from_key (the values are the un-normed keys), own_kv (False: the run order gives this entry another entry's cache),
    distance_bias (None or {"rows": B or None - the table's own row count -, "far": D}), q_temperature (None or {"coef": c, "every": n}), sink_zero (a key without
    a value and with score 0 joins the softmax), output_gate, plain_kernel, prefill_kernel;
    norm_over ("head", the default, or "projection": q.norm has heads * qk_dim entries, k.norm kv_heads * qk_dim),
    position (PartSpec of a rotary encoding, with norm_over "projection"), chunk (runs of that many positions, counted from the
    sequence's start; a query sees its own run) or window (a sliding window; its pages are given back behind it)."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh, self.nkv = int(p["hidden"]), int(p["n_heads"]), int(p["n_kv_heads"])
        self.dk, self.dv = int(p["qk_dim"]), int(p["v_dim"])
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        self.hd = (max(self.dk, self.dv) + 15) // 16 * 16
        if self.hd > 256:
            raise ValueError(f"attention: key / value size {max(self.dk, self.dv)} is not supported (up to 256)")
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.qkv_bias, self.gate = bool(p.get("qkv_bias", False)), bool(p.get("output_gate", False))
        self.v_from_k, self.own_kv = bool(p.get("value_from_key", False)), bool(p.get("own_kv", True))
        if self.v_from_k and self.dv != self.dk:
            raise ValueError("attention: values that are the keys have the keys' size")
        db = p.get("distance_bias")
        self.has_bias = bool(db)
        self.bias_rows, self.bias_far = (None if db.get("rows") is None else int(db["rows"]), int(db["far"])) if db else (0, 0)
        if self.bias_rows is not None and db:
            distance_buckets(self.bias_rows, self.bias_far)       # (checks the pair)
        qt = p.get("q_temperature")
        self.t_coef, self.t_every = (float(qt["coef"]), int(qt["every"])) if qt else (0.0, 0)
        if qt and self.t_every < 1:
            raise ValueError("attention: the query temperature's step must be at least 1")
        self.sink_zero = bool(p.get("sink_zero", False))
        self.norm_rows = str(p.get("norm_over", "head")) == "projection"
        if str(p.get("norm_over", "head")) not in ("head", "projection"):
            raise ValueError("attention: norm_over is 'head' or 'projection'")
        self.position = build_part("position", p.get("position") or PartSpec("none"), dtype)
        if self.position.has_transform or (self.position.rot_dim and not self.norm_rows) or self.position.rot_dim > self.dk:
            raise ValueError("attention: a rotary table of at most qk_dim dimensions, with the norm over the projection")
        if self.norm_rows and (self.v_from_k or qt):
            raise ValueError("attention: the norm over the projection goes with values of their own and no query temperature")
        self.window, self.chunk = p.get("window"), p.get("chunk")
        # the projection's columns: [q | k | v | g], k and v only with a cache of its own, v only if it is not k
        self.nq, self.nk, self.nvv = self.nh * self.dk, self.nkv * self.dk, self.nkv * self.dv
        self.q_off, off = 0, self.nq
        self.k_off = self.v_off = None
        if self.own_kv:
            self.k_off, off = off, off + self.nk
            if self.v_from_k:
                self.v_off = self.k_off
            else:
                self.v_off, off = off, off + self.nvv
        self.g_off = off
        self.n_proj = off + (self.nh * self.dv if self.gate else 0)
        self.n_proj_pad = (self.n_proj + 7) // 8 * 8
        self.proj = Linear(self.hidden, self.n_proj_pad, dtype)
        self.o_proj = Linear(self.nh * self.dv, self.hidden, dtype)
        self.core = PagedAttend(dtype, self.nh, self.nkv, self.hd, self.scale, self.window, bool(p.get("plain_kernel", False)),
                                str(p.get("prefill_kernel", "auto")), chunk=self.chunk)
        self.w_q = self.w_k = None

    def weight_specs(self) -> List[WeightSpec]:
        H = self.hidden
        specs = [WeightSpec("q", (self.nq, H)), WeightSpec("o", (H, self.nh * self.dv)),
                 WeightSpec("q.norm", (self.nq if self.norm_rows else self.dk,), "vector", ("ones_normal", 0.05))]
        if self.qkv_bias:
            specs.append(WeightSpec("q.b", (self.nq,), "vector", ("normal", 0.02)))
        if self.own_kv:
            specs += [WeightSpec("k", (self.nk, H)), WeightSpec("k.norm", (self.nk if self.norm_rows else self.dk,), "vector", ("ones_normal", 0.05))]
            if self.qkv_bias:
                specs.append(WeightSpec("k.b", (self.nk,), "vector", ("normal", 0.02)))
            if not self.v_from_k:
                specs.append(WeightSpec("v", (self.nvv, H)))
                if self.qkv_bias:
                    specs.append(WeightSpec("v.b", (self.nvv,), "vector", ("normal", 0.02)))
        if self.has_bias:
            specs.append(WeightSpec("rel", (-1 if self.bias_rows is None else self.bias_rows, self.nh), "vector", ("normal", 0.5), free=16))
        if self.gate:
            specs.append(WeightSpec("g", (self.nh * self.dv, H)))
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        dev = t["q"].device
        names = ["q"] + ((["k"] if self.v_from_k else ["k", "v"]) if self.own_kv else [])
        ws = [t[n] for n in names] + ([t["g"]] if self.gate else [])
        pad = self.n_proj_pad - self.n_proj
        if pad:
            ws.append(torch.zeros((pad, self.hidden), dtype=ws[0].dtype, device=dev))
        b = None
        if self.qkv_bias:
            bs = [t[n + ".b"].float() for n in names]
            b = torch.cat(bs + [torch.zeros(self.n_proj_pad - sum(x.numel() for x in bs), dtype=torch.float32, device=dev)])
        self.proj.set(torch.cat(ws, dim=0), b)
        self.o_proj.set(t["o"])
        self.w_q = t["q.norm"].to(torch.float32).contiguous()
        self.w_k = t["k.norm"].to(torch.float32).contiguous() if self.own_kv else None
        if self.has_bias:
            idx = torch.tensor(distance_buckets(int(t["rel"].shape[0]), self.bias_far), dtype=torch.long, device=dev)
            self.core.dist_bias = t["rel"].to(torch.float32)[idx].contiguous()          # [far + 1, heads]
        if self.sink_zero:
            self.core.sink = torch.zeros(self.nh, dtype=torch.float32, device=dev)
        self.position.to_device(dev)

    def cache_need(self) -> Optional[CacheNeed]:
        # (an entry that reads another's cache is never asked: the run order names the owner)
        return CacheNeed("paged_kv", n_kv_heads=self.nkv, head_dim=self.hd, window=self.window)

    def forward(self, x, ctx, cache):
        T, hd = x.shape[0], self.hd
        if cache is None or (self.own_kv and not cache.writable) or (not self.own_kv and cache.writable):
            raise ValueError("attention: a mixer with keys of its own writes its cache; one without reads another entry's")
        proj = self.proj(x, ctx.ws.rows("qna_proj", T, self.n_proj_pad, self.dtype))
        q = ctx.ws.rows("qna_q", T, self.nh * hd, self.dtype)
        if self.norm_rows:
            ops.qk_rows_norm_rope_store(proj, self.q_off, self.k_off, self.v_off if self.own_kv else 0, self.nh, self.nkv, self.dk, self.dv, hd,
                                        self.w_q, self.w_k, self.eps, self.position.rot_dim, self.position.inv_freq, q, ctx.tok_pos,
                                        ctx.tok_entry, cache.block_table, cache.storage if self.own_kv else None, cache.page_size)
        else:
            ops.qk_norm_store(proj, self.q_off, self.k_off, self.v_off if self.own_kv else 0, self.nh, self.nkv, self.dk, self.dv, hd,
                              self.w_q, self.w_k, self.eps, self.t_coef, self.t_every, q, ctx.tok_pos, ctx.tok_entry, cache.block_table,
                              cache.storage if self.own_kv else None, cache.page_size)
        att = ctx.ws.rows("qna_att", T, self.nh * hd, self.dtype)
        self.core.run(q, att, ctx, cache)
        if self.gate or hd != self.dv:
            gated = ctx.ws.rows("qna_gated", T, self.nh * self.dv, self.dtype)
            ops.gate_pack(att, hd, proj if self.gate else None, self.g_off, gated, self.nh, self.dv)
            att = gated
        return self.o_proj(att, ctx.ws.rows("qna_branch", T, self.hidden, self.dtype))


register_part("mixer", "qk_norm_attention", QKNormAttention)
