"""Attention whose keys and values are up-projections of one small latent vector per token, the only thing it caches.

Per token (h its normed input, H heads, d query/key dimensions and e value dimensions a head, r the latent's width):
    c_q = rms(W_dq h) * n_q,  q = W_uq c_q                       queries through a latent of their own
    c   = rms(W_dkv h) * n_kv                                    the cached latent
    k_j = W_uk[j] c,  v_j = W_uv[j] c                            per head j
    p   = softmax over the keys i <= t of (q_j . k_j) * scale, with exp(sink_j) in the denominator besides
    y   = W_o (concat_j(sum_i p_i v_j,i) * sigmoid(W_g h))

(`q_rank` None: no query latent, q = W_q h.)

The cache holds c alone, so the products with W_uk and W_uv are moved to the query side, which changes no value:
    q_j . (W_uk[j] c) = (W_uk[j]^T q_j) . c                      a query of width r against the latents themselves
    sum_i p_i W_uv[j] c_i = W_uv[j] (sum_i p_i c_i)              the weighted latent, up-projected once per query
What runs over the cache is then attention with one shared key/value head of width r, keys and values being the same
vectors: the paged attention kernels of the framework, with a sink. No position enters anywhere.
Norm statistics, scores, softmax and sink are float32; the products run in the compute dtype with float32 sums.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .attention import PagedAttend
from .base import Mixer, register_part
from .linear import Linear
from .spec import CacheNeed, WeightSpec


class LatentAttention(Mixer):
    """params: hidden, n_heads, qk_dim, v_dim, q_rank (None: the queries are projected from the input directly, tensor `q`
    instead of `dq`, `dq.norm`, `uq`), kv_rank, scale, eps (of the two latent norms), sink (a learned
    number per head in the softmax's denominator), gate (heads multiplied by sigmoid(W_g h)), window (None: all keys)."""
    graph_safe = True
    # From this many rows on, the bfloat16 path hands the two per-head products to the library's batched product (written
    # straight into the [token, head, column] rows through a strided view) and applies the gate with a kernel of its own:
    # this package's per-head kernel is built for a decode step's few rows (measured at 16 heads, 128 -> 256: 2.4 us for 8
    # rows in a replayed step, but 34 us for 2,048 rows, 62 TFLOP/s).
    LIBRARY_FROM_ROWS = 256

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.nh = int(p["hidden"]), int(p["n_heads"])
        self.d, self.e = int(p["qk_dim"]), int(p["v_dim"])
        self.direct_q = p.get("q_rank") is None
        self.qr, self.r = (0 if self.direct_q else int(p["q_rank"])), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.has_sink, self.has_gate = bool(p.get("sink", True)), bool(p.get("gate", True))
        self.window: Optional[int] = p.get("window")
        if min(self.hidden, self.nh, self.d, self.e, self.r) <= 0 or (self.qr <= 0 and not self.direct_q):
            raise ValueError("latent attention: sizes must be positive")
        if self.r > 1024:
            raise ValueError(f"latent attention: a latent of width {self.r} is beyond the attention kernels (1024; the fast ones end at 256)")
        self.n_q = self.nh * self.d if self.direct_q else self.qr     # the first columns of the joint product: the queries, or their latent
        self.n_down = self.n_q + self.r + (self.nh * self.e if self.has_gate else 0)
        self.down = Linear(self.hidden, self.n_down, dtype)          # rows: query latent (or queries) | key/value latent | gate
        self.up_q = None if self.direct_q else Linear(self.qr, self.nh * self.d, dtype)
        self.out = Linear(self.nh * self.e, self.hidden, dtype)
        self.core = PagedAttend(dtype, self.nh, 1, self.r, self.scale, self.window,
                                force_plain=bool(p.get("plain_kernel", False)), prefill_kernel=str(p.get("prefill_kernel", "auto")),
                                shared_kv=True)                      # the latent goes to both planes of the cache: decoding reads one

    def weight_specs(self) -> List[WeightSpec]:
        H, W = self.nh, self.hidden
        specs = [WeightSpec("q", (H * self.d, W))] if self.direct_q else [
            WeightSpec("dq", (self.qr, W)), WeightSpec("dq.norm", (self.qr,), "vector", ("ones_normal", 0.05)),
            WeightSpec("uq", (H * self.d, self.qr), init=("normal", 0.08))]
        specs += [WeightSpec("dkv", (self.r, W)), WeightSpec("dkv.norm", (self.r,), "vector", ("ones_normal", 0.05)),
                 WeightSpec("uk", (H * self.d, self.r), init=("normal", 0.08)), WeightSpec("uv", (H * self.e, self.r), init=("normal", 0.08)),
                 WeightSpec("o", (W, H * self.e))]
        if self.has_sink:
            specs.append(WeightSpec("sink", (H,), "vector", ("normal", 1.0)))
        if self.has_gate:
            specs.append(WeightSpec("g", (H * self.e, W)))
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        H = self.nh
        self.down.set(torch.cat([t["q" if self.direct_q else "dq"], t["dkv"]] + ([t["g"]] if self.has_gate else []), dim=0))
        if not self.direct_q:
            self.up_q.set(t["uq"])
        self.out.set(t["o"])
        # W_uk[j]^T as [H, r, d]: the product that turns a head's query into a query against the latents
        self.uk_t = t["uk"].to(self.dtype).view(H, self.d, self.r).transpose(1, 2).contiguous()
        self.uv = t["uv"].to(self.dtype).view(H, self.e, self.r).contiguous()
        self._uk_t_kn, self._uv_kn = self.uk_t.transpose(1, 2), self.uv.transpose(1, 2)      # [H, K, N] views for the library's batched product
        vec = torch.float32 if self.dtype == torch.float32 else t["dkv.norm"].dtype
        self.nq, self.nkv = (None if self.direct_q else t["dq.norm"].to(vec).contiguous()), t["dkv.norm"].to(vec).contiguous()
        self.core.sink = t["sink"].to(torch.float32).contiguous() if self.has_sink else None

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed("paged_kv", n_kv_heads=1, head_dim=self.r, window=self.window)

    def accepts_normed(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_ok(T, self.hidden)

    def fuses_tail(self, T):
        return self.dtype == torch.bfloat16 and ops.skinny_resid_ok(T, self.nh * self.e, self.hidden)

    def forward(self, x, ctx, cache, tail=None):
        T, H = x.shape[0], self.nh
        ws, dt = ctx.ws, self.dtype
        if isinstance(x, ops.NormedInput):       # rows whose norm the branch before left unfinished: this product divides by the rms
            proj = ws.rows("lat_down", T, self.n_down, dt)
            ops.gemm_skinny(x.xw, self.down.weight, proj, self.down.alpha, self.down.bias, norm_in=x)
        else:
            proj = self.down(x, ws.rows("lat_down", T, self.n_down, dt))
        cq = None if self.direct_q else ws.rows("lat_cq", T, self.qr, dt)
        ops.latent_norm_store(proj, 0, self.qr, self.n_q, self.r, self.nq, self.nkv, self.eps, cq, None, ctx.tok_pos, ctx.tok_entry,
                              cache.block_table, cache.storage if cache.writable else None, cache.page_size)
        q = proj[:, :self.n_q] if self.direct_q else self.up_q(cq, ws.rows("lat_q", T, H * self.d, dt))
        library = dt == torch.bfloat16 and T >= self.LIBRARY_FROM_ROWS and not bool(self.params.get("own_products_only", False))
        q_lat = ws.rows("lat_qlat", T, H * self.r, dt)
        if library:
            torch.bmm(q.view(T, H, self.d).transpose(0, 1), self._uk_t_kn, out=q_lat.view(T, H, self.r).transpose(0, 1))
        else:
            ops.gemm_grouped(q.view(T, H, self.d), self.uk_t, q_lat.view(T, H, self.r))
        o_lat = ws.rows("lat_olat", T, H * self.r, dt)
        self.core.run(q_lat, o_lat, ctx, cache)
        o = ws.rows("lat_o", T, H * self.e, dt)
        gate = proj[:, self.n_q + self.r:] if self.has_gate else None
        if library:
            torch.bmm(o_lat.view(T, H, self.r).transpose(0, 1), self._uv_kn, out=o.view(T, H, self.e).transpose(0, 1))
            if gate is not None:
                ops.sigmoid_gate(o, gate)
        else:
            ops.gemm_grouped(o_lat.view(T, H, self.r), self.uv, o.view(T, H, self.e), gate=None if gate is None else gate.view(T, H, self.e))
        if tail is not None:                      # the output product adds into the residual and prepares the next norm itself
            return ops.gemm_skinny_resid(o, self.out.weight, self.out.alpha, self.out.bias, tail.resid, tail.scale, tail.norm.weight,
                                         tail.norm.eps, ws.rows("xw_mixer", T, self.hidden, dt),
                                         ws.rows("sumsq_mixer", T, (self.hidden + 15) // 16, torch.float32))
        return self.out(o, ws.rows("branch", T, self.hidden, dt))


register_part("mixer", "latent_attention", LatentAttention)
