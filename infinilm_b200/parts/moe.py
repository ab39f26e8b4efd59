"""A routed feed-forward: every token runs `top` of `n_experts` small gated units, chosen by a router, plus - if the
model has one - a shared unit that every token runs.

    z = W_r h + b (float32);  the `top` largest z are chosen;  their weights are the softmax over the chosen z alone
    y = sum_k weight_k * unit_{e_k}(h)  (+ shared(h)),   unit(h) = W_down (silu(W_gate h) * (W_up h))

A second routing rule (`route_rule` "softmax_all"): s = softmax(z) over every output of the router; the `top` largest of
s + c are chosen (c: a stored correction per output, which only steers the choice); the weights are the chosen s over their
sum (+ 1e-20), times `route_scale`. The router's last `n_identity` outputs may stand for units without weights that return
their input (weight_k * h), and the shared unit may be multiplied by sigmoid(w_sg . h), one number per token: that row
rides along as one more row of the router's product and takes no part in the choice.

Everything stays on the device: the router kernel writes the choices, a sort kernel orders the (token, choice) slots by
expert, two products over those ragged groups run the experts (gate and up as one product with the SiLU in its
epilogue, then down), and a combine kernel sums a token's rows in the order of its choices. Nothing is read back, so a
step can be replayed as a graph, and a token's result does not depend on what else is in the batch.

The ragged products are this package's kernel (`csrc/gemm_grouped.cu`: float32 on the FP32 pipes; bfloat16 on the
tensor cores, built to stream the chosen experts' weights once for the few rows of a decode step). A prompt portion of
many rows on the bfloat16 path calls the library's grouped product instead (`torch.nn.functional.grouped_mm`, the
rows gathered into the order of the groups first), as the framework's dense products of that size call the library.
"""
from __future__ import annotations

from typing import Dict, List

import torch
import torch.nn.functional as F

from .. import ops
from .base import FeedForward, register_part
from .feed_forward import SwiGLU
from .linear import Linear
from .spec import WeightSpec


class RoutedExperts(FeedForward):
    """params: hidden, n_experts (units with weights), top, expert_ff, shared_ff (None: no shared unit), router_bias;
    route_rule ("top_logits", the default, or "softmax_all"), route_scale, n_identity (router outputs behind the experts' that
    return the input), shared_gate (the shared unit times the sigmoid of a row `shared.sg` [1, hidden]), bias_name (the tensor
    of the router's per-output numbers: "router.b")."""
    graph_safe = True
    # From this many (token, choice) rows on, the bfloat16 path calls the library's grouped product. Measured on a B200 with
    # 64 experts of 2,048 x 1,408, 6 chosen: gate+up for 512 tokens 197 us here against 171 us there, for 2,048 tokens 593
    # against 163 us; for 64 tokens 162 against 167 us, for 8 tokens 94 us (the library was not built for so few rows).
    LIBRARY_FROM_SLOTS = 2048
    # From this many tokens on, the bfloat16 path takes the router's logits from a matrix product on the tensor cores
    # (bfloat16 operands, which the row and the weights are anyway, exact products, float32 sums and float32 logits) and
    # only chooses in a kernel of its own: the FFMA router re-reads every weight row for each four tokens (2,048 tokens x 64
    # experts x 2,048: 86 us). Below it, and in float32, the router kernel computes the logits itself in a fixed order.
    ROUTER_PRODUCT_FROM = 256

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        p = params
        self.hidden, self.n, self.top, self.ff = int(p["hidden"]), int(p["n_experts"]), int(p["top"]), int(p["expert_ff"])
        self.shared_ff = None if p.get("shared_ff") is None else int(p["shared_ff"])
        self.router_bias = bool(p.get("router_bias", True))
        rule = str(p.get("route_rule", "top_logits"))
        if rule not in ("top_logits", "softmax_all"):
            raise ValueError("routed experts: route_rule is 'top_logits' or 'softmax_all'")
        self.rule = ops.ROUTE_SOFTMAX_ALL if rule == "softmax_all" else ops.ROUTE_TOP_LOGITS
        self.route_scale, self.n_id = float(p.get("route_scale", 1.0)), int(p.get("n_identity", 0))
        self.has_sg = bool(p.get("shared_gate", False))
        self.bias_name = str(p.get("bias_name", "router.b"))
        self.n_out = self.n + self.n_id           # the router's outputs: the experts, then the identity units
        # anything beyond the first rule: the logits go through memory (a product, then the choice), never the fused router
        self.extended = self.rule != ops.ROUTE_TOP_LOGITS or self.n_id > 0 or self.has_sg
        if self.n_id < 0 or (self.has_sg and p.get("shared_ff") is None):
            raise ValueError("routed experts: n_identity >= 0; a shared gate needs a shared unit")
        if not 0 < self.top <= min(self.n_out, ops.MOE_MAX_TOP) or self.n <= 0:
            raise ValueError(f"routed experts: top {self.top} must be in 1..min(router outputs, {ops.MOE_MAX_TOP})")
        self.small_router = bool(p.get("small_router", True))        # False: a decode step's router as one block a token (tests compare the two)
        self.shared = None if self.shared_ff is None else SwiGLU({"hidden": self.hidden, "intermediate": self.shared_ff}, prefix, dtype)

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec("router", (self.n_out, self.hidden), init=("normal", 0.3))]
        if self.router_bias:
            specs.append(WeightSpec(self.bias_name, (self.n_out,), "vector", ("normal", 0.3 if self.rule == ops.ROUTE_TOP_LOGITS else 0.002)))
        if self.has_sg:
            specs.append(WeightSpec("shared.sg", (1, self.hidden), init=("normal", 0.1)))
        for e in range(self.n):
            specs += [WeightSpec(f"e{e}.gate", (self.ff, self.hidden), init=("normal", 0.05)),
                      WeightSpec(f"e{e}.up", (self.ff, self.hidden), init=("normal", 0.05)),
                      WeightSpec(f"e{e}.down", (self.hidden, self.ff), init=("normal", 0.05))]
        if self.shared is not None:
            specs += [WeightSpec("shared.gate", (self.shared_ff, self.hidden), init=("normal", 0.05)),
                      WeightSpec("shared.up", (self.shared_ff, self.hidden), init=("normal", 0.05)),
                      WeightSpec("shared.down", (self.hidden, self.shared_ff), init=("normal", 0.05))]
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        rows = [t["router"]] + ([t["shared.sg"]] if self.has_sg else [])       # the gate's row behind the router's
        if self.extended and (self.n_out + len(rows) - 1) % 8:                  # zero rows up to a multiple of 8: the library's product of
            pad = -(self.n_out + len(rows) - 1) % 8                             # many rows is far slower on an odd number of outputs
            rows.append(torch.zeros((pad, self.hidden), dtype=t["router"].dtype, device=t["router"].device))
        self.router = torch.cat(rows, dim=0).to(self.dtype).contiguous()
        self.router_lin = None
        if self.extended or (self.dtype == torch.bfloat16 and self.hidden % 8 == 0 and not bool(self.params.get("own_products_only", False))):
            self.router_lin = Linear(self.hidden, self.router.shape[0], self.dtype)
            self.router_lin.set(self.router)
        self.router_b = t[self.bias_name].contiguous() if self.router_bias else None
        if self.router_b is not None and self.dtype == torch.float32:
            self.router_b = self.router_b.to(torch.float32)
        # per expert: gate rows, then up rows (one product, SiLU(gate) * up in its epilogue); then down
        self.w_gate_up = torch.stack([torch.cat([t[f"e{e}.gate"], t[f"e{e}.up"]], dim=0) for e in range(self.n)]).to(self.dtype).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down"] for e in range(self.n)]).to(self.dtype).contiguous()
        # the library's grouped product wants bfloat16 with rows of whole 16-byte chunks; it reads the same weights, transposed views
        self.library_ok = (self.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.ff % 8 == 0 and hasattr(F, "grouped_mm")
                           and not bool(self.params.get("own_products_only", False)))
        self._w_gate_up_t, self._w_down_t = self.w_gate_up.transpose(1, 2), self.w_down.transpose(1, 2)
        if self.shared is not None:
            self.shared.set_weights({"gate_proj.weight": t["shared.gate"], "up_proj.weight": t["shared.up"],
                                     "down_proj.weight": t["shared.down"]})

    def accepts_normed(self, T):
        """A few rows (a decode step) whose norm the product before left unfinished: the router multiplies its copy of
        the rows by rstd and hands rstd to the ragged gate+up product's epilogue; the shared unit takes such rows anyway."""
        return (self.dtype == torch.bfloat16 and not self.extended and ops.skinny_ok(T, self.hidden) and self.hidden % 8 == 0
                and T * self.top < self.LIBRARY_FROM_SLOTS and T < self.ROUTER_PRODUCT_FROM
                and (self.shared is None or self.shared.accepts_normed(T)))

    def fuses_tail(self, T):
        """A few rows: the combine adds into the residual and leaves the next norm's inputs (it is the branch's last step)."""
        return (self.dtype == torch.bfloat16 and not self.extended and 0 < T <= ops.SKINNY_MAX_ROWS and self.hidden % 4 == 0
                and (self.hidden + 15) // 16 <= ops.NORM_MAX_BLOCKS)

    def forward(self, x, ctx, tail=None):
        T, W, k = x.shape[0], self.hidden, self.top
        ws, dt, n_slots = ctx.ws, self.dtype, x.shape[0] * self.top
        idx = ws.rows("moe_idx", T, k, torch.int32)
        wt = ws.rows("moe_wt", T, k, torch.float32)
        normed_in, rstd = None, None
        group_off = ws.flat("moe_group_off", self.n_out + 1, torch.int32)
        pos_of_slot = ws.rows("moe_pos", T, k, torch.int32).view(-1)
        row_of_pos = ws.rows("moe_row", T, k, torch.int32).view(-1)
        if isinstance(x, ops.NormedInput):       # x.xw = residual * norm weight; the division by the rms is still to come
            normed_in, rstd = x, ws.flat("moe_rstd", T, torch.float32)
        rows = x if normed_in is None else x.xw
        EZ = self.router.shape[0]
        small = dt == torch.bfloat16 and self.small_router and ops.route_sort_small_ok(T, W, EZ) and rows.stride(0) % 8 == 0
        if self.extended and self.rule == ops.ROUTE_TOP_LOGITS and self.router_b is not None and EZ != self.n_out:
            small = False                         # (a bias on the logits beside a gate's row: the product, then the choice)
        z = None
        if self.extended:
            # the logits (and the shared unit's gate, their last column) through memory; the bias only steers the choice
            z = ws.rows("moe_logits", T, EZ, torch.float32)
            if small:
                ops.moe_route_sort_small(rows, self.router, self.router_b, z, idx, wt, k, group_off, pos_of_slot, row_of_pos,
                                         extra=EZ - self.n_out, rule=self.rule, out_scale=self.route_scale)
            else:
                self.router_lin(x, z, out_f32=True)
                ops.moe_select(z[:, :self.n_out], self.router_b, idx, wt, k, rule=self.rule, out_scale=self.route_scale)
        elif small:
            # a decode step: the logits a warp per (token, expert), then one block that chooses and sorts (two short kernels
            # where a block a token was a chain of round trips to memory, and the sort a third launch)
            ops.moe_route_sort_small(rows, self.router, self.router_b, ws.rows("moe_logits", T, self.n, torch.float32), idx, wt, k,
                                     group_off, pos_of_slot, row_of_pos, norm_in=normed_in, rstd_out=rstd)
        elif normed_in is not None:
            ops.moe_route(x.xw, self.router, self.router_b, idx, wt, k, norm_in=x, rstd_out=rstd)
        elif self.router_lin is not None and T >= self.ROUTER_PRODUCT_FROM:
            z = self.router_lin(x, ws.rows("moe_logits", T, self.n, torch.float32), out_f32=True)
            ops.moe_select(z, self.router_b, idx, wt, k)
        else:
            ops.moe_route(x, self.router, self.router_b, idx, wt, k)
        if not small:
            ops.moe_sort(idx, self.n_out, group_off, pos_of_slot, row_of_pos)
        act = ws.rows("moe_act", T, k * self.ff, dt).view(n_slots, self.ff)
        y = ws.rows("moe_y", T, k * W, dt).view(n_slots, W)
        if self.library_ok and n_slots >= self.LIBRARY_FROM_SLOTS and normed_in is None:
            xs = ws.rows("moe_x_sorted", T, k * W, dt).view(n_slots, W)
            ops.gather_rows(x, row_of_pos, xs)
            ends = group_off[1:self.n + 1]        # (the places of identity units, behind the last expert's, are not computed)
            ops.swiglu(F.grouped_mm(xs, self._w_gate_up_t, offs=ends), act)
            y = F.grouped_mm(act, self._w_down_t, offs=ends)
        else:
            ops.gemm_grouped(x if normed_in is None else x.xw, self.w_gate_up, act, group_off=group_off, a_rows=row_of_pos, n_rows=n_slots,
                             glu=True, row_scale=rstd)
            ops.gemm_grouped(act, self.w_down, y, group_off=group_off, n_rows=n_slots)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        if tail is not None:
            return ops.moe_combine_resid(y, pos_of_slot, wt, shared, tail.resid, tail.scale, tail.norm.weight, tail.norm.eps,
                                         ws.rows("xw_ffn", T, W, dt), ws.rows("sumsq_ffn", T, (W + 15) // 16, torch.float32))
        out = ws.rows("moe_out", T, W, dt)
        ops.moe_combine(y, pos_of_slot, wt, shared, out, group_off=group_off if self.n_id else None, n_real=self.n,
                        x=x if self.n_id else None, shared_gate=z[:, self.n_out] if self.has_sg else None)
        return out


register_part("feed_forward", "routed_experts", RoutedExperts)
