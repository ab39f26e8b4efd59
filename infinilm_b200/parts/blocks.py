"""Arrangements: how a layer's parts sit around the residual stream.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:49-57` (fused-residual
form: each norm first adds the previous branch to the residual, then normalises it) and `:59-71`
(the same as h += s*Attn(norm(h)); h += s*MLP(norm(h))). The branch scale s is a parameter of the
arrangement; InfiniLM passes it as the `alpha` of o_proj and down_proj (`:27,33`), here it
multiplies the branch in f32 inside the fused add, where the residual sum is kept in f32.
"""
from __future__ import annotations

import os
from typing import Dict, List

import torch

from .. import ops
from .base import Arrangement, Part, ResidualTail, register_part
from .spec import WeightSpec


class PreNormResidual(Arrangement):
    """params: residual_scale (default 1)."""

    # On a decode step of a few rows an add+norm kernel between two weight-streaming products costs about as much as
    # its boundary to them; where the parts on both sides can, the product before does the add and the product after
    # the division by the rms (ResidualTail / NormedInput). INFINILM_B200_FUSE_NORM=0: always the kernel.
    FUSE_NORM = os.environ.get("INFINILM_B200_FUSE_NORM", "1") != "0"

    takes_next_norm = True
    takes_pre_add = True

    def accepts_normed_input(self, T):
        return self.FUSE_NORM and self.mixer_norm.fusable_rms and self.mixer.accepts_normed(T)

    def run(self, resid, pending, ctx, cache, next_norm=None, pre_add=None):
        s = float(self.params.get("residual_scale", 1.0))
        T, H = resid.shape
        fuse = self.FUSE_NORM and ctx.tap is None
        if isinstance(pending, ops.NormedInput):
            if pre_add is not None:
                raise ValueError("a block that adds a vector first cannot take its first norm half done")
            normed = pending
        else:
            if isinstance(pending, ops.ResidualCopy) or getattr(pending, "nothing_pending", False):     # the block before left nothing to add
                pending = None
            branch, bscale = pending if pending is not None else (None, 1.0)
            if pre_add is None:
                normed = self.mixer_norm.add_norm(resid, branch, bscale, ctx.ws.rows("normed", T, H, ctx.dtype))
            else:
                normed = self.mixer_norm.add_norm(resid, branch, bscale, ctx.ws.rows("normed", T, H, ctx.dtype), vec=pre_add)
        if self.ffn is None:                      # a layer without a feed-forward: the mixer's branch is the block's
            return self.mixer.forward(normed, ctx, cache), s
        if fuse and self.ffn_norm.fusable_rms and self.mixer.fuses_tail(T) and self.ffn.accepts_normed(T):
            normed = self.mixer.forward(normed, ctx, cache, tail=ResidualTail(resid, s, self.ffn_norm))
        else:
            branch = self.mixer.forward(normed, ctx, cache)
            normed = self.ffn_norm.add_norm(resid, branch, s, ctx.ws.rows("normed", T, H, ctx.dtype))
        if fuse and next_norm is not None and next_norm.fusable_rms and self.ffn.fuses_tail(T):
            return self.ffn.forward(normed, ctx, tail=ResidualTail(resid, s, next_norm))
        branch = self.ffn.forward(normed, ctx)
        return branch, s


class BranchNormResidual(Arrangement):
    """h += s * norm1(mixer(h)); h += s * norm2(ffn(h)): the sublayers read the residual stream itself and the norms sit on
    their outputs. params: residual_scale (default 1). The stream stays float32; each sublayer reads its copy in the compute
    dtype, which the kernel that adds the sublayer before it writes along (one kernel: statistics of the branch row, the
    scaled add, the copy). Unlike a norm in front of a product, this one cannot move into the product before it: its
    statistics are those of that product's whole output row, which the product's blocks only hold between them."""

    takes_pre_add = True

    def _stream_copy(self, resid, ctx, tag="stream_copy"):
        if ctx.dtype == torch.float32:
            return resid
        T, H = resid.shape
        copy = ctx.ws.rows(tag, T, H, ctx.dtype)
        ops.cast_rows(resid, copy)
        return copy

    def run(self, resid, pending, ctx, cache, pre_add=None):
        s = float(self.params.get("residual_scale", 1.0))
        T, H = resid.shape
        x = None
        if getattr(pending, "nothing_pending", False):    # a block that kept several copies of the stream: their sum is in `resid`
            pending = None
        if isinstance(pending, ops.ResidualCopy) and pre_add is None:
            x = pending.rows
        elif isinstance(pending, ops.NormedInput):
            raise ValueError("a block that reads the residual stream itself cannot take a half-done norm")
        elif pending is not None and not isinstance(pending, ops.ResidualCopy) or pre_add is not None:
            # a block of another arrangement left its branch to be added (or a vector comes first): add it with the framework's
            # add + norm kernel, whose normalised rows are not needed here
            branch, bscale = pending if isinstance(pending, tuple) else (None, 1.0)
            self.mixer_norm.add_norm(resid, branch, bscale, ctx.ws.rows("normed", T, H, ctx.dtype), vec=pre_add)
        if x is None:
            x = self._stream_copy(resid, ctx)
        # the add behind a sublayer writes the stream's new copy over the one that sublayer has read (kernels run in order)
        copy = None if ctx.dtype == torch.float32 else x
        branch = self.mixer.forward(x, ctx, cache)
        self.mixer_norm.norm_add(resid, branch, s, copy)
        if self.ffn is not None:
            branch = self.ffn.forward(x, ctx)
            self.ffn_norm.norm_add(resid, branch, s, copy)
        return ops.ResidualCopy(x)


class StreamWeights(Part):
    """The numbers by which a block with several copies of the residual stream reads and writes them, per sublayer q (1: the
    mixer, 2: the feed-forward): hc<q>.in [S] (the sublayer's input is sum_s in[s] x_s), hc<q>.mix [S, S] (from, to) and
    hc<q>.out [S] (x_t <- sum_s mix[s, t] x_s + out[t] y). params: streams, sublayers. Held in float32."""
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.S, self.n_sub = int(params["streams"]), int(params["sublayers"])
        self.w_in, self.w_mix, self.w_out = {}, {}, {}

    def weight_specs(self) -> List[WeightSpec]:
        specs = []
        for q in range(1, self.n_sub + 1):
            specs += [WeightSpec(f"hc{q}.in", (self.S,), "vector", ("ones_normal", 0.3)),
                      WeightSpec(f"hc{q}.out", (self.S,), "vector", ("ones_normal", 0.3)),
                      WeightSpec(f"hc{q}.mix", (self.S, self.S), "vector", ("normal", 0.4))]
        return specs

    def set_weights(self, t: Dict[str, torch.Tensor]) -> None:
        for q in range(1, self.n_sub + 1):
            self.w_in[q] = t[f"hc{q}.in"].to(torch.float32).contiguous()
            self.w_out[q] = t[f"hc{q}.out"].to(torch.float32).contiguous()
            self.w_mix[q] = t[f"hc{q}.mix"].to(torch.float32).contiguous()


class HyperConnections(Arrangement):
    """Pre-norm sublayers over S copies of the residual stream (all equal to the embedding's output at the start):
        u = sum_s in[s] x_s;  y = sublayer(norm(u));  x_t <- sum_s mix[s, t] x_s + out[t] y   (every copy from the old ones)
    for the mixer and then the feed-forward, each with its own in / mix / out; what the model's last norm reads is the sum of
    the copies. params: streams, prefix (of the layer's hc<q>.* tensors). The copies live in the step's workspace as float32
    [T, S * H]; one kernel does what lies between two sublayers (write-back, the next input's sum and norm), also across the
    border to the next block of this kind; the model's `resid` receives the copies' sum where a block of another kind, the
    final norm or a debug tap reads it."""

    takes_next_block = True

    def __init__(self, mixer_norm, mixer, ffn_norm, ffn, params):
        super().__init__(mixer_norm, mixer, ffn_norm, ffn, params)
        self.S = int(params["streams"])
        if not 1 <= self.S <= ops.HYPER_MAX_STREAMS:
            raise ValueError(f"hyper-connections: 1 to {ops.HYPER_MAX_STREAMS} streams, not {self.S}")
        self.hc = StreamWeights({"streams": self.S, "sublayers": 1 if ffn is None else 2}, str(params.get("prefix", "")), mixer_norm.dtype)

    def parts(self):
        return super().parts() + [self.hc]

    def run(self, resid, pending, ctx, cache, next_block=None):
        T, H = resid.shape
        S, hc = self.S, self.hc
        streams = ctx.ws.rows("hc_streams", T, S * H, torch.float32)
        normed = ctx.ws.rows("normed", T, H, ctx.dtype)
        if isinstance(pending, ops.StreamSet):
            if pending.n_streams != S or pending.streams.data_ptr() != streams.data_ptr():
                raise ValueError("hyper-connections: the block before kept another number of streams")
            if pending.normed is not None:
                normed = pending.normed
            else:
                ops.hyper_step(streams, S, in_next=hc.w_in[1], norm_weight=self.mixer_norm.weight, eps=self.mixer_norm.eps, normed=normed)
        else:
            if isinstance(pending, ops.NormedInput):
                raise ValueError("hyper-connections: cannot take a half-done norm")
            if isinstance(pending, tuple):        # a block of another kind left its branch to be added to the one stream
                self.mixer_norm.add_norm(resid, pending[0], pending[1], normed)
            ops.hyper_step(streams, S, init=resid, in_next=hc.w_in[1], norm_weight=self.mixer_norm.weight, eps=self.mixer_norm.eps,
                           normed=normed)
        y = self.mixer.forward(normed, ctx, cache)
        q = 1
        if self.ffn is not None:
            normed = ctx.ws.rows("normed", T, H, ctx.dtype)
            ops.hyper_step(streams, S, y=y, mix=hc.w_mix[1], out_w=hc.w_out[1], in_next=hc.w_in[2], norm_weight=self.ffn_norm.weight,
                           eps=self.ffn_norm.eps, normed=normed)
            y = self.ffn.forward(normed, ctx)
            q = 2
        nxt = next_block if (isinstance(next_block, HyperConnections) and next_block.S == S and ctx.tap is None) else None
        if nxt is not None:                       # the write-back and the next block's first input in one pass
            normed = ctx.ws.rows("normed", T, H, ctx.dtype)
            ops.hyper_step(streams, S, y=y, mix=hc.w_mix[q], out_w=hc.w_out[q], in_next=nxt.hc.w_in[1], norm_weight=nxt.mixer_norm.weight,
                           eps=nxt.mixer_norm.eps, normed=normed)
            return ops.StreamSet(streams, S, normed)
        ops.hyper_step(streams, S, y=y, mix=hc.w_mix[q], out_w=hc.w_out[q], sum_out=resid)
        return ops.StreamSet(streams, S, None)


register_part("arrangement", "prenorm_residual", PreNormResidual)
register_part("arrangement", "hyper_connections", HyperConnections)
register_part("arrangement", "branch_norm_residual", BranchNormResidual)
