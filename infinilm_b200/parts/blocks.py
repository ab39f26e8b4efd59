"""Arrangements: how a layer's parts sit around the residual stream.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:49-57` (fused-residual
form: each norm first adds the previous branch to the residual, then normalises it) and `:59-71`
(the same as h += s*Attn(norm(h)); h += s*MLP(norm(h))). The branch scale s is a parameter of the
arrangement; InfiniLM passes it as the `alpha` of o_proj and down_proj (`:27,33`), here it
multiplies the branch in f32 inside the fused add, where the residual sum is kept in f32.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from .base import Arrangement, ResidualTail, register_part


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
            if isinstance(pending, ops.ResidualCopy):     # the block before left nothing to add
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


register_part("arrangement", "prenorm_residual", PreNormResidual)
register_part("arrangement", "branch_norm_residual", BranchNormResidual)
