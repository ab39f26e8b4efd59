"""A causal language model built from a `ModelSpec`: embedding, blocks in their run order,
final norm, head. It holds no size of its own and knows no architecture.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:89-101` (embed, run the
layers carrying (hidden, residual), final norm) and `:123-127` (head), with one difference that
is ours: the head runs only on the rows whose logits are wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..parts.base import Part, build_part, part_class
from ..parts.spec import CacheNeed, ModelSpec, WeightSpec


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype):
        self.spec, self.dtype = spec, dtype
        self.embedding = build_part("embedding", spec.embedding, dtype)
        self.blocks = []
        for ls in spec.layers:
            arr = part_class("arrangement", ls.arrangement)
            if (ls.ffn is None) != (ls.ffn_norm is None):
                raise ValueError("a layer has a feed-forward and its norm, or neither")
            self.blocks.append(arr(build_part("norm", ls.mixer_norm, dtype), build_part("mixer", ls.mixer, dtype),
                                   None if ls.ffn_norm is None else build_part("norm", ls.ffn_norm, dtype),
                                   None if ls.ffn is None else build_part("feed_forward", ls.ffn, dtype), ls.params))
        self.final_norm = build_part("norm", spec.final_norm, dtype)
        self.head = build_part("head", spec.head, dtype)
        self.order = list(spec.order)
        self.pass_vectors = None if spec.pass_vectors is None else build_part("embedding", spec.pass_vectors, dtype)
        for i, st in enumerate(self.order):
            if st.add_row is not None:
                if self.pass_vectors is None or not 0 <= st.add_row < self.pass_vectors.rows:
                    raise ValueError(f"run order entry {i} adds row {st.add_row} of a table the model does not have")
                if not self.blocks[st.layer].takes_pre_add:
                    raise ValueError(f"run order entry {i}: its block's arrangement cannot add a vector first")
            if st.add_embedding and (st.add_row is not None or not self.blocks[st.layer].takes_pre_add):
                raise ValueError(f"run order entry {i}: the embedding's output cannot be added before this block (or not beside a table row)")
            if not 0 <= st.layer < len(self.blocks):
                raise ValueError(f"run order entry {i} names layer {st.layer}, which does not exist")
            if st.cache_from is not None and not (0 <= st.cache_from < i and self.order[st.cache_from].cache_from is None):
                raise ValueError(f"run order entry {i}: cache_from must name an earlier entry that owns its cache")
        self.keeps_embedding = any(st.add_embedding for st in self.order)
        self.hidden = self.embedding.hidden
        self.vocab = self.head.vocab
        # decode steps are replayed as CUDA graphs only if every part says it can be (`Part.graph_safe`)
        self.graph_safe = all(p.graph_safe for p in self.parts())

    # -- weights ---------------------------------------------------------------------------
    def parts(self) -> List[Part]:
        out: List[Part] = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        if self.pass_vectors is not None:
            out.append(self.pass_vectors)
        out += [self.final_norm, self.head]
        return out

    def weight_specs(self) -> List[Tuple[Part, WeightSpec]]:
        return [(p, ws) for p in self.parts() for ws in p.weight_specs()]

    # -- cache -----------------------------------------------------------------------------
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """One entry per run-order entry: what it keeps (None: nothing, or it reads another's; a `CacheNeed`; or a tuple of
        them, for a mixer that keeps several things); then one more for the
        embedding, if that keeps something of a request between steps (`embedding_cache_index`)."""
        needs = []
        for st in self.order:
            needs.append(None if st.cache_from is not None else self.blocks[st.layer].mixer.cache_need())
        if self.embedding_cache_index is not None:
            needs.append(self.embedding.cache_need())
        return needs

    @property
    def embedding_cache_index(self) -> Optional[int]:
        need = getattr(self.embedding, "cache_need", None)
        return len(self.order) if need is not None and need() is not None else None

    # -- forward ---------------------------------------------------------------------------
    def forward(self, ctx, caches) -> torch.Tensor:
        """Runs the tokens of `ctx` and returns float32 logits [len(ctx.want_rows), vocab].
        `caches[i]` is the cache view of run-order entry i."""
        T = ctx.T
        resid = ctx.ws.rows("resid", T, self.hidden, torch.float32)
        if getattr(self.embedding, "takes_context", False):    # an embedding that reads positions or keeps state
            ec = self.embedding_cache_index
            self.embedding.forward(ctx.token_ids, resid, ctx, caches[ec] if ec is not None else None)
        else:
            self.embedding.forward(ctx.token_ids, resid)
        emb_out = None
        if self.keeps_embedding:                  # a later entry adds the embedding's output again: a second copy of it, float32
            emb_out = ctx.ws.rows("embedding_out", T, self.hidden, torch.float32)
            if getattr(self.embedding, "takes_context", False):
                raise ValueError("an embedding that keeps state cannot be run twice in a step")
            self.embedding.forward(ctx.token_ids, emb_out)
        pending = None
        for i, st in enumerate(self.order):
            # the block that runs next may take its first norm half done (its weights applied, the rms still to divide by)
            blk = self.blocks[st.layer]
            nxt_st = self.order[i + 1] if i + 1 < len(self.order) else None
            nxt = self.blocks[nxt_st.layer] if nxt_st is not None and nxt_st.add_row is None and not nxt_st.add_embedding else None
            kw = {"pre_add": emb_out} if st.add_embedding else {} if st.add_row is None else {"pre_add": self.pass_vectors.row(st.add_row)}
            if blk.takes_next_block:
                pending = blk.run(resid, pending, ctx, caches[i], next_block=nxt, **kw)
            elif blk.takes_next_norm and nxt is not None and nxt.accepts_normed_input(T):
                pending = blk.run(resid, pending, ctx, caches[i], next_norm=nxt.mixer_norm, **kw)
            else:
                pending = blk.run(resid, pending, ctx, caches[i], **kw)
            if ctx.tap is not None:
                ctx.tap(f"layer{i}", resid, pending)
        n = ctx.n_want
        logits = ctx.ws.rows("logits", n, self.vocab, torch.float32)
        if n == 0:
            return logits
        if isinstance(pending, ops.ResidualCopy) or getattr(pending, "nothing_pending", False):   # the last block added its branches itself
            pending = None
        branch, bscale = pending if pending is not None else (None, 1.0)
        normed = self.final_norm.add_norm(resid, branch, bscale, ctx.ws.rows("final_normed", n, self.hidden, self.dtype),
                                          rows=ctx.want_rows)
        return self.head.forward(normed, logits)
