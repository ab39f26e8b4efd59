"""Data that describes a model: which parts each layer is made of and the order layers run in.

An architecture's `describe(config)` returns a `ModelSpec`. Nothing in it is code: a part is
named by its kind (a key of the part registries) and carries its sizes and constants as
parameters, so two layers of one model may use different mixers or feed-forwards, and the run
order may name a layer twice or let a layer read another entry's cache.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    kind: str                                   # registry key, e.g. "attention", "swiglu", "rmsnorm"
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""                            # checkpoint name prefix of this part's tensors


@dataclass
class LayerSpec:
    """One block: two norms, a mixer and a feed-forward, and how they are arranged."""
    arrangement: str                            # registry key of the block, e.g. "prenorm_residual"
    mixer_norm: PartSpec
    mixer: PartSpec
    ffn_norm: Optional[PartSpec]                # None (with ffn None): the layer has no feed-forward
    ffn: Optional[PartSpec]
    params: Dict[str, Any] = field(default_factory=dict)   # e.g. {"residual_scale": s}


@dataclass
class RunStep:
    """One entry of the run order. `layer` indexes `ModelSpec.layers`.

    `cache_from` names an earlier entry of the order whose cache this entry reads instead of
    keeping its own (it then writes nothing). `add_row`: row of the model's `pass_vectors` table that is added to the
    residual stream right before this entry runs (a model that runs some layers several times marks each pass so).
    `add_embedding`: the embedding's output - every token's row as it entered the first entry - is added to the residual
    stream right before this entry runs (a model that feeds its input in again at the start of a later pass)."""
    layer: int
    cache_from: Optional[int] = None
    add_row: Optional[int] = None
    add_embedding: bool = False


@dataclass
class ModelSpec:
    embedding: PartSpec
    layers: List[LayerSpec]
    order: List[RunStep]
    final_norm: PartSpec
    head: PartSpec
    pass_vectors: Optional[PartSpec] = None     # a table of residual-wide vectors that `RunStep.add_row` names


@dataclass
class WeightSpec:
    """One checkpoint tensor a part wants.

    role: "matrix" (operand of a matrix product: held in the compute dtype), "vector" (norm
          weights, biases: a tensor stored in 32-bit stays 32-bit), "table" (integer table: int32).
    init: ("normal", std) | ("ones_normal", std) | ("zeros",) - used by the random-weights mode.
    fallback: another tensor's full name used when this one is absent (a tied head).
    A dimension written as -1 is a size that the stored tensor itself gives (the part reads it in `set_weights`); `free` is the
    size the random-weights mode gives it."""
    name: str                                   # local name, e.g. "q_proj.weight"
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal", 0.02)
    fallback: Optional[str] = None
    free: Optional[int] = None

    def fits(self, shape) -> bool:
        shape = tuple(shape)
        return len(shape) == len(self.shape) and all(w == g or (w == -1 and g >= 1) for w, g in zip(self.shape, shape))

    def drawn_shape(self) -> Tuple[int, ...]:
        if -1 in self.shape and self.free is None:
            raise ValueError(f"tensor {self.name}: a free dimension needs a size for random weights")
        return tuple(self.free if d == -1 else d for d in self.shape)


@dataclass
class CacheNeed:
    """What a mixer keeps between steps, per request.

    kind "paged_kv": keys and values in pages; `window` None keeps all keys, else only the last
    `window` positions are ever read, so pages behind the window are given back.
    kind "state": one fixed-size tensor of `shape` per request (slot 0 of the pool is the zero state).
    A mixer that keeps several things (pages and a state, two states) returns a tuple of needs from `cache_need()` and gets
    a tuple of views, in the same order."""
    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    shape: Tuple[int, ...] = ()
    dtype: str = "compute"                      # "compute" | "float32" | "int32"

    def group_key(self) -> Tuple:
        return (self.kind, self.n_kv_heads, self.head_dim, self.window, tuple(self.shape), self.dtype)
