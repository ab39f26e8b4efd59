"""Somipel described as data: a decoder whose sublayers read the residual stream itself and whose norms sit on their
outputs (x += m * norm(sublayer(x))), and whose layers mix tokens in one of three ways: softmax attention with normed
queries and keys, a learned bias by distance and an output gate ("attention", which may read the keys and values another
layer cached); softmax attention whose values are its un-normed keys, with a query temperature that grows with the
position and a sink in the softmax ("attention_2"); and the matrix memory of an xLSTM block ("mlstm"). Feed-forwards are
gated with SiLU and may be absent.

config.json: `vocab`, `width`, `norm.eps`, `residual_mult`, `layers` (per layer `type`, `mixer` with its sizes and constants,
`mlp` - `kind` "dense" with `ff` - or null). Tensors: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.gate|up|down`,
`final.norm`, `head`. The bias table's row count is the stored tensor's (`bias_rows` may name it: the random-weights mode
needs a number). The constant of the design that is not in config.json: 1e-6 in the matrix memory's denominator.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..config.model_config import ConfigError, ModelConfig, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep

DENOM_EPS = 1e-6
MIXERS = ("attention", "attention_2", "mlstm")
FEED_FORWARDS = ("dense",)


def _obj(raw: Dict[str, Any], key: str, required: bool = True) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: key '{key}' must be an object")
    return v


def _mixer(typ: str, m: Dict[str, Any]) -> Dict[str, Any]:
    if typ == "mlstm":
        out = {k: take(m, k, int) for k in ("heads", "dim", "vdim")}
        out["gate_cap"] = take(m, "gate_cap", float)
        return out
    out = {k: take(m, k, int) for k in ("heads", "kv_heads", "dim")}
    out["scale"] = take(m, "scale", float)
    if typ == "attention":
        out["vdim"] = take(m, "vdim", int)
        out["bias_max"] = take(m, "bias_max", int)
        out["bias_rows"] = take(m, "bias_rows", int, None)
        out["kv_from"] = take(m, "kv_from", int, None)
    else:
        out["vdim"] = take(m, "vdim", int, out["dim"])
        if out["vdim"] != out["dim"]:
            raise ConfigError("config.json: a mixer whose values are its keys has vdim = dim")
        qt = _obj(m, "q_temp", required=False)
        out["q_temp"] = None if qt is None else {"coef": take(qt, "coef", float), "every": take(qt, "every", int)}
    return out


@dataclass
class SomipelConfig(ModelConfig):
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    layers: List[Dict[str, Any]] = field(default_factory=list)

    @classmethod
    def from_json(cls, raw: Dict[str, Any]) -> "SomipelConfig":
        raw = dict(raw)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out_layers = []
        for i, L in enumerate(layers):
            typ = take(L, "type", str)
            if typ not in MIXERS:
                raise ConfigError(f"config.json: layer {i} has mixer type {typ!r} (known: {', '.join(MIXERS)})")
            mixer = _mixer(typ, _obj(L, "mixer"))
            mlp = None
            f = _obj(L, "mlp", required=False)
            if f is not None:
                kind = take(f, "kind", str)
                if kind not in FEED_FORWARDS:
                    raise ConfigError(f"config.json: layer {i} has feed-forward kind {kind!r} (known: {', '.join(FEED_FORWARDS)})")
                mlp = {"kind": kind, "ff": take(f, "ff", int)}
            out_layers.append({"type": typ, "mixer": mixer, "mlp": mlp})
        for i, L in enumerate(out_layers):          # a layer that reads another's keys and values: that one has its own, of the same sizes
            src = L["mixer"].get("kv_from")
            if src is None:
                continue
            ok = 0 <= src < i and out_layers[src]["type"] == "attention" and out_layers[src]["mixer"].get("kv_from") is None
            if not ok or any(out_layers[src]["mixer"][k] != L["mixer"][k] for k in ("kv_heads", "dim", "vdim")):
                raise ConfigError(f"config.json: layer {i}: kv_from must name an earlier 'attention' layer with keys of its own "
                                  "and the same kv_heads, dim and vdim")
        cfg = cls(architecture="Somipel", model_type="somipel", vocab_size=take(raw, "vocab", int), hidden_size=take(raw, "width", int),
                  max_position_embeddings=1 << 30, torch_dtype="bfloat16", eos_token_ids=[], raw=raw,
                  norm_eps=take(_obj(raw, "norm"), "eps", float), residual_mult=take(raw, "residual_mult", float, 1.0), layers=out_layers)
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg


def run_order(cfg: SomipelConfig) -> List[RunStep]:
    """Every layer once; a layer with `kv_from` reads the cache of that layer's entry."""
    return [RunStep(i, cache_from=L["mixer"].get("kv_from")) for i, L in enumerate(cfg.layers)]


def describe(cfg: SomipelConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps

    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": eps, "name": name}, prefix)
    layers = []
    for i, L in enumerate(cfg.layers):
        m, f, typ = L["mixer"], L["mlp"], L["type"]
        if typ == "mlstm":
            mixer = PartSpec("matrix_lstm", {"hidden": W, "n_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"],
                                             "gate_cap": m["gate_cap"], "eps": eps, "den_eps": DENOM_EPS}, f"l{i}.mix")
        else:
            p = {"hidden": W, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "qk_dim": m["dim"], "v_dim": m["vdim"],
                 "scale": m["scale"], "eps": eps}
            if typ == "attention":
                p.update(qkv_bias=True, output_gate=True, own_kv=m["kv_from"] is None,
                         distance_bias={"rows": m["bias_rows"], "far": m["bias_max"]})
            else:
                p.update(value_from_key=True, sink_zero=True, q_temperature=m["q_temp"])
            mixer = PartSpec("qk_norm_attention", p, f"l{i}.mix")
        ffn = ffn_norm = None
        if f is not None:
            ffn = PartSpec("swiglu", {"hidden": W, "intermediate": f["ff"], "activation": "silu",
                                      "names": {"gate": "gate", "up": "up", "down": "down"}}, f"l{i}.mlp")
            ffn_norm = norm(f"l{i}", "norm2")
        layers.append(LayerSpec("branch_norm_residual", norm(f"l{i}", "norm1"), mixer, ffn_norm, ffn, {"residual_scale": cfg.residual_mult}))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": W, "scale": 1.0, "name": "embed", "exact": True}, ""),
        layers=layers, order=run_order(cfg), final_norm=norm("final", "norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": W, "scale": 1.0, "tied_to": None, "name": "head"}, ""))


register_architecture(["Somipel", "somipel"], SomipelConfig, describe)
