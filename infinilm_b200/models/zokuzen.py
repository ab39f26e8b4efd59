"""Zokuzen described as data: a decoder that keeps several copies of its residual stream ("hyper-connections": a sublayer
reads a weighted sum of the copies through a norm, and its output goes back into every copy while the copies are mixed
among themselves), whose layers mix tokens in one of three ways - "attention": grouped-query softmax attention whose
queries and keys are normed over the whole projection, rotated on part of each head, and which sees runs of positions
(a layer may read the keys and values another layer cached); "latent_attention": keys and values of every head are
up-projections of one normed latent per token, the only thing cached, over a sliding window, without positions; "wkv": a
recurrence over a matrix state per head with a decay per key channel that depends on the token - and whose feed-forwards
route each token to a few of several small gated units (some of which may return their input) beside a gated shared unit.

config.json: `vocab`, `width`, `streams`, `norm.eps`, `layers` (per layer `type`, `mixer` with its sizes and constants, `mlp` -
`kind` "moe" with `expert.ff`, `router` {experts, top, identity, scale}, `shared.ff` - or null). Tensors: `embed` (also the
output head), `l<i>.norm1|norm2` (stored as deviations from one), `l<i>.hc1|hc2.in|out|mix`, `l<i>.mix.*`, `l<i>.mlp.*`,
`final.norm`. Every constant of the design is in config.json.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..config.model_config import ConfigError, ModelConfig, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXERS = ("attention", "latent_attention", "wkv")
FEED_FORWARDS = ("moe",)


def _obj(raw: Dict[str, Any], key: str, required: bool = True) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: key '{key}' must be an object")
    return v


def _mask(m: Dict[str, Any]) -> Optional[int]:
    mk = _obj(m, "mask", required=False)
    if mk is None:
        return None
    size = take(mk, "size", int)
    if size < 1:
        raise ConfigError("config.json: mask.size must be positive")
    return size


def _mixer(typ: str, m: Dict[str, Any]) -> Dict[str, Any]:
    if typ == "wkv":
        return {"heads": take(m, "heads", int), "dim": take(m, "dim", int), "decay_rank": take(m, "decay_rank", int, None)}
    out = {"heads": take(m, "heads", int), "dim": take(m, "dim", int), "scale": take(m, "scale", float), "mask": _mask(m)}
    out["vdim"] = take(m, "vdim", int, out["dim"])
    if typ == "latent_attention":
        out["kv_rank"] = take(m, "kv_rank", int)
        return out
    out["kv_heads"] = take(m, "kv_heads", int, out["heads"])
    out["kv_from"] = take(m, "kv_from", int, None)
    rot = _obj(m, "rot", required=False)
    out["rot"] = None
    if rot is not None and take(rot, "dims", int, 0) > 0:
        out["rot"] = {"dims": take(rot, "dims", int), "base": take(rot, "base", float)}
        if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["dim"]:
            raise ConfigError("config.json: rot.dims must be even and at most the head's dim")
    return out


def _mlp(f: Dict[str, Any]) -> Dict[str, Any]:
    kind = take(f, "kind", str)
    if kind not in FEED_FORWARDS:
        raise ConfigError(f"config.json: feed-forward kind {kind!r} (known: {', '.join(FEED_FORWARDS)})")
    r = _obj(f, "router")
    sh = _obj(f, "shared", required=False)
    return {"kind": kind, "ff": take(_obj(f, "expert"), "ff", int), "experts": take(r, "experts", int), "top": take(r, "top", int),
            "identity": take(r, "identity", int, 0), "scale": take(r, "scale", float, 1.0),
            "shared_ff": None if sh is None else take(sh, "ff", int)}


@dataclass
class ZokuzenConfig(ModelConfig):
    norm_eps: float = 0.0
    streams: int = 1
    layers: List[Dict[str, Any]] = field(default_factory=list)
    tie_word_embeddings: bool = True              # the output head is the embedding table

    @classmethod
    def from_json(cls, raw: Dict[str, Any]) -> "ZokuzenConfig":
        raw = dict(raw)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out_layers = []
        for i, L in enumerate(layers):
            typ = take(L, "type", str)
            if typ not in MIXERS:
                raise ConfigError(f"config.json: layer {i} has mixer type {typ!r} (known: {', '.join(MIXERS)})")
            f = _obj(L, "mlp", required=False)
            out_layers.append({"type": typ, "mixer": _mixer(typ, _obj(L, "mixer")), "mlp": None if f is None else _mlp(f)})
        for i, L in enumerate(out_layers):          # a layer that reads another's keys and values: that one has its own, laid out alike
            src = L["mixer"].get("kv_from")
            if src is None:
                continue
            ok = 0 <= src < i and out_layers[src]["type"] == "attention" and out_layers[src]["mixer"].get("kv_from") is None
            if not ok or any(out_layers[src]["mixer"][k] != L["mixer"][k] for k in ("kv_heads", "dim", "vdim")):
                raise ConfigError(f"config.json: layer {i}: kv_from must name an earlier 'attention' layer with keys of its own "
                                  "and the same kv_heads, dim and vdim")
        cfg = cls(architecture="Zokuzen", model_type="zokuzen", vocab_size=take(raw, "vocab", int), hidden_size=take(raw, "width", int),
                  max_position_embeddings=1 << 30, torch_dtype="bfloat16", eos_token_ids=[], raw=raw,
                  norm_eps=take(_obj(raw, "norm"), "eps", float), streams=take(raw, "streams", int, 1), layers=out_layers)
        if cfg.vocab_size <= 0 or cfg.hidden_size <= 0 or cfg.streams < 1:
            raise ConfigError("config.json: vocab, width and streams must be positive")
        return cfg


def run_order(cfg: ZokuzenConfig) -> List[RunStep]:
    """Every layer once; a layer with `kv_from` reads the cache of that layer's entry."""
    return [RunStep(i, cache_from=L["mixer"].get("kv_from")) for i, L in enumerate(cfg.layers)]


def describe(cfg: ZokuzenConfig) -> ModelSpec:
    W, eps = cfg.hidden_size, cfg.norm_eps

    def norm(prefix: str, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": eps, "weight_offset": 1.0, "name": name}, prefix)
    layers = []
    for i, L in enumerate(cfg.layers):
        m, f, typ = L["mixer"], L["mlp"], L["type"]
        if typ == "wkv":
            mixer = PartSpec("channel_decay", {"hidden": W, "n_heads": m["heads"], "dim": m["dim"], "decay_rank": m["decay_rank"], "eps": eps},
                             f"l{i}.mix")
        elif typ == "latent_attention":
            mixer = PartSpec("latent_attention", {"hidden": W, "n_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"], "q_rank": None,
                                                  "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps, "sink": False, "gate": False,
                                                  "window": m["mask"]}, f"l{i}.mix")
        else:
            pos = None if m["rot"] is None else PartSpec("rope", {"rot_dim": m["rot"]["dims"], "theta": m["rot"]["base"]})
            mixer = PartSpec("qk_norm_attention", {"hidden": W, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "qk_dim": m["dim"],
                                                   "v_dim": m["vdim"], "scale": m["scale"], "eps": eps, "norm_over": "projection",
                                                   "position": pos, "chunk": m["mask"], "own_kv": m["kv_from"] is None}, f"l{i}.mix")
        ffn = ffn_norm = None
        if f is not None:
            ffn = PartSpec("routed_experts", {"hidden": W, "n_experts": f["experts"], "top": f["top"], "expert_ff": f["ff"],
                                              "shared_ff": f["shared_ff"], "router_bias": True, "bias_name": "correction",
                                              "route_rule": "softmax_all", "route_scale": f["scale"], "n_identity": f["identity"],
                                              "shared_gate": f["shared_ff"] is not None}, f"l{i}.mlp")
            ffn_norm = norm(f"l{i}", "norm2")
        layers.append(LayerSpec("hyper_connections", norm(f"l{i}", "norm1"), mixer, ffn_norm, ffn, {"streams": cfg.streams, "prefix": f"l{i}"}))
    return ModelSpec(
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": W, "scale": 1.0, "name": "embed", "exact": True}, ""),
        layers=layers, order=run_order(cfg), final_norm=norm("final", "norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab_size, "hidden": W, "scale": 1.0, "tied_to": "embed", "name": "head"}, ""))


register_architecture(["Zokuzen", "zokuzen"], ZokuzenConfig, describe)
