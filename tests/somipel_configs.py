"""Small Somipel configurations that differ from one another in every size and option, and weights for them: drawn by the
framework's random-weights mode (values that bfloat16 holds exactly, so every path and the oracle compute with the same
numbers), then changed so that faults show: query and key norm weights scaled up so that attention is peaked (a key that
is lost, a bias row that is one off or a sink that is left out moves the output), bias tables of the scores' own size,
gates of the matrix memory in ranges where its state matters for hundreds of tokens and its running maximum moves."""
from __future__ import annotations

from typing import Dict

import torch


def _ff(ff):
    return None if ff is None else {"kind": "dense", "ff": ff}


def _att(heads, kv_heads, dim, vdim, scale, bias_rows, bias_max, ff, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max, "bias_rows": bias_rows}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": _ff(ff)}


def _att2(heads, kv_heads, dim, scale, q_temp, ff):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention_2", "mixer": m, "mlp": _ff(ff)}


def _mlstm(heads, dim, vdim, cap, ff):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": _ff(ff)}


def sp_a() -> dict:
    # the matrix memory first; grouped keys (4 heads on 2) with key size 32 below value size 64 (tensor-memory prefill at 64);
    # a layer without a feed-forward; the last layer reads layer 1's keys and values with a bias table of its own size
    return {"architecture": "Somipel", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "layers": [_mlstm(3, 16, 24, 8.0, 72),
                       _att(4, 2, 32, 64, 0.2, 12, 40, 64),
                       _att2(4, 2, 48, 0.11, (0.7, 16), None),
                       _att(4, 2, 32, 64, 0.3, 8, 20, 40, kv_from=1)]}


def sp_b() -> dict:
    # a width that is no multiple of 16; no query temperature in one layer, a step of 7 in the other; value size below key
    # size (64 and 16); a table of 32 rows that reaches its last row at distance 128; head size 128 in the last layer
    return {"architecture": "Somipel", "vocab": 300, "width": 120, "norm": {"eps": 1e-4}, "residual_mult": 1.0,
            "layers": [_att2(6, 6, 16, 0.25, None, 100),
                       _att(2, 1, 64, 16, 0.15, 32, 128, None),
                       _mlstm(2, 40, 8, 15.0, 56),
                       _att2(3, 1, 128, 0.09, (0.3, 7), 88)]}


def sp_c() -> dict:
    # head size 128 for keys and values; a bias that still changes at distance 300, beyond most test sequences; two layers
    # that read layer 0's cache; a matrix memory with a tight cap on its gates and no feed-forward
    return {"architecture": "Somipel", "vocab": 128, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.25,
            "layers": [_att(2, 2, 128, 128, 0.09, 6, 300, 96),
                       _att(2, 2, 128, 128, 0.12, 10, 17, None, kv_from=0),
                       _mlstm(4, 8, 32, 2.0, None),
                       _att(2, 2, 128, 128, 0.05, 4, 3, 48, kv_from=0)]}


def sp_d() -> dict:
    # a key size beyond 256 in the matrix memory (its kernel with the state in shared memory), one head; key size 20 and value
    # size 12 (heads laid out at 32); a table of 4 rows that ends at distance 5; a query temperature that grows at every token
    return {"architecture": "Somipel", "vocab": 64, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
            "layers": [_mlstm(1, 272, 12, 15.0, 40),
                       _att(3, 3, 20, 12, 0.22, 4, 5, 24),
                       _att2(2, 1, 24, 0.2, (1.0, 1), 40)]}


SOMIPEL = {"a": sp_a, "b": sp_b, "c": sp_c, "d": sp_d}


def make_weights(raw: dict, seed: int, peak: float = 4.0) -> Dict[str, torch.Tensor]:
    """`peak`: the standard deviation the scaled scores of an attention layer are brought to through its query norm's weight
    (normed queries and keys: the norm weights set how peaked the softmax is) - a few keys then carry most of the weight,
    while rounding to bfloat16 does not yet decide which."""
    from infinilm_b200.config import config_from_json
    from infinilm_b200.weights import random_tensors
    w = random_tensors(config_from_json(raw), seed, "cpu")
    for name in list(w):
        x = w[name].float()
        layer = raw["layers"][int(name[1:name.index(".")])] if name.startswith("l") and "." in name else None
        typ = layer["type"] if layer else None
        if name == "embed":
            x = x * 50.0
        elif name == "head":
            x = x * 10.0
        elif name.endswith(".q.norm"):
            m = layer["mixer"]
            x = x * peak / (m["scale"] * 2.0 * m["dim"] ** 0.5)
        elif name.endswith(".k.norm"):
            x = x * 2.0
        elif name.endswith(".rel"):
            x = x * 4.0
        elif name.endswith((".mix.q", ".mix.k", ".mix.v", ".mix.g")):
            x = x * (3.0 if typ == "mlstm" else 2.0)
        elif name.endswith((".q.b", ".k.b", ".v.b")):
            x = x * 20.0
        elif name.endswith((".mix.i", ".mix.f")):
            x = x * 6.0
        elif name.endswith(".f.b"):
            x = x * 2.0 + 3.0                     # forget gates mostly near one: the state carries far
        elif name.endswith(".i.b"):
            x = x * 4.0
        else:
            continue
        w[name] = x.to(torch.bfloat16)
    return w


def token_ids(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
