"""Small Zokuzen configurations that differ from one another in every size and option, and weights for them: drawn by the
framework's random-weights mode (values that bfloat16 holds exactly, so every path and the oracle compute with the same
numbers), then changed so that faults show: query norm weights scaled so that attention is peaked (a key that is lost or
a mask edge that is one off moves the output), decays near one so that the recurrent state matters for hundreds of
tokens, router corrections large enough to change choices, stream mixing matrices near a rotation so that no copy dies."""
from __future__ import annotations

from typing import Dict

import torch


def _moe(ff, experts, top, identity, scale, shared_ff):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity, "scale": scale}}
    if shared_ff is not None:
        f["shared"] = {"ff": shared_ff}
    return f


def _att(heads, kv_heads, dim, vdim, scale, chunk, rot, mlp, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _lat(heads, dim, vdim, rank, scale, window, mlp):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                                                  "mask": {"size": window}}, "mlp": mlp}


def _wkv(heads, dim, mlp):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def zk_a() -> dict:
    # two streams; the recurrence first; a chunk of 24 positions (no multiple of a page) with rotation on 8 of 32 dimensions;
    # a window of 20 over a latent of 32; a borrowed cache with a chunk size of its own; one identity unit, top 2 of 5
    return {"architecture": "Zokuzen", "vocab": 211, "width": 96, "streams": 2, "norm": {"eps": 1e-5},
            "layers": [_wkv(3, 32, _moe(40, 4, 2, 1, 1.5, 48)),
                       _att(4, 2, 32, 48, 0.2, 24, (8, 10000.0), _moe(40, 4, 2, 1, 1.5, 48)),
                       _lat(4, 16, 24, 32, 0.3, 20, None),
                       _att(4, 2, 32, 48, 0.25, 17, (8, 10000.0), _moe(24, 3, 1, 0, 1.0, None), kv_from=1)]}


def zk_b() -> dict:
    # one stream (the plain residual as a special case); a width that is no multiple of 16; whole heads rotated; a chunk of
    # one page exactly; value size below key size; three identity units among six outputs, every output chosen (top 6)
    return {"architecture": "Zokuzen", "vocab": 300, "width": 120, "streams": 1, "norm": {"eps": 1e-4},
            "layers": [_att(6, 6, 16, 16, 0.25, 16, (16, 500.0), _moe(56, 3, 6, 3, 2.0, 64)),
                       _lat(2, 64, 16, 48, 0.15, 33, _moe(56, 3, 2, 3, 0.5, None)),
                       _wkv(2, 60, None)]}


def zk_c() -> dict:
    # four streams; head size 128 (the tensor-memory prefill kernel) without rotation; a chunk longer than most test
    # sequences and one of 5; a window of 1 (a token sees itself alone); a latent of 128 under 2 heads of 128
    return {"architecture": "Zokuzen", "vocab": 128, "width": 128, "streams": 4, "norm": {"eps": 1e-6},
            "layers": [_att(2, 1, 128, 128, 0.09, 400, None, _moe(32, 7, 3, 2, 2.5, 32)),
                       _att(2, 1, 128, 128, 0.12, 5, None, None, kv_from=0),
                       _lat(2, 128, 128, 128, 0.06, 1, _moe(32, 2, 1, 0, 1.0, 16)),
                       _wkv(8, 16, _moe(16, 2, 2, 1, 3.0, None)),
                       _lat(2, 128, 64, 64, 0.08, 64, None)]}


def zk_d() -> dict:
    # three streams; a key size beyond 256 in the recurrence (its kernel with the state in shared memory), one head; key size
    # 20 and value size 12 (heads laid out at 32) with 4 rotated dimensions; a latent of 24 (no multiple of 16: the plain
    # attention kernel); a window of 7
    return {"architecture": "Zokuzen", "vocab": 64, "width": 72, "streams": 3, "norm": {"eps": 1e-5},
            "layers": [_wkv(1, 272, _moe(24, 2, 1, 1, 1.0, 40)),
                       _att(3, 3, 20, 12, 0.22, 9, (4, 100.0), _moe(24, 2, 2, 0, 2.5, 40)),
                       _lat(3, 8, 12, 24, 0.35, 7, _moe(24, 5, 3, 2, 1.0, None))]}


ZOKUZEN = {"a": zk_a, "b": zk_b, "c": zk_c, "d": zk_d}


def make_weights(raw: dict, seed: int, peak: float = 4.0, clear_choices: bool = False) -> Dict[str, torch.Tensor]:
    """`peak`: the standard deviation the scaled scores of an attention layer are brought to (through the query norm's weight
    where queries are normed, through the query projection otherwise): a few keys then carry most of the weight, while
    rounding to bfloat16 does not yet decide which.
    `clear_choices`: the routers' corrections are spread evenly over -0.4 .. 0.4 (in a drawn order) and their logits made
    small, so that no choice lies within rounding of turning: every position of a bfloat16 run can then be compared (the
    weights still follow the token through the scores)."""
    from infinilm_b200.config import config_from_json
    from infinilm_b200.weights import random_tensors
    w = random_tensors(config_from_json(raw), seed, "cpu")
    S = int(raw.get("streams", 1))
    g = torch.Generator().manual_seed(seed + 77)
    for name in list(w):
        x = w[name].float()
        layer = raw["layers"][int(name[1:name.index(".")])] if name.startswith("l") and "." in name and name[1].isdigit() else None
        typ = layer["type"] if layer else None
        m = layer["mixer"] if layer else None
        if name == "embed":
            x = x * 50.0
        elif name.endswith(".q.norm"):
            x = (1.0 + (x - 1.0)) * peak / (m["scale"] * 1.0 * m["dim"] ** 0.5)
        elif name.endswith(".k.norm"):
            x = x * 1.0
        elif typ == "latent_attention" and name.endswith(".mix.q"):
            x = x * peak / (m["scale"] * 0.02 * raw["width"] ** 0.5 * 0.08 * m["kv_rank"] ** 0.5 * m["dim"] ** 0.5) * 0.5
        elif typ == "attention" and name.endswith((".mix.q", ".mix.k", ".mix.v")):
            x = x * 2.0
        elif typ == "wkv" and name.endswith((".mix.r", ".mix.k", ".mix.v", ".mix.g")):
            x = x * 4.0
        elif name.endswith(".mix.w0"):
            x = x * 1.5 - 6.5                     # decays mostly near one (exp(-exp(-6.5)) = 0.9985): the state carries hundreds of tokens
        elif name.endswith(".mix.w1"):
            x = x * 10.0
        elif name.endswith(".mix.u"):
            x = x * 1.0
        elif ".mix.mu." in name:
            x = torch.rand(x.shape, generator=g)
        elif name.endswith(".correction"):
            x = x * 50.0                          # of the scores' own size (about 1 / outputs): it changes choices
            if clear_choices:
                x = torch.linspace(-0.4, 0.4, x.numel())[torch.randperm(x.numel(), generator=g)]
        elif name.endswith(".router"):
            x = x * (0.015 if clear_choices else 0.3)     # logits of size one: scores that move with the token but do not saturate
        elif name.endswith(".shared.sg"):
            x = x * 3.0
        elif name.endswith(".mix") and ".hc" in name:
            q, _ = torch.linalg.qr(torch.randn((S, S), generator=g))
            x = q * 0.9 + x * 0.1
        elif name.endswith((".hc1.in", ".hc2.in", ".hc1.out", ".hc2.out")):
            x = x * (1.0 if name.endswith("in") else 0.7)
        else:
            continue
        w[name] = x.to(torch.bfloat16)
    return w


def token_ids(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
