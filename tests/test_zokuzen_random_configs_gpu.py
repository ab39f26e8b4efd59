"""Zokuzen at sizes drawn from a seed: one to five streams, widths that are no multiple of 16, key and value sizes with and
without a fast attention kernel and unequal in either direction, grouped heads or not, rotation of none, part or all of a
head, runs of positions and windows from 1 position to beyond the sequence, latents of any width, recurrences of any head
size, routers with and without identity units, corrections, shared units, every output chosen or one, layers without a
feed-forward, any order of layers, layers that borrow an earlier layer's keys and values with a mask of their own. Each
configuration runs a prompt whole, in portions and token by token against the plain implementation, in both dtypes, and two
requests side by side."""
import random
import warnings

import pytest
import torch

import plain_zokuzen as P
from zokuzen_configs import _att, _lat, _moe, _wkv, make_weights, token_ids

pytestmark = pytest.mark.gpu


def _random_moe(rng):
    if rng.random() < 0.2:
        return None
    experts, identity = rng.randint(1, 9), rng.choice([0, 0, 1, 2, 3])
    top = rng.randint(1, min(experts + identity, 4)) if rng.random() < 0.8 else experts + identity
    return _moe(rng.choice([8, 24, 40, 72]), experts, top, identity, rng.choice([0.5, 1.0, 2.0, 2.5]), rng.choice([None, 16, 40, 96]))


def random_config(seed: int) -> dict:
    rng = random.Random(7000 + seed)
    width = rng.choice([40, 72, 96, 100, 136, 200, 256])
    layers, owners = [], []
    for i in range(rng.randint(1, 5)):
        mlp, r = _random_moe(rng), rng.random()
        if r < 0.3:
            layers.append(_wkv(rng.randint(1, 5), rng.choice([4, 8, 12, 20, 32, 64, 128]), mlp))
        elif r < 0.55:
            layers.append(_lat(rng.randint(1, 6), rng.choice([4, 8, 16, 24, 64]), rng.choice([4, 12, 32, 80]), rng.choice([8, 16, 24, 48, 80, 128, 272]),
                               round(rng.uniform(0.05, 0.4), 3), rng.choice([1, 2, 15, 16, 17, 40, 90, 1000]), mlp))
        else:
            chunk = rng.choice([1, 3, 16, 17, 32, 50, 210, 1000])
            if owners and rng.random() < 0.45:
                src = rng.choice(owners)
                m = layers[src]["mixer"]
                rot = (m["rot"]["dims"], m["rot"]["base"]) if "rot" in m else None
                layers.append(_att(m["kv_heads"] * rng.randint(1, 4), m["kv_heads"], m["dim"], m["vdim"], round(rng.uniform(0.05, 0.4), 3), chunk, rot, mlp,
                                   kv_from=src))
            else:
                kv, dim = rng.randint(1, 3), rng.choice([4, 8, 12, 16, 24, 40, 64, 96, 128])
                rot = rng.choice([None, (dim, 10000.0), (2 * rng.randint(1, dim // 2), rng.choice([50.0, 1e6]))])
                layers.append(_att(kv * rng.randint(1, 4), kv, dim, rng.choice([4, 8, 20, 32, 64, 80, 128]), round(rng.uniform(0.05, 0.4), 3), chunk, rot, mlp))
                owners.append(i)
    return {"architecture": "Zokuzen", "vocab": rng.choice([50, 129, 333]), "width": width, "streams": rng.randint(1, 5),
            "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "layers": layers}


def one_kind(kind: str) -> dict:
    """Models of a single kind of layer: nothing but recurrences (no pages at all), nothing but latents, nothing but attention,
    and one layer whose keys and values every other layer borrows."""
    f = _moe(24, 3, 2, 1, 1.5, 16)
    layers = {"wkv": [_wkv(2, 16, f), _wkv(3, 8, None)],
              "latent": [_lat(4, 16, 8, 32, 0.2, 10, f), _lat(2, 8, 8, 16, 0.3, 100, None)],
              "attention": [_att(2, 1, 16, 32, 0.25, 8, (8, 100.0), f), _att(4, 4, 64, 64, 0.1, 30, None, None)],
              "borrowers": [_att(2, 1, 32, 16, 0.2, 50, (16, 1e4), f), _att(3, 1, 32, 16, 0.3, 12, (16, 1e4), None, kv_from=0),
                            _att(1, 1, 32, 16, 0.1, 70, (16, 1e4), f, kv_from=0), _att(4, 1, 32, 16, 0.2, 7, (16, 1e4), f, kv_from=0)]}[kind]
    return {"architecture": "Zokuzen", "vocab": 97, "width": 64, "streams": 2, "norm": {"eps": 1e-5}, "layers": layers}


KINDS = ["wkv", "latent", "attention", "borrowers"]


def _plain(raw, w, ids):
    margins = []
    lg = P.forward(raw, w, ids, margins=margins)
    m = torch.stack(margins).amin(0) if margins else torch.full((len(ids),), float("inf"), dtype=torch.float64)
    return lg, torch.cummin(m, 0).values


def _err(got, ref):
    got, ref = got.double().cpu(), ref.double()
    got, ref = got - got.mean(dim=-1, keepdim=True), ref - ref.mean(dim=-1, keepdim=True)
    return (got - ref).pow(2).mean(dim=-1).sqrt() / ref.pow(2).mean(dim=-1).sqrt()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(16)) + KINDS)
def test_random_configuration(cuda_device, seed, dtype):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine, StepEntry
    raw = random_config(seed) if isinstance(seed, int) else one_kind(seed)
    seed = seed if isinstance(seed, int) else 50 + KINDS.index(seed)
    # (bfloat16: routing choices that rounding cannot turn, so that every position is compared)
    w = make_weights(raw, seed, peak=3.0 if dtype == "float32" else 2.0, clear_choices=dtype == "bfloat16")
    ids = token_ids(75, raw["vocab"], seed)
    other = token_ids(30, raw["vocab"], seed + 100)
    ref, ref_other = _plain(raw, w, ids), _plain(raw, w, other)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        eng = Engine.from_tensors(config_from_json(raw), w, dtype=dtype, page_size=16, num_pages=8, max_seqs=2, max_batch_tokens=128)
    tol = 3e-5 if dtype == "float32" else 5e-2
    margin = 1e-6 if dtype == "float32" else 2e-2

    def judge(got, want, what):
        keep = want[1] > margin                   # positions before which no routing choice was within rounding of turning
        assert float(keep.float().mean()) > (0.5 if dtype == "float32" else 0.99), "the test's weights leave too few clear choices"
        err = torch.where(keep, _err(got, want[0]), torch.zeros(len(keep), dtype=torch.float64))
        n_bad = int((err > tol).sum())
        assert torch.isfinite(got).all()
        assert n_bad <= (0 if dtype == "float32" else int(keep.sum()) // 15) and (dtype == "float32" or float(err.max()) <= 3 * tol), \
            f"seed {seed} {what}: {n_bad} positions over {tol:.0e}, worst {float(err.max()):.2e}; config {raw}"

    for cuts in ([75], [33, 2, 17, 1, 1, 21], [16] + [1] * 59):
        seq, outs, a = eng.open(str(cuts[0])), [], 0
        for c in cuts:
            outs.append(eng.step([StepEntry(seq, ids[a:a + c], list(range(c)))]).clone())
            a += c
        eng.close(seq)
        judge(torch.cat(outs, 0), ref, f"cuts {cuts[:3]}")
    # two requests side by side: a portion beside single tokens, then the other way round
    s1, s2 = eng.open("x"), eng.open("y")
    o1, o2 = [], []
    lg = eng.step([StepEntry(s1, ids[:40], list(range(40))), StepEntry(s2, other[:1], [0])]).clone()
    o1.append(lg[:40]), o2.append(lg[40:])
    for t in range(1, 6):
        lg = eng.step([StepEntry(s1, ids[39 + t:40 + t], [0]), StepEntry(s2, other[t:t + 1], [0])]).clone()
        o1.append(lg[:1]), o2.append(lg[1:])
    lg = eng.step([StepEntry(s1, ids[45:46], [0]), StepEntry(s2, other[6:30], list(range(24)))]).clone()
    o1.append(lg[:1]), o2.append(lg[1:])
    lg = eng.step([StepEntry(s1, ids[46:75], list(range(29)))]).clone()
    o1.append(lg)
    eng.close(s1), eng.close(s2)
    judge(torch.cat(o1, 0), ref, "side by side, first")
    judge(torch.cat(o2, 0), ref_other, "side by side, second")
    eng.synchronize()
    eng.cache.check_invariants()
