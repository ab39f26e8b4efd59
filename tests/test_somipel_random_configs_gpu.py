"""Somipel at sizes drawn from a seed: widths that are no multiple of 8, key and value sizes with and without a fast
attention kernel and unequal in either direction, one head or many, grouped or not, bias tables of 2 to 64 rows (odd counts
too) that end close by or far beyond the sequence, query temperatures that step at every token or never within the
sequence, or none, matrix memories of any head size with tight and loose caps, layers without a feed-forward, any order of
layers, layers that borrow an earlier layer's keys and values. Each configuration runs a prompt whole, in portions and
token by token against the plain implementation, in both dtypes, and two requests side by side."""
import random
import warnings

import pytest
import torch

import plain_somipel as P
from somipel_configs import _att, _att2, _mlstm, make_weights, token_ids

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    rng = random.Random(5000 + seed)
    width = rng.choice([40, 72, 100, 136, 200, 264])
    n_layers = rng.randint(1, 5)
    layers, owners = [], []
    for i in range(n_layers):
        ff = rng.choice([24, 56, 100]) if rng.random() < 0.8 else None
        r = rng.random()
        if r < 0.25:
            layers.append(_mlstm(rng.randint(1, 5), rng.choice([4, 8, 12, 20, 32, 64, 128]), rng.choice([4, 12, 32, 48, 72, 128]),
                                 rng.choice([1.0, 4.0, 15.0, 30.0]), ff))
        elif r < 0.5:
            kv = rng.randint(1, 3)
            temp = rng.choice([None, (round(rng.uniform(0.1, 1.2), 2), rng.choice([1, 3, 16, 50, 1000]))])
            layers.append(_att2(kv * rng.randint(1, 4), kv, rng.choice([4, 8, 12, 16, 24, 40, 64, 96, 128]), round(rng.uniform(0.05, 0.4), 3), temp, ff))
        elif owners and rng.random() < 0.45:
            src = rng.choice(owners)
            m = layers[src]["mixer"]
            rows = rng.choice([2, 3, 4, 7, 8, 16, 33, 64])
            layers.append(_att(m["kv_heads"] * rng.randint(1, 4), m["kv_heads"], m["dim"], m["vdim"], round(rng.uniform(0.05, 0.4), 3), rows,
                               rows // 2 + rng.choice([1, 2, 9, 40, 200, 5000]), ff, kv_from=src))
        else:
            kv = rng.randint(1, 3)
            rows = rng.choice([2, 3, 4, 7, 8, 16, 33, 64])
            layers.append(_att(kv * rng.randint(1, 4), kv, rng.choice([4, 8, 12, 16, 24, 40, 64, 96, 128]), rng.choice([4, 8, 20, 32, 64, 80, 128]),
                               round(rng.uniform(0.05, 0.4), 3), rows, rows // 2 + rng.choice([1, 2, 9, 40, 200, 5000]), ff))
            owners.append(i)
    return {"architecture": "Somipel", "vocab": rng.choice([50, 129, 333]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])},
            "residual_mult": rng.choice([0.2, 0.5, 1.0, 1.7]), "layers": layers}


def _err(got, ref):
    got, ref = got.double().cpu(), ref.double()
    got, ref = got - got.mean(dim=-1, keepdim=True), ref - ref.mean(dim=-1, keepdim=True)
    return (got - ref).pow(2).mean(dim=-1).sqrt() / ref.pow(2).mean(dim=-1).sqrt()


def one_kind(kind: str) -> dict:
    """Models of a single kind of layer: nothing but matrix memories (no pages at all), nothing but one kind of attention, and
    one layer whose keys and values every other layer borrows."""
    layers = {"mlstm": [_mlstm(2, 16, 24, 15.0, 40), _mlstm(3, 8, 8, 4.0, None)],
              "attention_2": [_att2(4, 2, 32, 0.2, (0.5, 4), 40), _att2(2, 2, 16, 0.3, None, None)],
              "attention": [_att(2, 1, 16, 32, 0.25, 8, 30, 40), _att(4, 4, 64, 64, 0.1, 16, 100, None)],
              "borrowers": [_att(2, 1, 32, 16, 0.2, 6, 50, 40), _att(3, 1, 32, 16, 0.3, 10, 12, None, kv_from=0),
                            _att(1, 1, 32, 16, 0.1, 4, 70, 24, kv_from=0), _att(4, 1, 32, 16, 0.2, 12, 7, 24, kv_from=0)]}[kind]
    return {"architecture": "Somipel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "layers": layers}


KINDS = ["mlstm", "attention_2", "attention", "borrowers"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", list(range(14)) + KINDS)
def test_random_configuration(cuda_device, seed, dtype):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine, StepEntry
    raw = random_config(seed) if isinstance(seed, int) else one_kind(seed)
    seed = seed if isinstance(seed, int) else 50 + KINDS.index(seed)
    w = make_weights(raw, seed, peak=3.0 if dtype == "float32" else 2.0)
    ids = token_ids(75, raw["vocab"], seed)
    other = token_ids(30, raw["vocab"], seed + 100)
    ref, ref_other = P.forward(raw, w, ids), P.forward(raw, w, other)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        eng = Engine.from_tensors(config_from_json(raw), w, dtype=dtype, page_size=16, num_pages=8, max_seqs=2, max_batch_tokens=128)
    tol = 2e-5 if dtype == "float32" else 5e-2

    def judge(got, want, what):
        err = _err(got, want)
        n_bad = int((err > tol).sum())
        assert torch.isfinite(got).all()
        assert n_bad <= (0 if dtype == "float32" else want.shape[0] // 15) and (dtype == "float32" or float(err.max()) <= 3 * tol), \
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
