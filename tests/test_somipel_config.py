"""Somipel on the CPU: configuration, run order, tensor names and cache needs, the random-weights folder, and the plain
implementation's own identities (the stabilised matrix memory against its unstabilised closed form, a state carried across a
cut, the bias table's buckets at their edges, the sink's limits, the query temperature's steps)."""
import json
import math
import os

import pytest
import torch

import plain_somipel as P
from somipel_configs import SOMIPEL, make_weights, token_ids

from infinilm_b200.config import ConfigError, config_from_json, describe_model
from infinilm_b200.models.causal_lm import CausalLM
from infinilm_b200.weights import FolderSource, check_against, write_model_folder


@pytest.mark.parametrize("name", sorted(SOMIPEL))
def test_run_order_and_shared_caches(name):
    raw = SOMIPEL[name]()
    spec = describe_model(config_from_json(raw))
    assert [s.layer for s in spec.order] == list(range(len(raw["layers"])))
    assert [s.cache_from for s in spec.order] == [L["mixer"].get("kv_from") for L in raw["layers"]]
    assert all(l.arrangement == "branch_norm_residual" for l in spec.layers) if hasattr(spec.layers[0], "arrangement") else True


@pytest.mark.parametrize("name", sorted(SOMIPEL))
def test_tensor_names_and_cache_needs(name):
    raw = SOMIPEL[name]()
    model = CausalLM(describe_model(config_from_json(raw)), torch.float32)
    names = {p.full_name(ws.name): ws.shape for p, ws in model.weight_specs()}
    W = raw["width"]
    assert names["embed"] == (raw["vocab"], W) and names["head"] == (raw["vocab"], W) and names["final.norm"] == (W,)
    for i, L in enumerate(raw["layers"]):
        m, typ, px = L["mixer"], L["type"], f"l{i}.mix"
        assert names[f"l{i}.norm1"] == (W,) and (f"l{i}.norm2" in names) == (L["mlp"] is not None)
        if L["mlp"]:
            assert names[f"l{i}.mlp.gate"] == (L["mlp"]["ff"], W) and names[f"l{i}.mlp.down"] == (W, L["mlp"]["ff"])
        assert names[f"{px}.q"] == (m["heads"] * m["dim"], W) and names[f"{px}.o"] == (W, m["heads"] * m["vdim"])
        if typ == "mlstm":
            assert names[f"{px}.i"] == (m["heads"], W) and names[f"{px}.f.b"] == (m["heads"],)
            assert names[f"{px}.norm"] == (m["heads"] * m["vdim"],) and names[f"{px}.g"] == (m["heads"] * m["vdim"], W)
            continue
        assert names[f"{px}.q.norm"] == (m["dim"],)
        own = m.get("kv_from") is None
        assert (f"{px}.k" in names) == own and (f"{px}.k.norm" in names) == own
        if typ == "attention":
            assert names[f"{px}.rel"] == (m["bias_rows"], m["heads"]) and names[f"{px}.g"] == (m["heads"] * m["vdim"], W)
            assert names[f"{px}.q.b"] == (m["heads"] * m["dim"],)
            assert (f"{px}.v" in names) == own and (f"{px}.v.b" in names) == own
        else:
            assert all(f"{px}.{n}" not in names for n in ("v", "g", "rel", "q.b", "k.b"))
    # a cache per layer that has keys of its own, the matrix memory's state and running maximum, none for a layer that borrows
    needs = model.cache_needs()
    flat = []
    for n in needs:
        flat += [] if n is None else list(n) if isinstance(n, (tuple, list)) else [n]
    kinds = []
    for L in raw["layers"]:
        if L["type"] == "mlstm":
            kinds += ["state", "state"]
        elif L["mixer"].get("kv_from") is None:
            kinds.append("paged_kv")
    assert sorted(n.kind for n in flat) == sorted(kinds)
    assert all(n.dtype == "float32" for n in flat if n.kind == "state")


def test_config_faults_name_the_key():
    raw = SOMIPEL["a"]()
    raw["layers"][0]["type"] = "something_else"
    with pytest.raises(ConfigError, match="something_else"):
        config_from_json(raw)
    raw = SOMIPEL["a"]()
    del raw["layers"][1]["mixer"]["bias_max"]
    with pytest.raises(ConfigError, match="bias_max"):
        config_from_json(raw)
    raw = SOMIPEL["a"]()
    raw["layers"][3]["mixer"]["kv_from"] = 2          # not an 'attention' layer
    with pytest.raises(ConfigError, match="kv_from"):
        config_from_json(raw)
    raw = SOMIPEL["a"]()
    raw["layers"][3]["mixer"]["kv_from"] = 3          # itself
    with pytest.raises(ConfigError, match="kv_from"):
        config_from_json(raw)
    raw = SOMIPEL["c"]()
    raw["layers"][1]["mixer"]["kv_from"] = 3          # a later layer
    with pytest.raises(ConfigError, match="kv_from"):
        config_from_json(raw)
    raw = SOMIPEL["b"]()
    raw["layers"][0]["mlp"] = {"kind": "sparse", "ff": 8}
    with pytest.raises(ConfigError, match="sparse"):
        config_from_json(raw)


def test_random_folder_round_trip(tmp_path):
    raw = SOMIPEL["a"]()
    cfg = config_from_json(raw)
    d = write_model_folder(cfg, 3, str(tmp_path / "m"))
    assert json.load(open(os.path.join(d, "config.json"))) == raw
    model = CausalLM(describe_model(cfg), torch.bfloat16)
    src = FolderSource(d)
    check_against(model, src)
    assert "l3.mix.k" not in src.names() and "l3.mix.rel" in src.names() and "l2.mix.v" not in src.names()
    src.close()


def test_bias_buckets_of_the_package_equal_the_plain_ones_at_every_edge():
    from infinilm_b200.parts.normed_attention import distance_buckets
    for rows, far in ((12, 40), (8, 20), (32, 128), (4, 5), (6, 300), (10, 17), (4, 3), (5, 9), (64, 4096)):
        got = distance_buckets(rows, far)
        assert got == [P.distance_bucket(n, rows, far) for n in range(far + 1)]
        half = rows // 2
        assert got[:half] == list(range(half)) and got[half] == half and got[far] == rows - 1
        assert all(b <= a for b, a in zip(got, got[1:])) and max(got) == rows - 1
        assert P.distance_bucket(far * 7, rows, far) == rows - 1
    with pytest.raises(ValueError):
        distance_buckets(8, 4)                        # the last row is never reached on a logarithmic scale that ends at rows/2


def test_query_temperature_steps():
    t = P.query_temperature(20, 0.5, 4, torch.float64)
    assert float(t[0]) == 1.0 and float(t[2]) == 1.0                     # positions 0..2: floor((p + 1) / 4) = 0
    assert abs(float(t[3]) - (1 + 0.5 * math.log(2))) < 1e-12            # position 3 is the first of the next step
    assert abs(float(t[10]) - (1 + 0.5 * math.log(3))) < 1e-12 and abs(float(t[11]) - (1 + 0.5 * math.log(4))) < 1e-12
    t1 = P.query_temperature(5, 1.0, 1, torch.float64)
    assert torch.allclose(t1, 1 + torch.log(torch.arange(2, 7, dtype=torch.float64)))


def test_sink_and_bias_in_the_plain_attention():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(6, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    plain = P.causal_attention(q, k, v, 0.5)
    mask = torch.ones(6, 6, dtype=torch.bool).triu(1)
    for h in range(2):
        s = (q[:, h] @ k[:, h].T * 0.5).masked_fill(mask, float("-inf"))
        assert torch.allclose(plain[:, h], torch.softmax(s, 1) @ v[:, h])
    # the sink: one more term exp(0) in the denominator; the first token's weight on itself is e^s / (1 + e^s)
    sunk = P.causal_attention(q, k, v, 0.5, sink_zero=True)
    s00 = float(q[0, 0] @ k[0, 0]) * 0.5
    assert torch.allclose(sunk[0, 0], v[0, 0] * (math.exp(s00) / (1 + math.exp(s00))))
    assert (sunk.norm(dim=-1) < plain.norm(dim=-1) + 1e-12).all()
    # a bias of minus infinity at distance 1 and beyond leaves every token its own value
    bias = torch.full((2, 6, 6), -1e9, dtype=torch.float64)
    bias[:, torch.arange(6), torch.arange(6)] = 0.0
    assert torch.allclose(P.causal_attention(q, k, v, 0.5, bias=bias), v)
    # grouped heads: 4 query heads on 2 key heads use heads 0, 0, 1, 1
    q4 = torch.randn(6, 4, 4, generator=g, dtype=torch.float64)
    o = P.causal_attention(q4, k, v, 0.3)
    assert torch.allclose(o[:, 1], P.causal_attention(q4[:, 1:2], k[:, :1], v[:, :1], 0.3)[:, 0])
    assert torch.allclose(o[:, 2], P.causal_attention(q4[:, 2:3], k[:, 1:], v[:, 1:], 0.3)[:, 0])


def test_matrix_memory_equals_its_unstabilised_form_and_carries_its_state():
    g = torch.Generator().manual_seed(1)
    T, H, d, dv = 11, 2, 3, 4
    q, k = (torch.randn(T, H, d, generator=g, dtype=torch.float64) for _ in range(2))
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    i_log = torch.randn(T, H, generator=g, dtype=torch.float64) * 2
    f_log = torch.nn.functional.logsigmoid(torch.randn(T, H, generator=g, dtype=torch.float64) * 2 + 1)
    o, state = P.matrix_memory(q, k, v, i_log, f_log)
    # unstabilised: C_t = e^f C + e^i k v^T, n_t likewise; the running maximum m_t = max(f + m, i) from m_0 = 0 only rescales,
    # except in the floor of the denominator: max(|n.q|, 1) in unstabilised units
    C, n, m = torch.zeros(H, d, dv, dtype=torch.float64), torch.zeros(H, d, dtype=torch.float64), torch.zeros(H, dtype=torch.float64)
    for t in range(T):
        C = torch.exp(f_log[t])[:, None, None] * C + torch.exp(i_log[t])[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = torch.exp(f_log[t])[:, None] * n + torch.exp(i_log[t])[:, None] * k[t]
        m = torch.maximum(f_log[t] + m, i_log[t])
        num = torch.einsum("hdv,hd->hv", C, q[t]) * torch.exp(-m)[:, None]
        den = torch.maximum(((n * q[t]).sum(-1) * torch.exp(-m)).abs(), torch.exp(-m)) + P.DENOM_EPS
        assert torch.allclose(o[t], num / den[:, None], atol=1e-12)
    for cut in (1, 2, 5, 10):
        o1, st = P.matrix_memory(q[:cut], k[:cut], v[:cut], i_log[:cut], f_log[:cut])
        o2, st2 = P.matrix_memory(q[cut:], k[cut:], v[cut:], i_log[cut:], f_log[cut:], st)
        assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-13)
        assert all(torch.allclose(a, b, atol=1e-13) for a, b in zip(st2, state))
    # the running maximum starts at 0, not at minus infinity: a first token with a very negative input gate keeps m = f < 0 ... 0
    o0, (S0, n0, m0) = P.matrix_memory(q[:1], k[:1], v[:1], torch.full((1, H), -9.0, dtype=torch.float64), f_log[:1])
    assert torch.allclose(m0, f_log[0]) and torch.allclose(S0, math.exp(-9.0) * torch.exp(-f_log[0])[:, None, None] * k[0][:, :, None] * v[0][:, None, :])


def test_capped_gates_stay_inside_the_cap():
    z = torch.tensor([-1e3, -3.0, 0.0, 3.0, 1e3], dtype=torch.float64)
    c = P.capped(z, 2.0)
    assert float(c.abs().max()) <= 2.0 and abs(float(c[2])) == 0.0 and torch.allclose(c[3], 2.0 * torch.tanh(torch.tensor(1.5, dtype=torch.float64)))


def test_a_layer_adds_the_normed_branch():
    """Scaling a sublayer's output weights changes nothing (its norm takes the scale off again), while the residual factor
    scales what is added."""
    raw = SOMIPEL["d"]()
    raw["norm"]["eps"] = 1e-30                        # (the eps under the root is what a scale would otherwise still move)
    w = make_weights(raw, 2)
    ids = token_ids(9, raw["vocab"], 1)
    a = P.forward(raw, w, ids)
    w2 = dict(w)
    w2["l0.mix.o"] = (w["l0.mix.o"].float() * 4.0).to(torch.bfloat16)        # (a power of two: exact in bfloat16)
    w2["l1.mlp.down"] = (w["l1.mlp.down"].float() * 0.5).to(torch.bfloat16)
    assert torch.allclose(P.forward(raw, w2, ids), a, rtol=1e-6, atol=1e-6 * float(a.abs().max()))
    raw0 = dict(raw, residual_mult=0.0)
    x = w["embed"].double()[torch.tensor(ids)]
    assert torch.allclose(P.forward(raw0, w, ids), P.rms_norm(x, w["final.norm"].double(), raw["norm"]["eps"]) @ w["head"].double().T)


def test_plain_forward_runs_every_configuration():
    for name in sorted(SOMIPEL):
        raw = SOMIPEL[name]()
        lg, streams = P.forward(raw, make_weights(raw, 5), token_ids(12, raw["vocab"], 1), want_layers=True)
        assert lg.shape == (12, raw["vocab"]) and torch.isfinite(lg).all()
        assert streams.shape == (len(raw["layers"]), 12, raw["width"])
