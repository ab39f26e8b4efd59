"""Zokuzen on the CPU: configuration and its faults, run order and borrowed caches, tensor names and cache needs, the
random-weights folder, and the plain implementation's own identities (a recurrent state carried across a cut, the masks'
edges, one stream against the plain residual, the routing rule's invariants, the rotation's pairs)."""
import json
import math
import os

import pytest
import torch

import plain_zokuzen as P
from zokuzen_configs import ZOKUZEN, make_weights, token_ids

from infinilm_b200.config import ConfigError, config_from_json, describe_model
from infinilm_b200.models.causal_lm import CausalLM
from infinilm_b200.weights import FolderSource, check_against, write_model_folder


@pytest.mark.parametrize("name", sorted(ZOKUZEN))
def test_run_order_and_shared_caches(name):
    raw = ZOKUZEN[name]()
    spec = describe_model(config_from_json(raw))
    assert [s.layer for s in spec.order] == list(range(len(raw["layers"])))
    assert [s.cache_from for s in spec.order] == [L["mixer"].get("kv_from") for L in raw["layers"]]
    assert all(l.arrangement == "hyper_connections" and l.params["streams"] == raw["streams"] for l in spec.layers)


@pytest.mark.parametrize("name", sorted(ZOKUZEN))
def test_tensor_names_and_cache_needs(name):
    raw = ZOKUZEN[name]()
    model = CausalLM(describe_model(config_from_json(raw)), torch.float32)
    specs = {p.full_name(ws.name): ws for p, ws in model.weight_specs()}
    names = {k: v.shape for k, v in specs.items()}
    W, S = raw["width"], raw["streams"]
    assert names["embed"] == (raw["vocab"], W) and names["final.norm"] == (W,)
    assert specs["head"].fallback == "embed"                      # the head is the embedding table
    for i, L in enumerate(raw["layers"]):
        m, typ, f, px = L["mixer"], L["type"], L["mlp"], f"l{i}.mix"
        assert names[f"l{i}.norm1"] == (W,) and (f"l{i}.norm2" in names) == (f is not None)
        assert names[f"l{i}.hc1.in"] == (S,) and names[f"l{i}.hc1.out"] == (S,) and names[f"l{i}.hc1.mix"] == (S, S)
        assert (f"l{i}.hc2.mix" in names) == (f is not None)
        if f:
            r = f["router"]
            n_out = r["experts"] + r.get("identity", 0)
            assert names[f"l{i}.mlp.router"] == (n_out, W) and names[f"l{i}.mlp.correction"] == (n_out,)
            assert names[f"l{i}.mlp.e{r['experts'] - 1}.down"] == (W, f["expert"]["ff"]) and f"l{i}.mlp.e{r['experts']}.gate" not in names
            assert (f"l{i}.mlp.shared.sg" in names) == ("shared" in f)
            if "shared" in f:
                assert names[f"l{i}.mlp.shared.sg"] == (1, W) and names[f"l{i}.mlp.shared.up"] == (f["shared"]["ff"], W)
        if typ == "wkv":
            n = m["heads"] * m["dim"]
            assert all(names[f"{px}.{x}"] == (n, W) for x in "rkvg") and names[f"{px}.o"] == (W, n)
            assert names[f"{px}.w1"][1] == W and names[f"{px}.w2"][0] == n and names[f"{px}.w0"] == (n,)
            assert names[f"{px}.u"] == (m["heads"], m["dim"]) and names[f"{px}.mu.w"] == (W,) and names[f"{px}.norm"] == (n,)
        elif typ == "latent_attention":
            assert names[f"{px}.q"] == (m["heads"] * m["dim"], W) and names[f"{px}.dkv"] == (m["kv_rank"], W)
            assert names[f"{px}.uk"] == (m["heads"] * m["dim"], m["kv_rank"]) and names[f"{px}.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            assert names[f"{px}.dkv.norm"] == (m["kv_rank"],) and names[f"{px}.o"] == (W, m["heads"] * m["vdim"])
            assert all(f"{px}.{x}" not in names for x in ("dq", "uq", "sink", "g"))
        else:
            own = m.get("kv_from") is None
            assert names[f"{px}.q.norm"] == (m["heads"] * m["dim"],) and names[f"{px}.o"] == (W, m["heads"] * m["vdim"])
            assert all((f"{px}.{x}" in names) == own for x in ("k", "v", "k.norm"))
            if own:
                assert names[f"{px}.k.norm"] == (m["kv_heads"] * m["dim"],) and names[f"{px}.v"] == (m["kv_heads"] * m["vdim"], W)
    flat = []
    for n in model.cache_needs():
        flat += [] if n is None else list(n) if isinstance(n, (tuple, list)) else [n]
    kinds = []
    for L in raw["layers"]:
        if L["type"] == "wkv":
            kinds += ["state", "state"]
        elif L["mixer"].get("kv_from") is None:
            kinds.append("paged_kv")
    assert sorted(n.kind for n in flat) == sorted(kinds)
    assert all(n.dtype == "float32" for n in flat if n.kind == "state")
    # a window's pages are given back behind it; a layer that sees runs of positions keeps its pages (another may read them)
    wins = [n.window for n in flat if n.kind == "paged_kv"]
    want = [L["mixer"]["mask"]["size"] if L["type"] == "latent_attention" else None for L in raw["layers"]
            if L["type"] != "wkv" and L["mixer"].get("kv_from") is None]
    assert wins == want


def test_config_faults_name_the_key():
    raw = ZOKUZEN["a"]()
    raw["layers"][0]["type"] = "something_else"
    with pytest.raises(ConfigError, match="something_else"):
        config_from_json(raw)
    raw = ZOKUZEN["a"]()
    del raw["layers"][2]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        config_from_json(raw)
    raw = ZOKUZEN["a"]()
    raw["layers"][3]["mixer"]["kv_from"] = 2          # not an 'attention' layer
    with pytest.raises(ConfigError, match="kv_from"):
        config_from_json(raw)
    raw = ZOKUZEN["a"]()
    raw["layers"][3]["mixer"]["kv_heads"] = 4         # not laid out like the layer it reads
    with pytest.raises(ConfigError, match="kv_from"):
        config_from_json(raw)
    raw = ZOKUZEN["a"]()
    raw["layers"][1]["mixer"]["rot"]["dims"] = 7
    with pytest.raises(ConfigError, match="rot.dims"):
        config_from_json(raw)
    raw = ZOKUZEN["a"]()
    raw["layers"][0]["mlp"]["router"].pop("top")
    with pytest.raises(ConfigError, match="top"):
        config_from_json(raw)
    raw = ZOKUZEN["a"]()
    raw["streams"] = 0
    with pytest.raises(ConfigError, match="streams"):
        config_from_json(raw)
    raw = ZOKUZEN["a"]()
    raw["layers"][0]["mlp"]["router"]["top"] = 6      # more than the router has outputs
    with pytest.raises(ValueError, match="top"):
        CausalLM(describe_model(config_from_json(raw)), torch.float32)


def test_random_folder_round_trip(tmp_path):
    raw = ZOKUZEN["d"]()
    cfg = config_from_json(raw)
    folder = write_model_folder(cfg, 5, str(tmp_path / "m"))
    assert json.load(open(os.path.join(folder, "config.json"))) == raw
    model = CausalLM(describe_model(cfg), torch.bfloat16)
    src = FolderSource(folder)
    check_against(model, src)
    assert "head" not in src.names() and "embed" in src.names()
    src.close()


# ---- the plain implementation's own identities ----------------------------------------------------------------------
def test_masks_edges():
    w = P.visible(12, "window", 4)
    assert w[7].nonzero().flatten().tolist() == [4, 5, 6, 7] and w[2].nonzero().flatten().tolist() == [0, 1, 2]
    c = P.visible(12, "chunk", 5)
    assert c[7].nonzero().flatten().tolist() == [5, 6, 7] and c[5].nonzero().flatten().tolist() == [5] and c[4].nonzero().flatten().tolist() == [0, 1, 2, 3, 4]
    assert P.visible(6, "window", 1).nonzero().tolist() == [[i, i] for i in range(6)]


def test_rotation_pairs_and_angles():
    x = torch.zeros((3, 1, 8), dtype=torch.float64)
    x[:, 0, 1] = 1.0                                  # dimension 1 of 4 rotated ones pairs with dimension 3
    x[:, 0, 6] = 2.0                                  # beyond the rotated part: passes
    y = P.rotate_half(x, 4, 100.0)
    for p in range(3):
        a = p * 100.0 ** (-2.0 * 1 / 4)
        assert torch.allclose(y[p, 0], torch.tensor([0, math.cos(a), 0, math.sin(a), 0, 0, 2.0, 0], dtype=torch.float64))
    q = torch.randn((5, 2, 8), dtype=torch.float64)
    assert torch.allclose(P.rotate_half(q, 8, 50.0).norm(dim=-1), q.norm(dim=-1))


def test_recurrent_state_across_a_cut():
    raw = ZOKUZEN["a"]()
    w = {k: v.double() for k, v in make_weights(raw, 2).items()}
    p, m = P.sub(w, "l0.mix"), raw["layers"][0]["mixer"]
    h = torch.randn((40, raw["width"]), dtype=torch.float64)
    whole, _ = P.wkv_mixer(h, p, m, 1e-5)
    a, st = P.wkv_mixer(h[:13], p, m, 1e-5)
    b, st = P.wkv_mixer(h[13:14], p, m, 1e-5, state=st)
    c, _ = P.wkv_mixer(h[14:], p, m, 1e-5, state=st)
    assert torch.allclose(torch.cat([a, b, c]), whole, rtol=1e-10, atol=1e-12)


def test_recurrence_against_its_closed_form():
    T, H, d = 6, 2, 3
    r, k, v = (torch.randn((T, H, d), dtype=torch.float64) for _ in range(3))
    dec = torch.rand((T, H, d), dtype=torch.float64)
    u = torch.randn((H, d), dtype=torch.float64)
    o, _ = P.wkv_recurrence(r, k, v, dec, u)
    for t in range(T):
        want = torch.einsum("hd,hd,he->he", r[t] * u, k[t], v[t])
        for j in range(t):
            decay = torch.ones((H, d), dtype=torch.float64)
            for i in range(j + 1, t):
                decay = decay * dec[i]
            want = want + torch.einsum("hd,hd,he->he", r[t] * decay, k[j], v[j])
        assert torch.allclose(o[t], want)


def test_one_stream_is_the_plain_residual():
    xs = torch.randn((1, 5, 8), dtype=torch.float64)
    y = torch.randn((5, 8), dtype=torch.float64)
    one = torch.ones(1, dtype=torch.float64)
    assert torch.equal(P.streams_read(xs, one), xs[0])
    assert torch.allclose(P.streams_write(xs, y, torch.ones((1, 1), dtype=torch.float64), one)[0], xs[0] + y)
    # the mix matrix is indexed [from, to]
    xs = torch.randn((2, 1, 3), dtype=torch.float64)
    mix = torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=torch.float64)      # copy 0 goes to copy 1, nothing else
    out = P.streams_write(xs, torch.zeros((1, 3), dtype=torch.float64), mix, torch.zeros(2, dtype=torch.float64))
    assert torch.equal(out[1], xs[0]) and torch.equal(out[0], torch.zeros_like(out[0]))


def test_routing_rule():
    g = torch.Generator().manual_seed(0)
    h = torch.randn((50, 16), generator=g, dtype=torch.float64)
    wr = torch.randn((6, 16), generator=g, dtype=torch.float64)
    idx0, wt0 = P.route(h, wr, torch.zeros(6, dtype=torch.float64), 3, 2.0)
    assert torch.allclose(wt0.sum(-1), torch.full((50,), 2.0, dtype=torch.float64))      # normalised, then scaled
    corr = torch.tensor([0, 0, 0, 0, 0, 10.0], dtype=torch.float64)                    # the correction steers the choice ...
    idx1, wt1 = P.route(h, wr, corr, 3, 2.0)
    assert (idx1[:, 0] == 5).all()
    s = torch.softmax(h @ wr.T, -1)
    assert torch.allclose(wt1 / 2.0, torch.gather(s, 1, idx1) / torch.gather(s, 1, idx1).sum(-1, keepdim=True))    # ... not the weights
    # an identity unit returns its input: with every weight on it the feed-forward is scale * h
    f = {"router": {"experts": 1, "identity": 1, "top": 1, "scale": 1.5}}
    p = {"router": torch.zeros((2, 16), dtype=torch.float64), "correction": torch.tensor([0.0, 1.0], dtype=torch.float64),
         "e0.gate": torch.randn((4, 16), dtype=torch.float64), "e0.up": torch.randn((4, 16), dtype=torch.float64),
         "e0.down": torch.randn((16, 4), dtype=torch.float64)}
    assert torch.allclose(P.routed_feed_forward(h, p, f), 1.5 * h)
