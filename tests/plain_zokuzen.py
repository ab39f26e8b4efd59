"""A plain, slow implementation of the Zokuzen design on whole sequences, one function per mechanism, written from the
design's equations in float64 (or any dtype given). It shares no code with the package: tensors in, tensors out, loops
over time where the design has a recurrence.

Notation: T tokens, W width, S residual streams; a linear weight is [out, in] and applied as x @ w.T; positions count
from 0. A layer keeps S copies of the residual stream; a sublayer reads a weighted sum of them, and its output goes back
into every copy while the copies are mixed among themselves.
"""
import math

import torch


def rms_norm(x, w, eps, one_plus=False):
    """y = x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight; one_plus: the weight is 1 + w)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * (1.0 + w) if one_plus else y * w


def silu(z):
    return z * torch.sigmoid(z)


def gated_unit(x, w_gate, w_up, w_down):
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


# ---- residual streams -------------------------------------------------------------------------------------------------
def streams_read(xs, w_in):
    """xs [S, T, W], w_in [S] -> the sublayer's input sum_s w_in[s] xs[s]."""
    return torch.einsum("s,stw->tw", w_in, xs)


def streams_write(xs, y, w_mix, w_out):
    """new[t] = sum_s w_mix[s, t] xs[s] + w_out[t] y, every new copy from the old ones."""
    return torch.einsum("sr,stw->rtw", w_mix, xs) + w_out[:, None, None] * y[None]


# ---- attention --------------------------------------------------------------------------------------------------------
def visible(T, kind, size):
    """[T, T] bool: may position i (row) see position j (column)? kind "window": 0 <= i - j < size; "chunk": j <= i and
    both in the same run of `size` positions counted from 0; None: j <= i."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if kind == "window":
        ok = ok & (i - j < size)
    elif kind == "chunk":
        ok = ok & (i // size == j // size)
    return ok


def softmax_attention(q, k, v, scale, mask):
    """q [T, H, d], k [T, G, d], v [T, G, e]; query head h uses kv head h // (H // G). mask [T, T] bool. -> [T, H, e]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.stack(out, dim=1)


def rotate_half(x, dims, base):
    """x [T, heads, d]: of each head's first `dims` dimensions, dimension i pairs with i + dims/2; the pair turns by the angle
    position * base^(-2 i / dims). The other dimensions pass."""
    T = x.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def chunked_attention(h, p, m, eps, kv=None):
    """Grouped-query attention whose queries and keys are normed over the whole projection (all heads at once), rotated on
    part of each head, and which sees only its own run of m["mask"]["size"] positions. kv: (k, v) of another layer, as that
    layer used them (normed, rotated) - then this layer has no k, v tensors. Returns (y, (k, v))."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    q = rms_norm(h @ p["q"].T, p["q.norm"], eps).view(T, H, d)
    if rot:
        q = rotate_half(q, rot["dims"], rot["base"])
    if kv is None:
        k = rms_norm(h @ p["k"].T, p["k.norm"], eps).view(T, G, d)
        if rot:
            k = rotate_half(k, rot["dims"], rot["base"])
        v = (h @ p["v"].T).view(T, G, e)
    else:
        k, v = kv
    o = softmax_attention(q, k, v, m["scale"], visible(T, "chunk", m["mask"]["size"]))
    return o.reshape(T, H * e) @ p["o"].T, (k, v)


def latent_window_attention(h, p, m, eps):
    """Keys and values of every head are up-projections of one normed latent per token; no positions; a sliding window."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T).view(T, H, d)
    c = rms_norm(h @ p["dkv"].T, p["dkv.norm"], eps)
    k = (c @ p["uk"].T).view(T, H, d)
    v = (c @ p["uv"].T).view(T, H, e)
    o = softmax_attention(q, k, v, m["scale"], visible(T, "window", m["mask"]["size"]))
    return o.reshape(T, H * e) @ p["o"].T


# ---- the recurrent mixer ----------------------------------------------------------------------------------------------
def wkv_recurrence(r, k, v, w, u, S=None):
    """r, k, w [T, H, d], v [T, H, e], u [H, d], S [H, d, e] (None: zeros).
    o_t = (S + diag(u) k_t v_t^T)^T r_t;  then S = diag(w_t) S + k_t v_t^T. Returns (o [T, H, e], S)."""
    T, H, d = k.shape
    e = v.shape[-1]
    S = torch.zeros((H, d, e), dtype=k.dtype) if S is None else S.clone()
    out = []
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hde,hd->he", S + u[:, :, None] * kv, r[t]))
        S = w[t][:, :, None] * S + kv
    return torch.stack(out), S


def wkv_mixer(h, p, m, eps, state=None):
    """Each projection reads its own blend of a token's input and its predecessor's, h + (h_prev - h) * mu; the decay per
    head and key channel is exp(-exp(w0 + W2 tanh(W1 blend))). state: (h of the last token before, S) or None."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    prev0 = torch.zeros((1, W), dtype=h.dtype) if state is None else state[0][None]
    prev = torch.cat([prev0, h[:-1]], dim=0)

    def blend(name):
        return h + (prev - h) * p["mu." + name]
    r = (blend("r") @ p["r"].T).view(T, H, d)
    k = (blend("k") @ p["k"].T).view(T, H, d)
    v = (blend("v") @ p["v"].T).view(T, H, d)
    gate = silu(blend("g") @ p["g"].T)
    w = torch.exp(-torch.exp(torch.tanh(blend("w") @ p["w1"].T) @ p["w2"].T + p["w0"])).view(T, H, d)
    o, S = wkv_recurrence(r, k, v, w, p["u"], None if state is None else state[1])
    o = rms_norm(o, None, eps).reshape(T, H * d) * p["norm"] * gate
    return o @ p["o"].T, (h[-1], S)


# ---- the routed feed-forward --------------------------------------------------------------------------------------------
def route(h, w_router, correction, top, scale, margins=None):
    """Scores are the softmax of the router's logits over all its outputs; the `top` largest of score + correction are
    chosen (the lower index wins a tie); the weights are the chosen scores themselves over their sum (+ 1e-20), times scale.
    Returns (idx [T, top], weights [T, top]). margins (a list, or None) receives per token the gap between the last chosen and
    the first rejected choice score (infinite where every output is chosen): how far rounding is from turning the choice."""
    s = torch.softmax(h @ w_router.T, dim=-1)
    c = s + correction
    full = torch.sort(c, dim=-1, descending=True, stable=True)
    order = full.indices[:, :top]
    if margins is not None:
        v = full.values
        margins.append(v[:, top - 1] - v[:, top] if top < v.shape[1] else torch.full((h.shape[0],), math.inf, dtype=h.dtype))
    chosen = torch.gather(s, 1, order)
    return order, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * scale


def routed_feed_forward(h, p, f, margins=None):
    """f: the layer's "mlp" object. The last router.identity outputs of the router stand for units that return their input."""
    r = f["router"]
    n, n_id, top = r["experts"], r.get("identity", 0), r["top"]
    idx, wt = route(h, p["router"], p["correction"], top, r.get("scale", 1.0), margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            y = h[t] if e >= n else gated_unit(h[t][None], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
            out[t] += wt[t, j] * y
    assert p["router"].shape[0] == n + n_id
    if f.get("shared") is not None:
        out = out + torch.sigmoid(h @ p["shared.sg"].T) * gated_unit(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    return out


# ---- the model ------------------------------------------------------------------------------------------------------------
def sub(tensors, prefix):
    return {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}


def forward(cfg, tensors, tokens, dtype=torch.float64, want_layers=False, margins=None):
    """cfg: the parsed config.json; tensors: name -> tensor. Returns logits [T, vocab] (and the sum of the residual streams
    after every layer, [layers, T, W]). margins: a list that receives every router's choice margins (see `route`)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, S = cfg["norm"]["eps"], int(cfg.get("streams", 1))
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    xs = torch.stack([x] * S)
    kept, sums = {}, []
    for i, L in enumerate(cfg["layers"]):
        p, m = sub(w, f"l{i}.mix"), L["mixer"]
        hc1, hc2 = sub(w, f"l{i}.hc1"), sub(w, f"l{i}.hc2")
        h = rms_norm(streams_read(xs, hc1["in"]), w[f"l{i}.norm1"], eps, one_plus=True)
        if L["type"] == "attention":
            src = m.get("kv_from")
            y, kept[i] = chunked_attention(h, p, m, eps, kv=None if src is None else kept[src])
        elif L["type"] == "latent_attention":
            y = latent_window_attention(h, p, m, eps)
        elif L["type"] == "wkv":
            y, _ = wkv_mixer(h, p, m, eps)
        else:
            raise ValueError(L["type"])
        xs = streams_write(xs, y, hc1["mix"], hc1["out"])
        if L.get("mlp") is not None:
            h = rms_norm(streams_read(xs, hc2["in"]), w[f"l{i}.norm2"], eps, one_plus=True)
            xs = streams_write(xs, routed_feed_forward(h, sub(w, f"l{i}.mlp"), L["mlp"], margins), hc2["mix"], hc2["out"])
        sums.append(xs.sum(0))
    logits = rms_norm(xs.sum(0), w["final.norm"], eps, one_plus=True) @ w["embed"].T
    return (logits, torch.stack(sums)) if want_layers else logits


def greedy_generate(cfg, tensors, prompt, n, dtype=torch.float64):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(forward(cfg, tensors, ids, dtype)[-1])))
    return ids[len(prompt):]
