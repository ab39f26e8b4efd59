"""A plain, slow implementation of the Somipel design on whole sequences, one function per mechanism, written from the
design's equations in float64 (or any dtype given). It shares no code with the package: tensors in, tensors out, loops
over time where the design has a recurrence.

Notation: T tokens, W width; a linear weight is [out, in] and applied as x @ w.T; positions count from 0.
A layer adds its sublayers' NORMED outputs: x += m * norm1(mixer(x)); x += m * norm2(ff(x)); the sublayers read x itself.
"""
import math

import torch

DENOM_EPS = 1e-6          # added to the matrix memory's denominator


def rms_norm(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w over the last axis (w may be None)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z * torch.sigmoid(z)


def gated_ff(x, w_gate, w_up, w_down):
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def distance_bucket(n, rows, far):
    """The row of a bias table for distance n >= 0: distances below rows/2 have a row each, the others share the rest on a
    logarithmic scale that reaches the last row at distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(T, table, far):
    """[heads, T, T]: table[bucket(i - j), h] for j <= i, zero above the diagonal (never read)."""
    rows, H = table.shape
    out = torch.zeros((H, T, T), dtype=table.dtype)
    for n in range(T):
        b = distance_bucket(n, rows, far)
        for i in range(n, T):
            out[:, i, i - n] = table[b]
    return out


def query_temperature(T, coef, every, dtype):
    """[T]: 1 + coef * ln(floor((p + 1) / every) + 1) at position p."""
    p = torch.arange(T, dtype=torch.float64)
    return (1.0 + coef * torch.log(torch.floor((p + 1) / every) + 1.0)).to(dtype)


def causal_attention(q, k, v, scale, bias=None, sink_zero=False):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h uses kv head h // (H // G); token i sees every j <= i.
    bias [H, T, T] is added to the scaled scores. sink_zero: the softmax's denominator holds one more term, exp(0), that
    has no value. Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            s = (k[: i + 1, g] @ q[i, h]) * scale
            if bias is not None:
                s = s + bias[h, i, : i + 1]
            m = s.max()
            if sink_zero:
                m = torch.clamp(m, min=0.0)
            e = torch.exp(s - m)
            den = e.sum() + (math.exp(-float(m)) if sink_zero else 0.0)
            out[i, h] = (e / den) @ v[: i + 1, g]
    return out


def bias_gated_attention(h, p, m, eps, kv=None):
    """The mixer 'attention'. p: tensors by local name; m: heads, kv_heads, dim, vdim, scale, bias_max. kv: (k, v) of
    another layer, used instead of projecting (the layer then has no k / v tensors). Returns (y, (k, v))."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).view(T, H, d)
    q = rms_norm(q, p["q.norm"], eps)
    if kv is None:
        k = (h @ p["k"].T + p["k.b"]).view(T, G, d)
        k = rms_norm(k, p["k.norm"], eps)
        v = (h @ p["v"].T + p["v.b"]).view(T, G, dv)
    else:
        k, v = kv
    bias = distance_bias(T, p["rel"], m["bias_max"])
    o = causal_attention(q, k, v, m["scale"], bias=bias)
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T, (k, v)


def key_value_attention(h, p, m, eps):
    """The mixer 'attention_2': the values are the projected keys before their norm; queries carry a temperature that grows
    with the position; the softmax has a sink of score 0."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ p["q"].T).view(T, H, d)
    k_raw = (h @ p["k"].T).view(T, G, d)
    q = rms_norm(q, p["q.norm"], eps)
    k = rms_norm(k_raw, p["k.norm"], eps)
    qt = m.get("q_temp")
    if qt is not None:
        q = q * query_temperature(T, qt["coef"], qt["every"], q.dtype)[:, None, None]
    o = causal_attention(q, k, k_raw, m["scale"], sink_zero=True)
    return o.reshape(T, H * d) @ p["o"].T


def capped(z, cap):
    return cap * torch.tanh(z / cap)


def matrix_memory(q, k, v, i_log, f_log, state=None):
    """The stabilised matrix memory, token by token. q, k [T, H, d] (q already scaled), v [T, H, dv], i_log, f_log [T, H]
    (log input gate, log forget gate). state: (S [H, d, dv], n [H, d], m [H]) or None (zeros; the running maximum starts
    at 0). Returns (o [T, H, dv], state)."""
    T, H, d = q.shape
    dv = v.shape[2]
    if state is None:
        S, n, m = torch.zeros((H, d, dv), dtype=q.dtype), torch.zeros((H, d), dtype=q.dtype), torch.zeros(H, dtype=q.dtype)
    else:
        S, n, m = (x.clone() for x in state)
    o = torch.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        a = torch.exp(f_log[t] + m - m_new)
        b = torch.exp(i_log[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + DENOM_EPS
        o[t] = num / den[:, None]
    return o, (S, n, m)


def mlstm_mixer(h, p, m, eps, state=None):
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ p["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ p["k"].T).view(T, H, d)
    v = (h @ p["v"].T).view(T, H, dv)
    i_log = capped(h @ p["i"].T + p["i.b"], cap)
    f_log = torch.nn.functional.logsigmoid(capped(h @ p["f"].T + p["f.b"], cap))
    o, state = matrix_memory(q, k, v, i_log, f_log, state)
    o = rms_norm(o, None, eps).reshape(T, H * dv) * p["norm"] * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T, state


def sub(tensors, prefix):
    return {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}


def forward(cfg, tensors, tokens, dtype=torch.float64, want_layers=False):
    """cfg: the parsed config.json; tensors: name -> tensor. Returns logits [T, vocab] (and the residual stream after every
    layer, [layers, T, W])."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = {}
    streams = []
    for i, L in enumerate(cfg["layers"]):
        p, m = sub(w, f"l{i}.mix"), L["mixer"]
        if L["type"] == "attention":
            src = m.get("kv_from")
            y, kv = bias_gated_attention(x, p, m, eps, kv=None if src is None else kept[src])
            kept[i] = kv
        elif L["type"] == "attention_2":
            y = key_value_attention(x, p, m, eps)
        elif L["type"] == "mlstm":
            y, _ = mlstm_mixer(x, p, m, eps)
        else:
            raise ValueError(L["type"])
        x = x + mult * rms_norm(y, w[f"l{i}.norm1"], eps)
        if L.get("mlp") is not None:
            f = sub(w, f"l{i}.mlp")
            x = x + mult * rms_norm(gated_ff(x, f["gate"], f["up"], f["down"]), w[f"l{i}.norm2"], eps)
        streams.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(streams)) if want_layers else logits
