"""Each mechanism of the Zokuzen parts alone, on the device, against the plain implementation: the step between two
sublayers over several copies of the residual stream; the norm over a whole projection with the rotation of part of each
head and the cache write; the two masks (runs of positions, sliding window) in each of the four attention kernels with a
key that stands out just inside and just outside every edge and at page borders; the blend of a token with its
predecessor through state slots that are used again; the channel-decay recurrence in both kernels, whole against portions
against token by token and a batch against each alone; the routing rule, identity units and the gated shared unit."""
import math

import pytest
import torch

import plain_zokuzen as P

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _i32(x, dev="cuda"):
    return torch.tensor(x, dtype=torch.int32, device=dev)


def _close(got, ref, dtype, what, tol=None):
    got, ref = got.double().cpu(), ref.double()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    tol = tol or (3e-5 if dtype == "float32" else 2.5e-2)
    err = float((got - ref).abs().max()) / max(float(ref.abs().max()), 1e-9)
    assert err <= tol, f"{what}: relative error {err:.2e}"


# ---- several copies of the residual stream -----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,S,H", [(1, 1, 72), (5, 2, 120), (33, 3, 256), (4, 4, 2048), (2, 8, 13), (3, 5, 5000), (2, 16, 40)])
def test_step_between_sublayers(cuda_device, dtype, T, S, H):
    from infinilm_b200 import ops
    g = torch.Generator().manual_seed(T * S + H)
    dt = DT[dtype]
    emb = torch.randn(T, H, generator=g) * 3
    w_in, w_out, w_in2 = (torch.randn(S, generator=g) for _ in range(3))
    mix = torch.randn(S, S, generator=g)
    nw = 1.0 + 0.1 * torch.randn(H, generator=g)
    y = torch.randn(T, H, generator=g).to(dt)
    streams = torch.full((T, S * H), 7.0, device="cuda")
    normed = torch.empty(T, H, dtype=dt, device="cuda")
    # the copies start as the embedding's output; the first sublayer's input
    ops.hyper_step(streams, S, init=emb.cuda(), in_next=w_in.cuda(), norm_weight=nw.cuda(), eps=1e-5, normed=normed)
    xs = torch.stack([emb.double()] * S)
    assert torch.equal(streams.view(T, S, H).cpu(), xs.transpose(0, 1).float())
    _close(normed, P.rms_norm(P.streams_read(xs, w_in.double()), nw.double(), 1e-5), dtype, "first input")
    # write-back, the next input, and the sum in one pass
    total = torch.empty(T, H, device="cuda")
    ops.hyper_step(streams, S, y=y.cuda(), mix=mix.cuda(), out_w=w_out.cuda(), in_next=w_in2.cuda(), norm_weight=nw.cuda(), eps=1e-5,
                   normed=normed, sum_out=total)
    xs = P.streams_write(xs, y.double(), mix.double(), w_out.double())
    _close(streams.view(T, S, H).transpose(0, 1), xs, "float32", "write-back")
    _close(total, xs.sum(0), "float32", "sum of the copies")
    _close(normed, P.rms_norm(P.streams_read(xs, w_in2.double()), nw.double(), 1e-5), dtype, "next input")
    # reading alone changes nothing
    before = streams.clone()
    ops.hyper_step(streams, S, in_next=w_in.cuda(), norm_weight=nw.cuda(), eps=1e-5, normed=normed)
    assert torch.equal(before, streams)
    _close(normed, P.rms_norm(P.streams_read(xs, w_in.double()), nw.double(), 1e-5), dtype, "input read alone")


# ---- norm over the whole projection, rotation of part of a head, cache write ----------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,dk,dv,rot", [(4, 2, 32, 48, 8), (6, 6, 16, 16, 16), (2, 1, 128, 128, 0), (3, 3, 20, 12, 4), (2, 1, 64, 64, 16),
                                             (5, 1, 40, 7, 40), (1, 1, 256, 130, 2)])
def test_projection_norm_rotation_and_store(cuda_device, dtype, nh, nkv, dk, dv, rot):
    from infinilm_b200 import ops
    g = torch.Generator().manual_seed(nh * dk + rot)
    dt = DT[dtype]
    hd = (max(dk, dv) + 15) // 16 * 16
    pos, ent = list(range(29, 36)) + [0, 1, 2] + [1000], [0] * 7 + [1] * 3 + [2]       # over a page border; a sequence's start; far out
    bt = torch.full((3, 63), -1, dtype=torch.int32)
    bt[0, :3], bt[1, 0], bt[2, 62] = torch.tensor([5, 2, 7]), 3, 1
    bt = bt.cuda()
    T, lead = len(pos), 3
    nq, nk, nv = nh * dk, nkv * dk, nkv * dv
    proj = (torch.randn(T, lead + nq + nk + nv + 5, generator=g) * 2.0).to(dt)
    wq, wk = 1.0 + 0.2 * torch.randn(nq, generator=g), 1.0 + 0.2 * torch.randn(nk, generator=g)
    base = 777.0
    inv = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float().cuda() if rot else None
    cache = torch.full((9, 2, nkv, 16, hd), 9.0, dtype=dt, device="cuda")
    q_out = torch.full((T, nh * hd), 9.0, dtype=dt, device="cuda")
    ops.qk_rows_norm_rope_store(proj.cuda(), lead, lead + nq, lead + nq + nk, nh, nkv, dk, dv, hd, wq.cuda(), wk.cuda(), 1e-5, rot, inv, q_out,
                                _i32(pos), _i32(ent), bt, cache, 16)
    x = proj.double()

    def want(cols, w, heads):
        z = P.rms_norm(cols, w.double(), 1e-5).view(T, heads, dk)          # one root mean square for all heads of a token
        if not rot:
            return z
        full = torch.zeros(1001, heads, dk, dtype=torch.float64)
        full[pos] = z
        return P.rotate_half(full, rot, base)[pos]
    q, k = want(x[:, lead:lead + nq], wq, nh), want(x[:, lead + nq:lead + nq + nk], wk, nkv)
    v = x[:, lead + nq + nk:lead + nq + nk + nv].view(T, nkv, dv)
    # (angles are float32 on the device: at position 1000 their rounding is what the 32-bit comparison allows for)
    tol = 2e-4 if dtype == "float32" else None
    got_q = q_out.view(T, nh, hd)
    _close(got_q[:, :, :dk], q, dtype, "q", tol)
    assert hd == dk or float(got_q[:, :, dk:].float().abs().max()) == 0.0
    for t_, (p, e) in enumerate(zip(pos, ent)):
        page = int(bt[e, p // 16])
        _close(cache[page, 0, :, p % 16, :dk], k[t_], dtype, f"k of token {t_}", tol)
        assert torch.equal(cache[page, 1, :, p % 16, :dv].double().cpu(), v[t_])
        assert hd == dk or float(cache[page, 0, :, p % 16, dk:].float().abs().max()) == 0.0
        assert hd == dv or float(cache[page, 1, :, p % 16, dv:].float().abs().max()) == 0.0
    untouched = cache.clone()
    for p, e in zip(pos, ent):
        untouched[int(bt[e, p // 16]), :, :, p % 16] = 9.0
    assert float((untouched.float() - 9.0).abs().max()) == 0.0
    q2 = torch.empty_like(q_out)                  # a mixer without keys of its own: only the queries
    ops.qk_rows_norm_rope_store(proj.cuda(), lead, None, 0, nh, nkv, dk, dv, hd, wq.cuda(), None, 1e-5, rot, inv, q2, _i32(pos), _i32(ent), bt, None, 16)
    assert torch.equal(q2, q_out)


# ---- the masks in the four attention kernels ---------------------------------------------------------------------------------
def _attn_case(nh, nkv, hd, starts, qlens, seed, marked=None):
    """Entries e with starts[e] cached tokens before their qlens[e] new ones; pages handed out in a scrambled order.
    marked (entry, key): that key is made to outweigh all others for every query of the entry that may see it."""
    g = torch.Generator().manual_seed(seed)
    E = len(starts)
    lens = [s + q for s, q in zip(starts, qlens)]
    n_pages = sum((n + 15) // 16 for n in lens)
    perm = torch.randperm(n_pages + 3, generator=g).tolist()
    bt = torch.full((E, max((n + 15) // 16 for n in lens)), -1, dtype=torch.int32)
    ks = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    qs = [torch.randn(ql, nh, hd, generator=g) for ql in qlens]
    if marked is not None:
        e, key = marked
        ks[e][key] *= 3.0
        qs[e] = qs[e] * 0.3 + ks[e][key].repeat_interleave(nh // nkv, 0)[None] * 0.4
    cache = torch.zeros(n_pages + 4, 2, nkv, 16, hd)
    n = 0
    for e in range(E):
        for pi in range((lens[e] + 15) // 16):
            bt[e, pi] = perm[n]
            c = min(16, lens[e] - pi * 16)
            cache[perm[n], 0, :, :c] = ks[e][pi * 16: pi * 16 + c].transpose(0, 1)
            cache[perm[n], 1, :, :c] = vs[e][pi * 16: pi * 16 + c].transpose(0, 1)
            n += 1
    return dict(E=E, starts=starts, qlens=qlens, lens=lens, k=ks, v=vs, q=qs, bt=bt, cache=cache)


def _attn_reference(c, scale, kind, size, dtype):
    outs = []
    for e in range(c["E"]):
        k, v, q = (x.to(DT[dtype]).double() for x in (c["k"][e], c["v"][e], c["q"][e]))
        n, s0 = c["lens"][e], c["starts"][e]
        full = torch.zeros(n, q.shape[1], q.shape[2], dtype=torch.float64)      # rows before the portion: their queries do not matter
        full[s0:] = q
        outs.append(P.softmax_attention(full, k, v, scale, P.visible(n, kind, size))[s0:])
    return torch.cat(outs, 0).reshape(sum(c["qlens"]), -1)


def _run_attention(kernel, c, nh, nkv, hd, scale, mask_arg, dtype, splits=1):
    from infinilm_b200 import ops
    dt = DT[dtype]
    q = torch.cat(c["q"], 0).reshape(-1, nh * hd).to(dt).cuda()
    cache, bt = c["cache"].to(dt).cuda(), c["bt"].cuda()
    T = q.shape[0]
    out = torch.full((T, nh * hd), float("nan"), device="cuda", dtype=dt)
    qstart = [0]
    for ql in c["qlens"]:
        qstart.append(qstart[-1] + ql)
    G = nh // nkv
    if kernel == "plain":
        pos = [s + i for s, ql in zip(c["starts"], c["qlens"]) for i in range(ql)]
        ent = [e for e, ql in enumerate(c["qlens"]) for _ in range(ql)]
        ops.attention_plain(q, out, cache, bt, _i32(pos), _i32(ent), 16, nh, nkv, hd, scale, mask_arg)
    elif kernel == "decode":
        rows = T * nh * splits
        ops.attention_decode(q, out, cache, bt, _i32(c["lens"]), T, 16, nh, nkv, hd, scale, mask_arg, 0, splits,
                             torch.empty(rows * hd, device="cuda"), torch.empty(rows * 2, device="cuda"), kv_map=ops.kv_tensor_map(cache))
    elif kernel == "prefill":
        tpt = max(1, 64 // G)
        ops.attention_prefill(q, out, cache, bt, _i32(qstart), _i32(c["lens"]), 0, c["E"], sum((x + tpt - 1) // tpt for x in c["qlens"]),
                              16, nh, nkv, hd, scale, mask_arg)
    else:
        tpt = max(1, ops.prefill_tc5_rows(hd) // G)
        ops.attention_prefill_tc5(q, out, ops.kv_tensor_map(cache), bt, _i32(qstart), _i32(c["lens"]), 0, c["E"],
                                  sum((x + tpt - 1) // tpt for x in c["qlens"]), 16, nh, nkv, hd, scale, mask_arg)
    torch.cuda.synchronize()
    ops.check_status("cuda:0")
    return out


MASKS = [("chunk", 24), ("chunk", 16), ("chunk", 210), ("chunk", 5), ("chunk", 1), ("window", 20), ("window", 90), ("window", 1), ("window", 17)]


@pytest.mark.parametrize("kernel,dtype,nh,nkv,hd", [("plain", "float32", 3, 1, 40), ("plain", "bfloat16", 6, 3, 48), ("prefill", "bfloat16", 6, 3, 48),
                                                    ("prefill", "bfloat16", 8, 8, 80), ("tc5", "bfloat16", 4, 2, 64), ("tc5", "bfloat16", 9, 1, 128),
                                                    ("tc5", "bfloat16", 4, 1, 256)])
def test_masks_over_portions(cuda_device, kernel, dtype, nh, nkv, hd):
    """Portions that start and end anywhere against runs of positions and windows of several sizes, with one key made to stand
    out: the last one before a run's border or a window's edge, the first one behind it, and keys at page borders. A query
    that may see the key follows it; one that may not must not."""
    starts, qlens = [0, 250, 31, 16, 0], [70, 9, 2, 33, 1]
    for kind, size in MASKS:
        marks = [None, (1, 255), (1, 240), (0, 0), (0, 23), (0, 24), (0, 47), (0, 48), (3, 15), (3, 16), (3, 31), (1, 258 - size if size < 200 else 209),
                 (1, 259 - size if size < 200 else 210)]
        for mk in marks[:5] + marks[5 + (size % 4) * 2: 7 + (size % 4) * 2] + marks[-2:]:
            c = _attn_case(nh, nkv, hd, starts, qlens, nh * hd + size, mk)
            got = _run_attention(kernel, c, nh, nkv, hd, 0.2, -size if kind == "chunk" else size, dtype)
            _close(got, _attn_reference(c, 0.2, kind, size, dtype), dtype, f"{kernel} {kind} {size}, marked {mk}")


@pytest.mark.parametrize("kernel,dtype,nh,nkv,hd,splits", [("plain", "float32", 3, 1, 40, 1), ("decode", "bfloat16", 6, 3, 48, 1), ("decode", "bfloat16", 3, 1, 64, 4),
                                                           ("decode", "bfloat16", 8, 1, 80, 3), ("decode", "bfloat16", 4, 2, 128, 7), ("decode", "bfloat16", 2, 2, 256, 2)])
def test_masks_of_single_tokens(cuda_device, kernel, dtype, nh, nkv, hd, splits):
    """Single tokens at lengths around page borders and around every mask's edges: the token at a run's first position sees
    itself alone; the one before it sees its whole run; a window's oldest key is seen, the one before it is not."""
    starts, qlens = [0, 15, 16, 17, 399, 63, 23, 24, 47, 48, 210, 209], [1] * 12
    for kind, size in MASKS:
        for mk in (None, (4, 399), (4, 400 - size if kind == "window" else (399 // size) * size), (4, max(0, 399 - size) if kind == "window" else max(0, (399 // size) * size - 1)),
                   (5, 48), (5, 47)):
            c = _attn_case(nh, nkv, hd, starts, qlens, nh * hd + size, mk)
            got = _run_attention(kernel, c, nh, nkv, hd, 0.2, -size if kind == "chunk" else size, dtype, splits)
            _close(got, _attn_reference(c, 0.2, kind, size, dtype), dtype, f"{kernel} {kind} {size}, marked {mk}")


# ---- a token blended with its predecessor -------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,n_mix", [(72, 5), (256, 5), (130, 1), (8, 3)])
def test_blend_with_the_predecessor_through_slots(cuda_device, dtype, W, n_mix):
    from infinilm_b200 import ops
    g = torch.Generator().manual_seed(W)
    dt = DT[dtype]
    mu = torch.rand(n_mix, W, generator=g)
    seqs = {"a": torch.randn(23, W, generator=g).to(dt), "b": torch.randn(9, W, generator=g).to(dt), "c": torch.randn(4, W, generator=g).to(dt)}

    def want(h):
        prev = torch.cat([torch.zeros(1, W, dtype=torch.float64), h.double()[:-1]])
        return torch.cat([h.double() + (prev - h.double()) * mu[m].double() for m in range(n_mix)], dim=1)
    state = torch.zeros(3, W, device="cuda")      # slot 0: the zero state
    state[1:] = 5.0                               # what an earlier request left in the slots
    # steps: (request, tokens, read slot, write slot); a: slot 1, b: slot 2, then c takes slot 2 again after b has ended
    steps = [[("a", 10, 0, 1), ("b", 1, 0, 2)], [("b", 8, 2, 2), ("a", 1, 1, 1)], [("a", 12, 1, 1), ("c", 2, 0, 2)], [("c", 1, 2, 2)], [("c", 1, 2, 2)]]
    done, got = {k: 0 for k in seqs}, {k: [] for k in seqs}
    for st in steps:
        rows = torch.cat([seqs[k][done[k]:done[k] + n] for k, n, _, _ in st])
        qs = [0]
        for _, n, _, _ in st:
            qs.append(qs[-1] + n)
        ent = [e for e, (_, n, _, _) in enumerate(st) for _ in range(n)]
        out = torch.empty(rows.shape[0], n_mix * W, dtype=dt, device="cuda")
        ops.token_shift_mix(rows.cuda(), mu.cuda(), state, _i32([s[2] for s in st]), _i32([s[3] for s in st]), _i32(ent), _i32(qs), out)
        for e, (k, n, _, _) in enumerate(st):
            got[k].append(out[qs[e]:qs[e + 1]].clone())
            done[k] += n
        assert float(state[0].abs().max()) == 0.0
    for k in seqs:
        _close(torch.cat(got[k]), want(seqs[k]), dtype, f"request {k}", 1e-6 if dtype == "float32" else 1e-2)
    assert torch.equal(state[1].cpu(), seqs["a"][-1].float()) and torch.equal(state[2].cpu(), seqs["c"][-1].float())


def test_decay_from_its_pre_activation_and_tanh(cuda_device):
    from infinilm_b200 import ops
    g = torch.Generator().manual_seed(1)
    z, w0 = torch.randn(37, 100, generator=g) * 3, torch.randn(60, generator=g)
    zz = z.clone().cuda()
    ops.double_exp_decay(zz[:, :80], w0.cuda(), 60)
    _close(zz[:, :60], torch.exp(-torch.exp(z.double()[:, :60] + w0.double())), "float32", "decay", 1e-6)
    assert torch.equal(zz[:, 60:].cpu(), z[:, 60:])
    for dt in (torch.float32, torch.bfloat16):
        out = torch.empty(37, 100, dtype=dt, device="cuda")
        ops.tanh_rows(z.cuda(), out)
        _close(out, torch.tanh(z.double()), "float32" if dt == torch.float32 else "bfloat16", "tanh", 1e-6 if dt == torch.float32 else 5e-3)


# ---- the channel-decay recurrence ----------------------------------------------------------------------------------------------
@pytest.fixture(params=[False, True], ids=["registers", "shared"])
def generic(request):
    return request.param


def _scan(ops, r, k, v, w, u, H, d, state, rd, wr, qstart, generic, single=False):
    T = r.shape[0]
    out = torch.full((T, H * d), float("nan"), device="cuda")
    ops.matrix_state_scan(ops.SCAN_CHANNEL_DECAY, r, k, v, H, H, d, d, 0, u, None, w, state, _i32(rd), _i32(wr), _i32(qstart), len(rd), out,
                          generic=generic, single=single)
    return out


@pytest.mark.parametrize("H,d", [(2, 32), (3, 16), (4, 8), (1, 20), (2, 64), (1, 128), (1, 256), (2, 40), (1, 10), (1, 3), (1, 272)])
def test_channel_decay_whole_portions_and_token_by_token(cuda_device, generic, H, d):
    from infinilm_b200 import ops
    if d > 256 and not generic:
        pytest.skip("key sizes beyond 256 run the kernel with the state in shared memory")
    g = torch.Generator().manual_seed(H * d)
    T = 75
    r, k, v = (torch.randn(T, H * d, generator=g) for _ in range(3))
    w = torch.exp(-torch.exp(torch.randn(T, H * d, generator=g) - 2.0))          # mostly near one, some channels forget fast
    u = torch.randn(H, d, generator=g)
    ref, S_ref = P.wkv_recurrence(*(x.double().view(T, H, d) for x in (r, k, v, w)), u.double())
    ref = ref.reshape(T, H * d)
    rc, kc, vc, wc, uc = (x.cuda() for x in (r, k, v, w, u))
    # decays as a view with a row stride (columns of a wider product)
    wide = torch.zeros(T, H * d + 8, device="cuda")
    wide[:, :H * d] = wc
    state = torch.zeros(3, H, d, d, device="cuda")
    state[1:] = 3.0
    got = _scan(ops, rc, kc, vc, wide[:, :H * d], uc, H, d, state, [0], [1], [0, T], generic)
    _close(got, ref, "float32", "whole")
    _close(state[1].transpose(-1, -2), S_ref, "float32", "state (stored column by column)")
    assert float(state[0].abs().max()) == 0.0 and float((state[2] - 3.0).abs().max()) == 0.0
    # portions down to two tokens and one, the state carried through slot 2
    outs, a, rd = [], 0, 0
    for n in (2, 1, 7, 8, 9, 16, 1, 1, 30):
        outs.append(_scan(ops, rc[a:a + n], kc[a:a + n], vc[a:a + n], wc[a:a + n], uc, H, d, state, [rd], [2], [0, n], generic, single=(n == 1)))
        a, rd = a + n, 2
    assert a == T
    _close(torch.cat(outs), ref, "float32", "portions")
    _close(state[2], state[1].cpu(), "float32", "state after portions", 1e-5)


def test_channel_decay_of_a_batch_equals_each_alone(cuda_device, generic):
    from infinilm_b200 import ops
    H, d = 3, 24
    g = torch.Generator().manual_seed(5)
    lens = [1, 1, 1, 19, 2, 40]                   # single tokens first, as the engine orders a step
    T = sum(lens)
    r, k, v = (torch.randn(T, H * d, generator=g).cuda() for _ in range(3))
    w = torch.exp(-torch.exp(torch.randn(T, H * d, generator=g) - 2.0)).cuda()
    u = torch.randn(H, d, generator=g).cuda()
    base = torch.randn(7, H, d, d, generator=g).cuda() * 0.3
    base[0] = 0.0
    qs = [0]
    for n in lens:
        qs.append(qs[-1] + n)
    rd = [1, 2, 0, 3, 4, 0]
    wr = [1, 2, 5, 3, 4, 6]

    class Ctx:
        n_decode, n_entries, T = 3, 6, sum(lens)
    st = base.clone()
    out = torch.full((T, H * d), float("nan"), device="cuda")
    ops.matrix_state_scan_step(Ctx, ops.SCAN_CHANNEL_DECAY, r, k, v, H, H, d, d, 0, u, None, w, st, _i32(rd), _i32(wr), _i32(qs), out=out, generic=generic)
    for e, n in enumerate(lens):
        st1 = base.clone()
        o1 = _scan(ops, r[qs[e]:qs[e + 1]], k[qs[e]:qs[e + 1]], v[qs[e]:qs[e + 1]], w[qs[e]:qs[e + 1]], u, H, d, st1, [rd[e]], [wr[e]], [0, n], generic, single=(n == 1))
        assert torch.equal(o1, out[qs[e]:qs[e + 1]]), f"entry {e}"
        assert torch.equal(st1[wr[e]], st[wr[e]])
    ref, _ = P.wkv_recurrence(*(x[qs[3]:qs[4]].double().cpu().view(19, H, d) for x in (r, k, v, w)), u.double().cpu(), base[3].double().cpu().transpose(-1, -2))
    _close(out[qs[3]:qs[4]], ref.reshape(19, H * d), "float32", "an entry that starts from a state")


def test_a_bonus_that_decides_and_a_channel_that_forgets(cuda_device):
    """The token's own k v^T reaches its read-out through the bonus alone and only the state through the decays: with the bonus
    zero a first token reads nothing; with a channel's decay zero, what went in through that channel is gone a token later."""
    from infinilm_b200 import ops
    H, d, T = 1, 16, 3
    r, k, v = torch.ones(T, d).cuda(), torch.zeros(T, d).cuda(), torch.ones(T, d).cuda()
    k[0, 3], k[0, 5] = 1.0, 2.0
    w = torch.ones(T, d).cuda()
    w[1, 5] = 0.0                                 # token 1 wipes channel 5 AFTER it has read
    state = torch.zeros(2, H, d, d).cuda()
    for u_val, want in ((0.0, [0.0, 3.0, 1.0]), (0.5, [1.5, 3.0, 1.0])):
        out = _scan(ops, r, k, v, w, torch.full((H, d), u_val).cuda(), H, d, state, [0], [1], [0, T], False)
        assert out[:, 0].tolist() == want


# ---- routing ------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top", [(10, 3), (5, 5), (64, 6), (2, 1), (33, 32)])
def test_choice_by_corrected_scores(cuda_device, E, top):
    from infinilm_b200 import ops
    g = torch.Generator().manual_seed(E)
    T = 200
    z = torch.randn(T, E + 1, generator=g) * 2            # one more column that is no expert's
    corr = torch.randn(E, generator=g) * (3.0 / E)
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wt = torch.empty(T, top, device="cuda")
    ops.moe_select(z.cuda()[:, :E], corr.cuda(), idx, wt, top, rule=ops.ROUTE_SOFTMAX_ALL, out_scale=2.5)
    s = torch.softmax(z[:, :E].double(), -1)
    c = s + corr.double()
    order = torch.sort(c, dim=-1, descending=True, stable=True)
    clear = (order.values[:, top - 1] - order.values[:, top] > 1e-6) if top < E else torch.ones(T, dtype=torch.bool)
    assert clear.float().mean() > 0.9
    assert torch.equal(idx.cpu()[clear].long(), order.indices[clear][:, :top])
    chosen = torch.gather(s, 1, idx.cpu().long())
    _close(wt[clear], (chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * 2.5)[clear], "float32", "weights", 1e-5)
    # ties: the lower output wins
    zt = torch.zeros(4, E + 1).cuda()
    ops.moe_select(zt[:, :E], None, idx[:4], wt[:4], top, rule=ops.ROUTE_SOFTMAX_ALL, out_scale=1.0)
    assert idx[:4].cpu().tolist() == [list(range(top))] * 4


class _Ctx:
    def __init__(self, dtype, max_tokens=512):
        from infinilm_b200.engine.step import Workspace
        self.ws, self.dtype, self.tap = Workspace(torch.device("cuda"), max_tokens), dtype, None


def _moe_part(raw_mlp, W, dtype, seed, scale_corr=100.0):
    from infinilm_b200.parts.moe import RoutedExperts
    r = raw_mlp["router"]
    part = RoutedExperts({"hidden": W, "n_experts": r["experts"], "top": r["top"], "expert_ff": raw_mlp["expert"]["ff"],
                          "shared_ff": raw_mlp["shared"]["ff"] if raw_mlp.get("shared") else None, "router_bias": True, "bias_name": "correction",
                          "route_rule": "softmax_all", "route_scale": r["scale"], "n_identity": r["identity"],
                          "shared_gate": raw_mlp.get("shared") is not None}, "f", DT[dtype])
    g = torch.Generator().manual_seed(seed)
    w = {}
    for ws in part.weight_specs():
        x = torch.randn(ws.shape, generator=g) * (ws.init[1] if ws.init[0] != "ones_normal" else 0.1)
        if ws.name == "correction":
            x = x * scale_corr
        w[ws.name] = x.to(torch.bfloat16)
    part.set_weights({k: v.cuda() for k, v in w.items()})
    return part, w


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,ff,experts,top,identity,scale,shared", [(96, 40, 4, 2, 1, 1.5, 48), (120, 56, 3, 6, 3, 2.0, 64), (128, 32, 7, 4, 2, 2.0, None),
                                                                      (72, 24, 2, 1, 0, 1.0, 40), (256, 88, 9, 3, 2, 1.5, 136), (100, 20, 1, 2, 1, 0.5, 12)])
def test_routed_feed_forward_with_identity_units_and_gated_shared_unit(cuda_device, dtype, W, ff, experts, top, identity, scale, shared):
    mlp = {"expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity, "scale": scale}}
    if shared:
        mlp["shared"] = {"ff": shared}
    part, w = _moe_part(mlp, W, dtype, W + ff)
    ctx = _Ctx(DT[dtype], 1200)
    p = {k: v.double() for k, v in w.items()}
    for T in (1, 2, 16, 17, 150, 1100):           # a few rows: the two short router kernels; many: bfloat16 hands the experts' products to the library
        h = torch.randn(T, W, generator=torch.Generator().manual_seed(T)).to(DT[dtype])
        margins = []
        ref = P.routed_feed_forward(h.double(), p, mlp, margins)
        got = part.forward(h.cuda(), ctx)
        if dtype == "bfloat16":                   # a choice that rounding can turn is not compared
            keep = margins[0] > 0.02
            assert T < 100 or keep.float().mean() > 0.5
            got, ref = got[keep.cuda()], ref[keep]
        _close(got, ref, dtype, f"T={T}")
        if T == 150:                              # a token's result does not depend on what else is in the batch
            alone = part.forward(h[40:41].cuda(), ctx).clone()
            both = part.forward(h.cuda(), ctx)[40:41]
            assert torch.allclose(alone.float(), both.float(), rtol=0, atol=1e-6 * float(both.abs().max()) if dtype == "float32" else 2e-2 * float(both.abs().max()))
