"""Each mechanism of the Somipel parts alone, on the device, against the plain implementation: the norm on a branch with
its residual add and copy; the per-head norms of queries and keys with the query temperature, the cache write and values
that are the un-normed keys; the gate per column with packing; the bias by distance in each of the four attention
kernels, with a key that stands out at page borders and at the table's edges, alone and beside a sink; the log-space
gates with their running maximum through slots that are used again; the gated sum over a matrix state in both kernels,
whole against portions against token by token; the read-out's denominator with the grouped norm and gate."""
import math

import pytest
import torch

import plain_somipel as P

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


# ---- the norm on the branch ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H", [(1, 72), (33, 120), (40, 2048), (3, 5000), (7, 13)])
def test_norm_on_the_branch_then_add(cuda_device, dtype, T, H):
    from infinilm_b200 import ops
    torch.manual_seed(T + H)
    dt = DT[dtype]
    resid, branch = torch.randn(T, H), (torch.randn(T, H) * 3.0).to(dt)
    w = (1.0 + 0.1 * torch.randn(H)).to(torch.bfloat16)
    want = resid.double() + 0.3 * P.rms_norm(branch.double(), w.double(), 1e-5)
    for wd in (torch.float32, torch.bfloat16):
        r = resid.clone().cuda()
        copy = None if dtype == "float32" else torch.empty(T, H, dtype=dt, device="cuda")
        ops.norm_add(r, branch.cuda(), w.to(wd).cuda(), 1e-5, 0.3, copy)
        _close(r, want, "float32", f"norm_add {T}x{H}")
        if copy is not None:
            assert torch.equal(copy.float(), r.to(dt).float())
    if dtype == "bfloat16":
        c = torch.empty(T, H, dtype=dt, device="cuda")
        ops.cast_rows(resid.cuda(), c)
        assert torch.equal(c.cpu(), resid.to(dt))


# ---- query and key norms, temperature, cache write -----------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,dk,dv,v_from_k,temp", [(4, 2, 32, 64, False, None), (3, 1, 24, 24, True, (0.7, 5)), (2, 2, 128, 128, False, (0.5, 1)),
                                                         (6, 3, 20, 12, False, None), (5, 5, 40, 40, True, (1.5, 16)), (2, 1, 18, 7, False, (0.3, 2)),
                                                         (1, 1, 256, 132, False, None)])
@pytest.mark.parametrize("lead,tail", [(3, 5), (4, 8)])      # segments on and off 16-byte borders: both forms of the kernel
def test_qk_norm_temperature_and_store(cuda_device, dtype, nh, nkv, dk, dv, v_from_k, temp, lead, tail):
    from infinilm_b200 import ops
    torch.manual_seed(nh * dk)
    dt = DT[dtype]
    hd = (max(dk, dv) + 15) // 16 * 16
    # two entries in one step: positions 30..36 of one request (over a page border), 0..2 of another; pages out of order
    pos, ent = list(range(30, 37)) + [0, 1, 2], [0] * 7 + [1] * 3
    bt = _i32([[5, 2, 7], [3, -1, -1]])
    T = len(pos)
    nq, nk, nv = nh * dk, nkv * dk, (0 if v_from_k else nkv * dv)
    proj = (torch.randn(T, lead + nq + nk + nv + tail) * 2.0).to(dt)
    q_off, k_off = lead, lead + nq
    v_off = k_off if v_from_k else k_off + nk
    wq, wk = 1.0 + 0.2 * torch.randn(dk), 1.0 + 0.2 * torch.randn(dk)
    cache = torch.full((9, 2, nkv, 16, hd), 9.0, dtype=dt, device="cuda")
    q_out = torch.full((T, nh * hd), 9.0, dtype=dt, device="cuda")
    ops.qk_norm_store(proj.cuda(), q_off, k_off, v_off, nh, nkv, dk, dv, hd, wq.cuda(), wk.cuda(), 1e-5, temp[0] if temp else 0.0,
                      temp[1] if temp else 0, q_out, _i32(pos), _i32(ent), bt, cache, 16)
    x = proj.double()
    q = P.rms_norm(x[:, q_off:q_off + nq].view(T, nh, dk), wq.double(), 1e-5)
    if temp:
        t = torch.tensor([1.0 + temp[0] * math.log((p + 1) // temp[1] + 1) for p in pos], dtype=torch.float64)
        q = q * t[:, None, None]
        assert torch.allclose(t, P.query_temperature(40, temp[0], temp[1], torch.float64)[pos])
    k = P.rms_norm(x[:, k_off:k_off + nk].view(T, nkv, dk), wk.double(), 1e-5)
    v = x[:, v_off:v_off + nkv * dv].view(T, nkv, dv)
    got_q = q_out.view(T, nh, hd)
    _close(got_q[:, :, :dk], q, dtype, "q")
    assert float(got_q[:, :, dk:].float().abs().max() if hd > dk else 0.0) == 0.0
    for t_, (p, e) in enumerate(zip(pos, ent)):
        page = int(bt[e, p // 16])
        _close(cache[page, 0, :, p % 16, :dk], k[t_], dtype, f"k of token {t_}")
        assert torch.equal(cache[page, 1, :, p % 16, :dv].double().cpu(), v[t_])            # values are copied, not computed
        if hd > dk:
            assert float(cache[page, 0, :, p % 16, dk:].float().abs().max()) == 0.0
        if hd > dv:
            assert float(cache[page, 1, :, p % 16, dv:].float().abs().max()) == 0.0
    untouched = cache.clone()
    for p, e in zip(pos, ent):
        untouched[int(bt[e, p // 16]), :, :, p % 16] = 9.0
    assert float((untouched.float() - 9.0).abs().max()) == 0.0                               # no other slot was written
    # a mixer without keys of its own: only the queries
    q2 = torch.empty_like(q_out)
    ops.qk_norm_store(proj.cuda(), q_off, None, 0, nh, nkv, dk, dv, hd, wq.cuda(), None, 1e-5, 0.0, 0, q2, _i32(pos), _i32(ent), bt, None, 16)
    _close(q2.view(T, nh, hd)[:, :, :dk], P.rms_norm(x[:, q_off:q_off + nq].view(T, nh, dk), wq.double(), 1e-5), dtype, "q alone")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gate_per_column_with_packing(cuda_device, dtype):
    from infinilm_b200 import ops
    torch.manual_seed(3)
    dt = DT[dtype]
    for T, nh, hd, dv, lead in ((37, 3, 32, 20, 7), (37, 3, 32, 20, 8), (5, 2, 128, 128, 0), (9, 4, 16, 13, 4), (3000, 16, 64, 64, 64)):
        y, gate = torch.randn(T, nh * hd).to(dt), (torch.randn(T, lead + nh * dv + (-(lead + nh * dv)) % 4) * 3).to(dt)
        out = torch.empty(T, nh * dv, dtype=dt, device="cuda")
        ops.gate_pack(y.cuda(), hd, gate.cuda(), lead, out, nh, dv)
        want = y.double().view(T, nh, hd)[:, :, :dv].reshape(T, -1) * torch.sigmoid(gate.double()[:, lead:lead + nh * dv])
        _close(out, want, dtype, f"gate_pack {T, nh, hd, dv, lead}")
        ops.gate_pack(y.cuda(), hd, None, 0, out, nh, dv)
        assert torch.equal(out.cpu(), y.view(T, nh, hd)[:, :, :dv].reshape(T, -1))


# ---- the bias by distance in the four attention kernels ---------------------------------------------------------------------
def _bias_case(nh, nkv, hd, starts, qlens, seed, far_key=None):
    """Entries e with `starts[e]` cached tokens before their qlens[e] new ones; pages handed out in a scrambled order."""
    g = torch.Generator().manual_seed(seed)
    E = len(starts)
    lens = [s + q for s, q in zip(starts, qlens)]
    n_pages = sum((n + 15) // 16 for n in lens)
    perm = torch.randperm(n_pages + 3, generator=g).tolist()
    width = max((n + 15) // 16 for n in lens)
    bt = torch.full((E, width), -1, dtype=torch.int32)
    ks = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g) for n in lens]
    q = [torch.randn(ql, nh, hd, generator=g) for ql in qlens]
    if far_key is not None:                       # one key that the entry's queries all point at: it outweighs the rest
        e, key = far_key
        ks[e][key] *= 3.0
        q[e] = q[e] * 0.3 + ks[e][key].repeat_interleave(nh // nkv, 0)[None] * 0.4
    cache = torch.zeros(n_pages + 4, 2, nkv, 16, hd)
    k = 0
    for e in range(E):
        for pi in range((lens[e] + 15) // 16):
            bt[e, pi] = perm[k]
            n = min(16, lens[e] - pi * 16)
            cache[perm[k], 0, :, :n] = ks[e][pi * 16: pi * 16 + n].transpose(0, 1)
            cache[perm[k], 1, :, :n] = vs[e][pi * 16: pi * 16 + n].transpose(0, 1)
            k += 1
    return dict(E=E, starts=starts, qlens=qlens, lens=lens, k=ks, v=vs, q=q, bt=bt, cache=cache)


def _bias_reference(c, scale, table, far, dtype, sink):
    outs = []
    for e in range(c["E"]):
        k, v, q = (x.to(DT[dtype]).double() for x in (c["k"][e], c["v"][e], c["q"][e]))
        n, s0 = c["lens"][e], c["starts"][e]
        full = torch.zeros(n, q.shape[1], q.shape[2], dtype=torch.float64)                  # rows before the portion: their queries do not matter
        full[s0:] = q
        bias = None if table is None else P.distance_bias(n, table.double(), far)
        outs.append(P.causal_attention(full, k, v, scale, bias=bias, sink_zero=sink)[s0:])
    return torch.cat(outs, 0).reshape(sum(c["qlens"]), -1)


def _run_attention(kernel, c, nh, nkv, hd, scale, table, far, dtype, sink, splits=1):
    from infinilm_b200 import ops
    from infinilm_b200.parts.normed_attention import distance_buckets
    dt = DT[dtype]
    q = torch.cat(c["q"], 0).reshape(-1, nh * hd).to(dt).cuda()
    cache, bt = c["cache"].to(dt).cuda(), c["bt"].cuda()
    db = None
    if table is not None:
        db = table[torch.tensor(distance_buckets(table.shape[0], far))].contiguous().float().cuda()      # [far + 1, heads]
    sk = torch.zeros(nh, device="cuda") if sink else None
    T = q.shape[0]
    out = torch.full((T, nh * hd), float("nan"), device="cuda", dtype=dt)
    qstart = [0]
    for ql in c["qlens"]:
        qstart.append(qstart[-1] + ql)
    G = nh // nkv
    if kernel == "plain":
        pos = [s + i for s, ql in zip(c["starts"], c["qlens"]) for i in range(ql)]
        ent = [e for e, ql in enumerate(c["qlens"]) for _ in range(ql)]
        ops.attention_plain(q, out, cache, bt, _i32(pos), _i32(ent), 16, nh, nkv, hd, scale, None, sk, db)
    elif kernel == "decode":
        rows = T * nh * splits
        ops.attention_decode(q, out, cache, bt, _i32(c["lens"]), T, 16, nh, nkv, hd, scale, None, 0, splits,
                             torch.empty(rows * hd, device="cuda"), torch.empty(rows * 2, device="cuda"),
                             kv_map=ops.kv_tensor_map(cache), sink=sk, dist_bias=db)
    elif kernel == "prefill":
        tpt = max(1, 64 // G)
        ops.attention_prefill(q, out, cache, bt, _i32(qstart), _i32(c["lens"]), 0, c["E"], sum((x + tpt - 1) // tpt for x in c["qlens"]),
                              16, nh, nkv, hd, scale, None, sink=sk, dist_bias=db)
    else:
        tpt = max(1, ops.prefill_tc5_rows(hd) // G)
        ops.attention_prefill_tc5(q, out, ops.kv_tensor_map(cache), bt, _i32(qstart), _i32(c["lens"]), 0, c["E"],
                                  sum((x + tpt - 1) // tpt for x in c["qlens"]), 16, nh, nkv, hd, scale, None, sink=sk, dist_bias=db)
    torch.cuda.synchronize()
    ops.check_status("cuda:0")
    return out


PORTIONS = dict(starts=[0, 250, 31, 16, 0], qlens=[70, 9, 2, 33, 1])
SINGLES = dict(starts=[0, 15, 16, 17, 399, 63], qlens=[1] * 6)
TABLES = [(16, 120), (4, 5), (32, 300), (6, 1000)]          # (rows, distance of the last row)


@pytest.mark.parametrize("kernel,dtype,nh,nkv,hd", [("plain", "float32", 3, 1, 40), ("plain", "float32", 4, 2, 128), ("plain", "bfloat16", 6, 3, 48),
                                                    ("prefill", "bfloat16", 6, 3, 48), ("prefill", "bfloat16", 3, 1, 64), ("prefill", "bfloat16", 8, 8, 16),
                                                    ("tc5", "bfloat16", 4, 2, 64), ("tc5", "bfloat16", 9, 1, 128), ("tc5", "bfloat16", 2, 2, 64),
                                                    ("tc5", "bfloat16", 4, 1, 256)])
@pytest.mark.parametrize("far_key", [None, (1, 16), (1, 255), (0, 0), (1, 139)])
def test_distance_bias_over_portions(cuda_device, kernel, dtype, nh, nkv, hd, far_key):
    c = _bias_case(nh, nkv, hd, PORTIONS["starts"], PORTIONS["qlens"], nh * hd, far_key)
    for i, (rows, far) in enumerate(TABLES):
        table = torch.randn(rows, nh, generator=torch.Generator().manual_seed(rows)) * 3.0
        sink = i % 2 == 1
        got = _run_attention(kernel, c, nh, nkv, hd, 0.23, table, far, dtype, sink)
        _close(got, _bias_reference(c, 0.23, table, far, dtype, sink), dtype, f"{kernel} table {rows}/{far} key {far_key}")


@pytest.mark.parametrize("kernel,dtype,nh,nkv,hd,splits", [("plain", "float32", 3, 1, 40, 1), ("decode", "bfloat16", 6, 3, 48, 1), ("decode", "bfloat16", 3, 1, 64, 4),
                                                           ("decode", "bfloat16", 9, 1, 128, 7), ("decode", "bfloat16", 20, 1, 32, 13),
                                                           ("decode", "bfloat16", 4, 4, 96, 2), ("decode", "bfloat16", 34, 2, 64, 3)])
@pytest.mark.parametrize("far_key", [None, (4, 16), (4, 383), (4, 280), (2, 15), (4, 395)])
def test_distance_bias_of_single_tokens(cuda_device, kernel, dtype, nh, nkv, hd, splits, far_key):
    c = _bias_case(nh, nkv, hd, SINGLES["starts"], SINGLES["qlens"], nh + hd, far_key)
    for i, (rows, far) in enumerate(TABLES):
        table = torch.randn(rows, nh, generator=torch.Generator().manual_seed(rows)) * 3.0
        sink = i % 2 == 0
        got = _run_attention(kernel, c, nh, nkv, hd, 0.31, table, far, dtype, sink, splits)
        _close(got, _bias_reference(c, 0.31, table, far, dtype, sink), dtype, f"{kernel} table {rows}/{far} key {far_key} splits {splits}")


@pytest.mark.parametrize("kernel", ["plain", "decode", "prefill", "tc5"])
def test_a_bias_row_decides_the_answer(cuda_device, kernel):
    """All keys alike; one row of the table towers: the output is the value at exactly that distance, in every kernel."""
    nh, nkv, hd = 2, 1, 64
    decode = kernel == "decode"
    starts, qlens = ([70, 20], [1, 1]) if decode else ([40, 0], [31, 21])
    c = _bias_case(nh, nkv, hd, starts, qlens, 5)
    for e in range(2):
        c["k"][e][:] = c["k"][e][0]
    c = dict(c, cache=c["cache"].clone())
    for e in range(2):
        for pi in range((c["lens"][e] + 15) // 16):
            n = min(16, c["lens"][e] - pi * 16)
            c["cache"][int(c["bt"][e, pi]), 0, :, :n] = c["k"][e][pi * 16: pi * 16 + n].transpose(0, 1)
    rows, far = 16, 120
    for row, dist in ((3, [3]), (7, [7]), (8, [8, 9, 10, 11]), (9, [12, 13, 14, 15, 16])):      # rows from 8 on cover ranges of distances
        table = torch.zeros(rows, nh)
        table[row] = 60.0
        got = _run_attention(kernel, c, nh, nkv, hd, 0.2, table, far, "bfloat16", False, 2 if decode else 1).float().cpu()
        ref = _bias_reference(c, 0.2, table, far, "bfloat16", False)
        _close(got, ref, "bfloat16", f"{kernel} row {row}")
        # the last token of the first entry sits at position lens - 1: with one distance in the row, its output is that value row
        if len(dist) == 1 and c["lens"][0] - 1 - dist[0] >= 0:
            v = c["v"][0][c["lens"][0] - 1 - dist[0], 0].to(torch.bfloat16).float()
            assert float((got[qlens[0] - 1, :hd] - v).abs().max()) < 0.05


# ---- the matrix memory ---------------------------------------------------------------------------------------------------
def _gate_inputs(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(T, 2 * H + 3, generator=g) * 6.0
    z[:, 1 + H: 1 + 2 * H] += 3.0
    return z


@pytest.mark.parametrize("cap", [15.0, 2.0, 0.0])
@pytest.mark.parametrize("H", [1, 3, 8])
def test_log_space_gates_and_running_maximum_in_portions(cuda_device, H, cap):
    from infinilm_b200 import ops
    T = 1100                                      # (beyond two chunks of the kernel's form for long portions, and of its other form)
    z = _gate_inputs(T, H, H)
    zi, zf = z[:, 1:1 + H].double(), z[:, 1 + H:1 + 2 * H].double()
    il = P.capped(zi, cap) if cap > 0 else zi
    fl = torch.nn.functional.logsigmoid(P.capped(zf, cap) if cap > 0 else zf)
    m = torch.zeros(H, dtype=torch.float64)
    want = []
    for t in range(T):
        mn = torch.maximum(fl[t] + m, il[t])
        want.append(torch.stack([torch.exp(fl[t] + m - mn), torch.exp(il[t] - mn), torch.exp(-mn)]))
        m = mn
    want = torch.stack(want)                      # [T, 3, H]
    for cuts in ([T], [129, 1, 1, 2, 127, 40, 800], [1] * 20 + [280, 800], [511, 513, 76], [200, 255, 257, 388]):
        mstate = torch.zeros(4, H, device="cuda")
        mstate[2] = 5.0                           # a slot that an earlier request left dirty: the first step reads slot 0
        outs, a = [], 0
        for i, n in enumerate(cuts):
            zz = z[a:a + n].cuda()
            dec, inw, flo = (torch.empty(n, H, device="cuda") for _ in range(3))
            ops.stabilized_gates(zz, 1, 1 + H, cap, mstate, _i32([0 if i == 0 else 2]), _i32([2]), _i32([0, n]), 1, dec, inw, flo, H)
            outs.append(torch.stack([dec, inw, flo], 1))
            a += n
        got = torch.cat(outs).cpu().double()
        assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max()), cuts
        assert float((mstate[2].cpu().double() - m).abs().max()) <= 1e-5 * max(1.0, float(m.abs().max()))


@pytest.fixture(params=[False, True], ids=["registers", "shared"])
def generic(request):
    return request.param


def _gated_scan(ops, q, k, v, dec, inw, H, d, dv, state, rd, wr, generic):
    n = q.shape[0]
    out = torch.empty(n, H * (dv + 1), device="cuda")
    ops.matrix_state_scan(ops.SCAN_GATED, q, k, v, H, H, d, dv + 1, 0, None, inw, dec, state, _i32([rd]), _i32([wr]), _i32([0, n]), 1, out,
                          generic=generic, single=(n == 1))
    return out


@pytest.mark.parametrize("H,d,dv", [(2, 32, 32), (3, 16, 24), (4, 8, 32), (1, 20, 12), (2, 128, 64), (1, 256, 35), (2, 40, 8), (1, 10, 1), (1, 50, 127)])
def test_gated_sum_whole_portions_and_token_by_token(cuda_device, generic, H, d, dv):
    """The matrix memory through the framework's scan and read-out kernels against the token loop of the definition."""
    from infinilm_b200 import ops
    torch.manual_seed(d + dv)
    T, cap, eps = 300, 15.0, 1e-5
    q, k, v = torch.randn(T, H * d), torch.randn(T, H * d), torch.randn(T, H * dv)
    z = _gate_inputs(T, H, 7)
    gate = torch.randn(T, H * dv)
    w = 1.0 + 0.1 * torch.randn(H * dv)
    il, fl = P.capped(z[:, 1:1 + H].double(), cap), torch.nn.functional.logsigmoid(P.capped(z[:, 1 + H:1 + 2 * H].double(), cap))
    o, (S, n_, m) = P.matrix_memory(q.double().view(T, H, d) * d ** -0.5, k.double().view(T, H, d), v.double().view(T, H, dv), il, fl)
    want = (P.rms_norm(o, None, eps).reshape(T, H * dv) * w.double() * torch.sigmoid(gate.double()))
    for cuts in ([T], [257] + [1] * 43, [2, 126, 1, 1, 130, 40]):
        state = torch.zeros(4, H, dv + 1, d, device="cuda")
        mstate = torch.zeros(4, H, device="cuda")
        state[3], mstate[3] = 3.0, -2.0           # the slot held something else: a request's first step reads slot 0
        outs, a = [], 0
        for i, n in enumerate(cuts):
            sl = slice(a, a + n)
            dec, inw, flo = (torch.empty(n, H, device="cuda") for _ in range(3))
            rd = 0 if i == 0 else 3
            ops.stabilized_gates(z[sl].cuda(), 1, 1 + H, cap, mstate, _i32([rd]), _i32([3]), _i32([0, n]), 1, dec, inw, flo, H)
            raw = _gated_scan(ops, q[sl].cuda(), k[sl].cuda(), v[sl].cuda(), dec, inw, H, d, dv, state, rd, 3, generic)
            out = torch.empty(n, H * dv, device="cuda")
            ops.group_norm_gate(raw, w.cuda(), eps, gate[sl].cuda(), 0, ops.GATE_SIGMOID, out, dv, den_floor=flo, x_scale=d ** -0.5, den_eps=1e-6)
            outs.append(out)
            a += n
        got = torch.cat(outs).cpu().double()
        assert float((got - want).abs().max()) <= 5e-5 * float(want.abs().max()), cuts
        # the state: S column by column with the normaliser n as the last column, and the running maximum
        Sg = state[3].cpu().double()
        assert float((Sg[:, :dv] - S.transpose(1, 2)).abs().max()) <= 5e-5 * float(S.abs().max())
        assert float((Sg[:, dv] - n_).abs().max()) <= 5e-5 * float(n_.abs().max())
        assert float((mstate[3].cpu().double() - m).abs().max()) <= 1e-5 * max(1.0, float(m.abs().max()))


def test_gated_sum_of_a_batch_equals_each_alone(cuda_device, generic):
    """Unequal entries in one launch, single tokens first as a step lays them out: bit for bit what each gives alone."""
    from infinilm_b200 import ops
    torch.manual_seed(1)
    H, d, dv = 3, 24, 20
    lens = [1, 1, 9, 40, 2]
    T = sum(lens)
    q, k, v = (torch.randn(T, H * x, device="cuda") for x in (d, d, dv))
    dec, inw = torch.rand(T, H, device="cuda"), torch.rand(T, H, device="cuda")
    start = torch.randn(6, H, dv + 1, d, device="cuda")
    start[0] = 0.0
    qs = [0]
    for n in lens:
        qs.append(qs[-1] + n)
    state = start.clone()
    out = torch.empty(T, H * (dv + 1), device="cuda")
    rd, wr = _i32([1, 0, 2, 3, 0]), _i32([1, 4, 2, 3, 5])
    ops.matrix_state_scan(ops.SCAN_GATED, q, k, v, H, H, d, dv + 1, 0, None, inw, dec, state, rd, wr, _i32(qs), 2, out, generic=generic, single=True)
    ops.matrix_state_scan(ops.SCAN_GATED, q, k, v, H, H, d, dv + 1, 0, None, inw, dec, state, rd, wr, _i32(qs), 3, out, generic=generic, first_entry=2)
    for e, n in enumerate(lens):
        sl = slice(qs[e], qs[e + 1])
        st = start.clone()
        alone = _gated_scan(ops, q[sl], k[sl], v[sl], dec[sl].contiguous(), inw[sl].contiguous(), H, d, dv, st, int(rd[e]), int(wr[e]), generic)
        assert torch.equal(alone, out[sl]) and torch.equal(st[int(wr[e])], state[int(wr[e])]), e


def test_a_running_maximum_that_moves_far(cuda_device):
    """Input gates that grow by hundreds (no cap): sums stay finite because they are kept relative to the running maximum,
    and the read-out's floor exp(-m) vanishes instead of overflowing."""
    from infinilm_b200 import ops
    H, d, dv, T = 1, 16, 8, 64
    torch.manual_seed(2)
    q, k, v = torch.randn(T, d), torch.randn(T, d), torch.randn(T, dv)
    z = torch.zeros(T, 2)
    z[:, 0] = torch.linspace(-200.0, 300.0, T)
    z[:, 1] = 4.0
    o, _ = P.matrix_memory(q.double().view(T, 1, d) * 0.25, k.double().view(T, 1, d), v.double().view(T, 1, dv), z[:, :1].double(),
                           torch.nn.functional.logsigmoid(z[:, 1:].double()))
    state, mstate = torch.zeros(2, 1, dv + 1, d, device="cuda"), torch.zeros(2, 1, device="cuda")
    dec, inw, flo = (torch.empty(T, 1, device="cuda") for _ in range(3))
    ops.stabilized_gates(z.cuda(), 0, 1, 0.0, mstate, _i32([0]), _i32([1]), _i32([0, T]), 1, dec, inw, flo, 1)
    raw = _gated_scan(ops, q.cuda(), k.cuda(), v.cuda(), dec, inw, 1, d, dv, state, 0, 1, False)
    out = torch.empty(T, dv, device="cuda")
    ops.group_norm_gate(raw, torch.ones(dv, device="cuda"), 1e-5, torch.full((T, dv), 50.0, device="cuda"), 0, ops.GATE_SIGMOID, out, dv,
                        den_floor=flo, x_scale=0.25, den_eps=1e-6)
    want = P.rms_norm(o, None, 1e-5).reshape(T, dv)
    assert torch.isfinite(out).all() and float((out.cpu().double() - want).abs().max()) <= 1e-4 * float(want.abs().max())
