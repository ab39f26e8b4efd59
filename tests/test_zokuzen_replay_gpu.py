"""Zokuzen through the engine against the plain implementation under every way of cutting the work: whole prompts; a
prompt and then its last tokens one by one (long decoding, with and without replayed graphs); decoding from the first
token; portions of changing size down to two tokens and one; up to four live requests mixed, unequal, with so few pages and
state slots that both are used again; a marked token at every distance around the edges of the position runs and of the
windows and around page borders; a first token that only the recurrence carries to position 300; greedy generation through
`LLM.generate` and the scheduler; the command line; and the trace runner as a process."""
import json
import os
import subprocess
import sys
import warnings

import pytest
import torch

import plain_zokuzen as P
from zokuzen_configs import ZOKUZEN, make_weights, token_ids

pytestmark = pytest.mark.gpu

TOL = {"float32": 3e-5, "bfloat16": 5e-2}
MARGIN = {"float32": 1e-6, "bfloat16": 2e-2}      # a routing choice closer than this to turning is not compared
LENGTHS = {"a": [1, 2, 15, 16, 17, 41, 130], "b": [3, 33, 131, 140], "c": [1, 16, 17, 90], "d": [2, 6, 50, 150]}
CASES = [("a", 0), ("b", 1), ("c", 2), ("d", 3)]
DTYPES = ["float32", "bfloat16"]
PEAK = {"float32": 4.0, "bfloat16": 2.5}


def _engine(raw, w, dtype, num_pages=48, max_seqs=4, max_batch_tokens=512):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        return Engine.from_tensors(config_from_json(raw), w, dtype=dtype, page_size=16, num_pages=num_pages, max_seqs=max_seqs,
                                   max_batch_tokens=max_batch_tokens)


_oracle_cache = {}


def _weights(name, seed, dtype):
    # (bfloat16: routing choices that rounding cannot turn, so that every position is compared)
    return make_weights(ZOKUZEN[name](), seed, peak=PEAK[dtype], clear_choices=dtype == "bfloat16")


def _plain(raw, w, ids):
    """(logits, per position the smallest margin of any router's choice)."""
    margins = []
    lg = P.forward(raw, w, ids, margins=margins)
    m = torch.stack(margins).amin(0) if margins else torch.full((len(ids),), float("inf"), dtype=torch.float64)
    return lg, m


def _oracle(name, seed, ids, dtype):
    key = (name, seed, tuple(ids), PEAK[dtype])
    if key not in _oracle_cache:
        _oracle_cache[key] = _plain(ZOKUZEN[name](), _weights(name, seed, dtype), ids)
    return _oracle_cache[key]


def _check(got, oracle, dtype, what, cum=True):
    """Per position: the root mean square over the vocabulary of the logits' difference (each side's mean taken off), relative
    to that of the expected logits. A position is compared only where neither it nor an earlier position of its sequence made
    a routing choice that rounding can turn (the token's own feed-forward would differ, and later tokens read it).
    cum False: the margins given are already the smallest up to each row's position."""
    ref, margin = oracle
    got, ref = got.double().cpu(), ref.double()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    keep = (torch.cummin(margin, 0).values if cum else margin) > MARGIN[dtype]
    assert keep.float().mean() > (0.5 if dtype == "float32" else 0.99), f"{what}: the test's weights leave too few clear choices"
    got, ref = got - got.mean(dim=-1, keepdim=True), ref - ref.mean(dim=-1, keepdim=True)
    err = (got - ref).pow(2).mean(dim=-1).sqrt() / ref.pow(2).mean(dim=-1).sqrt()
    err = torch.where(keep, err, torch.zeros_like(err))
    bad = torch.nonzero(err > TOL[dtype])
    n = int(keep.sum())
    allowed = 0 if dtype == "float32" else max(1, n // 25)
    worst = float(err.max()) if n else 0.0
    assert bad.numel() <= allowed and (dtype == "float32" or worst <= 2 * TOL[dtype]), \
        f"{what}: first wrong position {int(bad[0])} of {ref.shape[0]} (rel err {float(err[int(bad[0])]):.2e}, worst {worst:.2e}, {bad.numel()} wrong)"


def _tail(oracle, n):
    return oracle[0][-n:], torch.cummin(oracle[1], 0).values[-n:]


def _run_cut(eng, ids, cuts, seq_id="r"):
    from infinilm_b200.engine import StepEntry
    assert sum(cuts) == len(ids)
    seq, outs, a = eng.open(seq_id), [], 0
    for c in cuts:
        outs.append(eng.step([StepEntry(seq, ids[a:a + c], list(range(c)))]).clone())
        a += c
    eng.close(seq)
    return torch.cat(outs, 0)


def _run_schedule(eng, requests, schedule):
    from infinilm_b200.engine import StepEntry
    done, seqs, outs = {k: 0 for k in requests}, {}, {k: [] for k in requests}
    for step in schedule:
        entries = []
        for rid, n in step:
            if rid not in seqs:
                seqs[rid] = eng.open(rid)
            entries.append(StepEntry(seqs[rid], requests[rid][done[rid]:done[rid] + n], list(range(n))))
            done[rid] += n
        logits, r = eng.step(entries).clone(), 0
        for rid, n in step:
            outs[rid].append(logits[r:r + n])
            r += n
            if done[rid] == len(requests[rid]):
                eng.close(seqs.pop(rid))
        eng.cache.check_invariants()
    assert all(done[k] == len(requests[k]) for k in requests)
    return {k: torch.cat(v, 0) for k, v in outs.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_whole_prompts(cuda_device, name, seed, dtype):
    raw = ZOKUZEN[name]()
    eng = _engine(raw, _weights(name, seed, dtype), dtype)
    for n in LENGTHS[name]:
        ids = token_ids(n, raw["vocab"], 100 + n)
        _check(_run_cut(eng, ids, [n]), _oracle(name, seed, ids, dtype), dtype, f"{name} whole prompt of {n}")
    eng.synchronize()
    eng.cache.check_invariants()


@pytest.mark.parametrize("name,seed", CASES)
def test_every_layer_in_32_bit(cuda_device, name, seed):
    """The sum of the stream's copies after every layer, against the plain implementation."""
    from infinilm_b200.engine import StepEntry
    raw = ZOKUZEN[name]()
    w = _weights(name, seed, "float32")
    eng = _engine(raw, w, "float32")
    ids = token_ids(70, raw["vocab"], 5)
    _, want = P.forward(raw, w, ids, want_layers=True)
    got = []
    eng.runner.tap = lambda nm, resid, pending: got.append(resid.detach().clone().cpu())
    seq = eng.open("x")
    eng.step([StepEntry(seq, ids, [69])])
    eng.close(seq)
    eng.runner.tap = None
    assert len(got) == len(raw["layers"])
    for i, g in enumerate(got):
        err = float((g.double() - want[i]).abs().max()) / float(want[i].abs().max())
        assert err < 3e-5, f"layer {i}: {err:.2e}"


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_prompt_then_token_by_token(cuda_device, name, seed, dtype, graphs):
    """Prefill against decoding through the cache and the states: the last 60 tokens one by one, and a sequence decoded from
    its very first token on. With `graphs` the single-token steps are captured and replayed as CUDA graphs."""
    raw = ZOKUZEN[name]()
    eng = _engine(raw, _weights(name, seed, dtype), dtype)
    if graphs:
        eng.enable_graphs()
        assert eng.model.graph_safe
    ids = token_ids(110, raw["vocab"], 7)
    _check(_run_cut(eng, ids, [50] + [1] * 60), _oracle(name, seed, ids, dtype), dtype, f"{name} 50 + 60 x 1")
    ids = token_ids(45, raw["vocab"], 8)
    _check(_run_cut(eng, ids, [1] * 45), _oracle(name, seed, ids, dtype), dtype, f"{name} 45 x 1")
    eng.synchronize()
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_portions_of_changing_size(cuda_device, name, seed, dtype):
    raw = ZOKUZEN[name]()
    eng = _engine(raw, _weights(name, seed, dtype), dtype)
    ids = token_ids(131, raw["vocab"], 9)
    ref = _oracle(name, seed, ids, dtype)
    for cuts in ([2, 2, 3, 16, 1, 31, 17, 2, 40, 15, 2], [64, 64, 3], [5] * 26 + [1], [15, 1, 16, 32, 33, 34], [23, 2, 24, 1, 25, 56]):
        _check(_run_cut(eng, ids, cuts), ref, dtype, f"{name} portions {cuts[:6]}")
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_mixed_batches_reuse_pages_and_slots(cuda_device, name, seed, dtype):
    """Five unequal requests through three state slots and a pool that cannot hold them all at once: single tokens beside
    portions, requests that pause, pages and slots given back and taken again."""
    raw = ZOKUZEN[name]()
    eng = _engine(raw, _weights(name, seed, dtype), dtype, num_pages=14, max_seqs=3)
    req = {k: token_ids(n, raw["vocab"], 20 + i) for i, (k, n) in enumerate((("p", 90), ("q", 37), ("r", 3), ("s", 70), ("t", 18)))}
    schedule = [[("p", 40), ("q", 2)], [("p", 1), ("q", 1), ("r", 2)], [("q", 30), ("p", 1)], [("r", 1), ("p", 17), ("q", 1)],
                [("p", 1), ("q", 1), ("s", 33)], [("s", 1), ("p", 20), ("q", 2)], [("s", 2), ("p", 10), ("t", 17)], [("s", 34), ("t", 1)]]
    got = _run_schedule(eng, req, schedule)
    for k, ids in req.items():
        _check(got[k], _oracle(name, seed, ids, dtype), dtype, f"{name} mixed, request {k}")
    eng.synchronize()
    assert len(eng.cache.live) == 0 and all(n == grp.pool.n_pages for grp in eng.cache.groups if grp.pool for n in [grp.pool.n_free])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", [("a", 11), ("d", 12)])
def test_a_marked_token_at_the_masks_edges_and_at_page_borders(cuda_device, name, seed, dtype):
    """One token with an embedding far from the others stands at every distance around the edges of the runs of positions
    (24 and 17 in "a", 9 in "d"), of the windows (20; 7) and around page borders from the token whose logits are compared,
    in a prompt, in portions and decoded alone: a key that is seen one position too long, or lost one too early, moves them."""
    raw = ZOKUZEN[name]()
    w = make_weights(raw, seed, peak=PEAK[dtype], clear_choices=dtype == "bfloat16")
    w["embed"][5] = (w["embed"][5].float() * 4.0).to(torch.bfloat16)        # the marked token
    eng = _engine(raw, w, dtype)
    base = [t if t != 5 else 6 for t in token_ids(64, raw["vocab"], 12)]
    for at in (63, 62, 57, 56, 55, 54, 51, 50, 48, 47, 45, 44, 43, 40, 39, 32, 31, 24, 23, 17, 16, 15, 1, 0):
        ids = list(base)
        ids[at] = 5
        ref = _plain(raw, w, ids)
        for cuts in ([64], [at + 1] + [1] * (63 - at), [at, 2] + [1] * (62 - at) if at + 2 <= 64 else [64], [33, 15, 16]):
            if sum(cuts) != 64 or min(cuts) < 1:
                continue
            _check(_run_cut(eng, ids, cuts), ref, dtype, f"marker at {at}, cuts {cuts[:3]}")
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_reaches_the_end(cuda_device, dtype):
    """A change of the first token must still move the logits 300 tokens later - through the recurrence alone (decays near
    one): every attention layer of this configuration has forgotten it - and the engine must follow the plain implementation
    there, whole, decoded and in portions."""
    raw = ZOKUZEN["a"]()
    w = make_weights(raw, 13, peak=PEAK[dtype], clear_choices=dtype == "bfloat16")
    ids = token_ids(300, raw["vocab"], 14)
    other = [(ids[0] + 1) % raw["vocab"]] + ids[1:]
    ref, ref2 = _plain(raw, w, ids), _plain(raw, w, other)
    assert float((ref[0][-1] - ref2[0][-1]).abs().max()) > 3e-4 * float(ref[0][-1].abs().max())
    eng = _engine(raw, w, dtype)
    _check(_run_cut(eng, ids, [300])[-40:], _tail(ref, 40), dtype, "far token, whole", cum=False)
    _check(_run_cut(eng, other, [260] + [1] * 40)[-40:], _tail(ref2, 40), dtype, "far token, decoded", cum=False)
    _check(_run_cut(eng, other, [7, 130, 2, 121] + [1] * 40)[-40:], _tail(ref2, 40), dtype, "far token, portions then decoded", cum=False)
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_llm(cuda_device, dtype):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.llm import LLM, SamplingParams
    raw = ZOKUZEN["c"]()
    w = make_weights(raw, 4, peak=PEAK[dtype], clear_choices=dtype == "bfloat16")
    prompts = [token_ids(n, raw["vocab"], 30 + n) for n in (5, 21, 40)]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        llm = LLM.from_tensors(config_from_json(raw), w, dtype=dtype, num_blocks=40, block_size=16, max_batch_size=3)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(top_k=1, max_tokens=24, ignore_eos=True))
    for p, o in zip(prompts, outs):
        got = list(o.outputs[0].token_ids)
        assert len(got) == 24
        ids = list(p)
        for t in got:                             # every token is the plain implementation's argmax, where that is clear
            lg, margin = _plain(raw, w, ids)
            top2 = torch.topk(lg[-1], 2).values
            if float(margin.min()) < MARGIN[dtype]:
                break                             # a routing choice that rounding can turn: the sequences may part here
            if float(top2[0] - top2[1]) > (1e-3 if dtype == "float32" else 0.2 * float(lg[-1].abs().max())):
                assert t == int(torch.argmax(lg[-1])), f"token {len(ids) - len(p)}"
            ids.append(t)
    llm.close()


def test_command_line_on_a_random_folder(cuda_device, tmp_path):
    """The package's command line: write a folder of random weights for a configuration, then generate from it."""
    from infinilm_b200 import cli
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(ZOKUZEN["a"]()))
    folder = str(tmp_path / "m")
    assert cli.main(["--write-random-model", folder, "--config", str(cfg_path), "--seed", "3"]) == 0
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        rc = cli.main(["--model", folder, "--enable-paged-attn", "--block-size", "16", "--num-blocks", "32", "--prompt-len", "21",
                       "--max-new-tokens", "9", "--batch-size", "2", "--ignore-eos", "--enable-graph", "--log-level", "ERROR"])
    assert rc == 0


def test_trace_runner_as_a_process(cuda_device, tmp_path):
    """A model folder (the head is the embedding table: no tensor of its own) replayed step by step by the runner."""
    from infinilm_b200.weights.safetensors_io import write_safetensors
    raw = ZOKUZEN["b"]()
    w = make_weights(raw, 6, peak=PEAK["bfloat16"], clear_choices=True)
    folder = str(tmp_path / "m")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw, f)
    assert "head" not in w
    write_safetensors(os.path.join(folder, "model.safetensors"), w)
    req = {k: token_ids(n, raw["vocab"], 40 + n) for k, n in (("a", 70), ("b", 9), ("c", 33), ("d", 50), ("e", 20))}
    steps = [[("a", 30), ("b", 2)], [("a", 1), ("b", 7), ("c", 3)], [("a", 39), ("c", 30), ("d", 1)], [("d", 49), ("e", 20)]]
    done, lines, wants = {k: 0 for k in req}, [], []
    for n, st in enumerate(steps):
        entries, end = [], []
        for rid, c in st:
            a = done[rid]
            entries.append({"id": rid, "tokens": req[rid][a:a + c], "want": [0, c - 1] if c > 1 else [0]})
            wants.append([(rid, a), (rid, a + c - 1)] if c > 1 else [(rid, a)])
            done[rid] = a + c
            if done[rid] == len(req[rid]):
                end.append(rid)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out_dir = str(tmp_path / "out")
    ref = {k: _plain(raw, w, ids) for k, ids in req.items()}
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
                            "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {n}" for n in range(len(steps))]
        k0 = 0
        for n, st in enumerate(steps):
            rows = [x for e in wants[k0:k0 + len(st)] for x in e]
            k0 += len(st)
            got = torch.frombuffer(bytearray(open(os.path.join(out_dir, f"{n}.f32"), "rb").read()), dtype=torch.float32).view(len(rows), raw["vocab"])
            want = torch.stack([ref[rid][0][pos] for rid, pos in rows])
            margin = torch.stack([torch.cummin(ref[rid][1], 0).values[pos] for rid, pos in rows])
            _check(got, (want, margin), dtype, f"trace step {n} ({dtype})", cum=False)
