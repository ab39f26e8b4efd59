"""Somipel through the engine against the plain implementation under every way of cutting the work: whole prompts; a
prompt and then its last tokens one by one (long decoding, with and without replayed graphs); decoding from the first
token; portions of changing size down to two tokens and one; up to four live requests mixed, unequal, with so few pages and
state slots that both are used again; a marked key at every distance around the bias table's edges and around page borders;
a first token that only the matrix memory carries to position 300, and one that attention finds among hundreds; greedy
generation through `LLM.generate` and the scheduler; the command line; and the trace runner as a process."""
import json
import os
import subprocess
import sys
import warnings

import pytest
import torch

import plain_somipel as P
from somipel_configs import SOMIPEL, make_weights, token_ids

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 5e-2}
LENGTHS = {"a": [1, 2, 15, 16, 17, 41, 130], "b": [3, 33, 129, 140], "c": [1, 16, 17, 90], "d": [2, 6, 50, 150]}
CASES = [("a", 0), ("b", 1), ("c", 2), ("d", 3)]
DTYPES = ["float32", "bfloat16"]


def _engine(raw, w, dtype, num_pages=48, max_seqs=4, max_batch_tokens=512):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.engine import Engine
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        return Engine.from_tensors(config_from_json(raw), w, dtype=dtype, page_size=16, num_pages=num_pages, max_seqs=max_seqs,
                                   max_batch_tokens=max_batch_tokens)


_oracle_cache = {}


# How peaked the attention is made (the standard deviation of the scaled scores): in 32-bit as sharp as the test wants it; in
# bfloat16 less, since every sublayer's output is normed to unit size before it is added, so what rounding does to a sharp
# softmax reaches the logits undamped.
PEAK = {"float32": 4.0, "bfloat16": 2.5}


def _weights(name, seed, dtype):
    return make_weights(SOMIPEL[name](), seed, peak=PEAK[dtype])


def _oracle(name, seed, ids, dtype):
    key = (name, seed, tuple(ids), PEAK[dtype])
    if key not in _oracle_cache:
        _oracle_cache[key] = P.forward(SOMIPEL[name](), _weights(name, seed, dtype), ids)
    return _oracle_cache[key]


def _check(got, ref, dtype, what):
    """Per position: the root mean square over the vocabulary of the logits' difference (each side's mean taken off: a shift
    of all logits changes no probability), relative to the root mean square of the expected logits."""
    got, ref = got.double().cpu(), ref.double()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    got, ref = got - got.mean(dim=-1, keepdim=True), ref - ref.mean(dim=-1, keepdim=True)
    err = (got - ref).pow(2).mean(dim=-1).sqrt() / ref.pow(2).mean(dim=-1).sqrt()
    bad = torch.nonzero(err > TOL[dtype])
    n = ref.shape[0]
    allowed = 0 if dtype == "float32" else n // 25
    worst = float(err.max()) if n else 0.0
    assert bad.numel() <= allowed and (dtype == "float32" or worst <= 2 * TOL[dtype]), \
        f"{what}: first wrong position {int(bad[0])} of {n} (rel err {float(err[int(bad[0])]):.2e}, worst {worst:.2e}, {bad.numel()} wrong)"


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
    raw = SOMIPEL[name]()
    eng = _engine(raw, _weights(name, seed, dtype), dtype)
    for n in LENGTHS[name]:
        ids = token_ids(n, raw["vocab"], 100 + n)
        _check(_run_cut(eng, ids, [n]), _oracle(name, seed, ids, dtype), dtype, f"{name} whole prompt of {n}")
    eng.synchronize()
    eng.cache.check_invariants()


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_prompt_then_token_by_token(cuda_device, name, seed, dtype, graphs):
    """Prefill against decoding through the cache and the states: the last 60 tokens one by one, and a sequence decoded from
    its very first token on. With `graphs` the single-token steps are captured and replayed as CUDA graphs."""
    raw = SOMIPEL[name]()
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
    raw = SOMIPEL[name]()
    eng = _engine(raw, _weights(name, seed, dtype), dtype)
    ids = token_ids(131, raw["vocab"], 9)
    ref = _oracle(name, seed, ids, dtype)
    for cuts in ([2, 2, 3, 16, 1, 31, 17, 2, 40, 15, 2], [64, 64, 3], [5] * 26 + [1], [15, 1, 16, 32, 33, 34]):
        _check(_run_cut(eng, ids, cuts), ref, dtype, f"{name} portions {cuts[:6]}")
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,seed", CASES)
def test_mixed_batches_reuse_pages_and_slots(cuda_device, name, seed, dtype):
    """Five unequal requests through three state slots and a pool that cannot hold them all at once: single tokens beside
    portions, requests that pause, pages and slots given back and taken again."""
    raw = SOMIPEL[name]()
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
def test_a_marked_key_at_the_bias_tables_edges_and_at_page_borders(cuda_device, name, seed, dtype):
    """One token with an embedding far from the others stands at every distance around the bias tables' edges (rows/2, the
    distance of the last row) and around page borders from the token whose logits are compared, in a prompt, in portions
    and decoded alone: a bias row that is one off, or a key that is lost, moves those logits."""
    raw = SOMIPEL[name]()
    w = make_weights(raw, seed, peak=PEAK[dtype])
    w["embed"][5] = (w["embed"][5].float() * 4.0).to(torch.bfloat16)        # the marked token
    eng = _engine(raw, w, dtype)
    base = [t if t != 5 else 6 for t in token_ids(64, raw["vocab"], 12)]
    for at in (63, 62, 60, 59, 58, 57, 48, 47, 44, 43, 42, 32, 31, 24, 23, 22, 16, 15, 1, 0):
        ids = list(base)
        ids[at] = 5
        ref = P.forward(raw, w, ids)
        for cuts in ([64], [at + 1] + [1] * (63 - at), [at, 2] + [1] * (62 - at) if at + 2 <= 64 else [64], [33, 15, 16]):
            if sum(cuts) != 64 or min(cuts) < 1:
                continue
            _check(_run_cut(eng, ids, cuts), ref, dtype, f"marker at {at}, cuts {cuts[:3]}")
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_reaches_the_end(cuda_device, dtype):
    """A change of the first token must still move the logits 300 tokens later - through the matrix memory (forget gates near
    one) and through attention that finds it among hundreds of keys - and the engine must follow the plain implementation
    there, whole and decoded."""
    raw = SOMIPEL["a"]()
    w = make_weights(raw, 13, peak=PEAK[dtype])
    ids = token_ids(300, raw["vocab"], 14)
    other = [(ids[0] + 1) % raw["vocab"]] + ids[1:]
    ref, ref2 = P.forward(raw, w, ids), P.forward(raw, w, other)
    assert float((ref[-1] - ref2[-1]).abs().max()) > 1e-3 * float(ref[-1].abs().max())
    eng = _engine(raw, w, dtype)
    _check(_run_cut(eng, ids, [300])[-40:], ref[-40:], dtype, "far token, whole")
    _check(_run_cut(eng, other, [260] + [1] * 40)[-40:], ref2[-40:], dtype, "far token, decoded")
    _check(_run_cut(eng, other, [7, 130, 2, 121] + [1] * 40)[-40:], ref2[-40:], dtype, "far token, portions then decoded")
    eng.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_llm(cuda_device, dtype):
    from infinilm_b200.config import config_from_json
    from infinilm_b200.llm import LLM, SamplingParams
    raw = SOMIPEL["c"]()
    w = make_weights(raw, 4, peak=PEAK[dtype])
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
            lg = P.forward(raw, w, ids)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) > (1e-3 if dtype == "float32" else 0.2 * float(lg.abs().max())):
                assert t == int(torch.argmax(lg)), f"token {len(ids) - len(p)}"
            ids.append(t)
    llm.close()


def test_command_line_on_a_random_folder(cuda_device, tmp_path):
    """The package's command line: write a folder of random weights for a configuration, then generate from it."""
    from infinilm_b200 import cli
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(SOMIPEL["a"]()))
    folder = str(tmp_path / "m")
    assert cli.main(["--write-random-model", folder, "--config", str(cfg_path), "--seed", "3"]) == 0
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", RuntimeWarning)
        rc = cli.main(["--model", folder, "--enable-paged-attn", "--block-size", "16", "--num-blocks", "32", "--prompt-len", "21",
                       "--max-new-tokens", "9", "--batch-size", "2", "--ignore-eos", "--enable-graph", "--log-level", "ERROR"])
    assert rc == 0


def test_trace_runner_as_a_process(cuda_device, tmp_path):
    """A folder whose config.json does not name the bias tables' row count: the stored tensors give it."""
    from infinilm_b200.config import config_from_json
    from infinilm_b200.weights import write_model_folder
    raw = SOMIPEL["b"]()
    folder = write_model_folder(config_from_json(raw), 6, str(tmp_path / "m"))
    stripped = json.loads(json.dumps(raw))
    for L in stripped["layers"]:
        L["mixer"].pop("bias_rows", None)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(stripped, f)
    from infinilm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    w = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
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
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
                            "--max-tokens", "192"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {n}" for n in range(len(steps))]
        ref = {k: P.forward(raw, w, ids) for k, ids in req.items()}
        k0 = 0
        for n, st in enumerate(steps):
            rows = [x for e in wants[k0:k0 + len(st)] for x in e]
            k0 += len(st)
            got = torch.frombuffer(bytearray(open(os.path.join(out_dir, f"{n}.f32"), "rb").read()), dtype=torch.float32).view(len(rows), raw["vocab"])
            _check(got, torch.stack([ref[rid][pos] for rid, pos in rows]), dtype, f"trace step {n} ({dtype})")
