"""The Mamusun family through the engine's step function, cache manager and entry points, against the plain restatement of
tests/plain_mamusun.py: every way of cutting the same requests into steps (whole, the last tokens one by one, portions down
to two tokens, mixed batches over a pool so small that pages and slots are used again), the first tokens, long decoding across
many windows and pages, every mixer and feed-forward alone in a model of one layer, and greedy generation through
`LLM.generate`.  CPU cases run the host logic with the plain-torch kernel double; `-m gpu` cases run the CUDA kernels.

bfloat16 and routed experts: a token whose best router outputs lie closer together than bfloat16 rounding moves them may pick
another expert than the float64 restatement does.  So in bfloat16 the configurations run with softer attention scales, once
with their routed feed-forwards replaced by dense ones (`soft_variant`: there the ways of cutting must also agree with one
another) and once as they are; both under bounds on the median and the ninth decile of the error.  float32 is compared at
every position, with the configurations as they are."""
import copy

import pytest
import torch

import plain_mamusun as plain
import replay_cases as cases
from helpers import make_engine, rel_err, run_steps
from mamusun_models import CONFIGS, attention, config, dense, layer, moe, parallel, sink_attention, write_model

FP32_TOL, BF16_TOL = 3e-4, 5e-2
# lengths around every window (10, 21; 5, 16, 23; 1; 4) and page size (16, 8, 16, 4) of the configurations
LENGTHS = {"A": [1, 9, 10, 11, 22, 33, 70], "B": [2, 5, 6, 16, 17, 24, 40, 97], "C": [3, 16, 17, 40, 75], "D": [4, 5, 7, 15, 16, 17, 69, 130]}

GPU = pytest.mark.gpu
CASES = [pytest.param("cpu", "float32", n, id=f"cpu-fp32-{n}") for n in "ABCD"] + \
        [pytest.param("cuda:0", dt, n, marks=GPU, id=f"gpu-{dt}-{n}") for dt in ("float32", "bfloat16") for n in "ABCD"]


def mixers_of(cfg):
    for lay in cfg["layers"]:
        yield lay["mixer"]["left"] if lay["type"] == "parallel" else lay["mixer"]


def soft_variant(cfg, dense_ff=True):
    cfg = copy.deepcopy(cfg)
    for m in mixers_of(cfg):
        m["scale"] *= 0.25
    for lay in cfg["layers"]:
        if dense_ff and lay["mlp"] is not None and lay["mlp"]["kind"] == "moe":
            lay["mlp"] = {"kind": "dense", "ff": lay["mlp"]["expert"]["ff"]}
    return cfg


def has_experts(name):
    return any(l["mlp"] is not None and l["mlp"]["kind"] == "moe" for l in CONFIGS[name][0]["layers"])


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for name, (cfg, seed, _) in CONFIGS.items():
        out[name] = write_model(cfg, str(tmp_path_factory.mktemp(f"mam_{name}")), seed)
        out[name + "-dense"] = write_model(soft_variant(cfg), str(tmp_path_factory.mktemp(f"mam_{name}_dense")), seed)
        out[name + "-soft"] = write_model(soft_variant(cfg, dense_ff=False), str(tmp_path_factory.mktemp(f"mam_{name}_soft")), seed)
    return out


@pytest.fixture(scope="module")
def refs(dirs):
    out = {}
    for key, d in dirs.items():
        cfg, seed, _ = CONFIGS[key[0]]
        reqs = cases.requests_for(cfg["vocab"], LENGTHS[key[0]], seed + 10)
        c, w = plain.read_model_dir(d)
        out[key] = (reqs, {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()})
    return out


def errors(rows, ref, reqs):
    """Per position: largest difference of the logits row over the largest logit of the request."""
    out = []
    for rid, toks in reqs.items():
        got = torch.stack([rows[(rid, i)] for i in range(len(toks))])
        top = max(ref[rid].abs().max().item(), 1e-30)
        out += ((got.float().cpu() - ref[rid]).abs().amax(dim=1) / top).tolist()
    return out


def compare(rows, ref, reqs, tol, strict=True):
    """float32 (`strict`): every position within `tol`.  bfloat16: the median within `tol` and nine positions in ten within
    twice that: the configurations are ill-conditioned on purpose (peaked softmax, norms that bring a small sum back to full
    size), so single positions magnify bfloat16's rounding whatever the kernels do."""
    e = sorted(errors(rows, ref, reqs))
    if strict:
        assert e[-1] <= tol, e[-1]
    else:
        assert e[len(e) // 2] <= tol and e[int(0.9 * (len(e) - 1))] <= 2 * tol, (e[len(e) // 2], e[int(0.9 * (len(e) - 1))], e[-1])


def agree(rows, base, ref, tol):
    worst = max(((rows[k].float() - base[k].float()).abs().max() / ref[k[0]].abs().max()).item() for k in base)
    assert worst <= tol, worst


def variants(name, dtype):
    if dtype == "float32":
        return [(name, True, True)]
    return [(name + "-dense", False, True)] + ([(name + "-soft", False, False)] if has_experts(name) else [])


@pytest.mark.parametrize("device,dtype,name", CASES)
def test_every_way_of_cutting(dirs, refs, device, dtype, name):
    page = CONFIGS[name][2]
    tol = FP32_TOL if dtype == "float32" else BF16_TOL
    for key, strict, cuts_agree in variants(name, dtype):
        reqs, ref = refs[key]
        mixed_steps, peak = cases.mixed(reqs, live=3, seed=2)
        pages = peak // page
        eng = make_engine(dirs[key], dtype, page, pages, device=device, max_num_seqs=3, max_num_batched_tokens=peak)
        base = None
        for steps in (cases.whole(reqs), cases.last_one_by_one(reqs, tail=20), cases.portions(reqs), mixed_steps):
            rows = run_steps(eng, steps)
            eng.cache.check()
            assert all(eng.cache.groups[i].pool.num_free == eng.cache.groups[i].pool.num_pages for i in eng.cache.paged)
            assert len(eng.cache.free_slots) == 3
            compare(rows, ref, reqs, tol, strict)
            if cuts_agree and base is not None:
                agree(rows, base, ref, tol if strict else 2e-2)
            base = base or rows


@pytest.mark.parametrize("device,dtype,name", CASES)
def test_first_tokens_and_token_by_token(dirs, refs, device, dtype, name):
    """A whole request one token a step: nothing before position 0 (a window and a convolution that reach before the start,
    a recurrence that starts from zero, a history of one layer)."""
    page = CONFIGS[name][2]
    for key, strict, _ in variants(name, dtype):
        reqs, ref = refs[key]
        rid, toks = max(reqs.items(), key=lambda kv: len(kv[1]) if len(kv[1]) <= 40 else 0)
        eng = make_engine(dirs[key], dtype, page, 16, device=device, max_num_seqs=2)
        rows = run_steps(eng, [([(rid, toks[i:i + 1], [0])], []) for i in range(len(toks))])
        compare(rows, ref, {rid: toks}, FP32_TOL if dtype == "float32" else BF16_TOL, strict)


# every mechanism alone: models of one layer (two where a layer borrows), float32, every way of cutting
SINGLE = {
    "window": config(32, 50, 1e-5, 1.5, [layer("attention", attention(4, 2, 8, 12, 0.9, window=7), None)]),
    "causal": config(32, 50, 1e-5, 1.0, [layer("attention", attention(2, 1, 16, 8, 0.9), None)]),
    "borrow": config(32, 50, 1e-5, 2.0, [layer("attention", attention(2, 2, 8, 8, 0.9, window=3), None),
                                         layer("attention", attention(4, 2, 8, 8, 0.7, window=9, kv_from=0), None)]),
    "sink": config(32, 50, 1e-5, 3.0, [layer("attention_2", sink_attention(4, 2, 8, 0.9, 6, base=100.0, scaling=(8.0, 16, 4.0, 1.0)), None)]),
    "parallel": config(24, 50, 1e-5, 0.7, [layer("parallel", parallel(2, 1, 8, 8, 0.9, 6, 4, 16, 2, 4, base=30.0, scaling=(2.0, 1.0, 3.0, 8)), None)]),
    "dense": config(24, 50, 1e-5, 1.0, [layer("attention", attention(1, 1, 8, 8, 0.5, window=2), dense(40))]),
    "routed": config(24, 50, 1e-5, 1.0, [layer("attention", attention(1, 1, 8, 8, 0.5, window=2), moe(6, 3, 12, 0.8))]),
}


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=GPU)])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, device, name):
    cfg = SINGLE[name]
    d = write_model(cfg, str(tmp_path / name), 7)
    reqs = cases.requests_for(cfg["vocab"], [1, 2, 8, 19, 45], 3)
    c, w = plain.read_model_dir(d)
    ref = {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()}
    mixed_steps, peak = cases.mixed(reqs, live=2, seed=5)
    eng = make_engine(d, "float32", 4, peak // 4, device=device, max_num_seqs=2, max_num_batched_tokens=peak)
    for steps in (cases.whole(reqs), cases.last_one_by_one(reqs, tail=12), cases.portions(reqs), mixed_steps):
        compare(run_steps(eng, steps), ref, reqs, FP32_TOL)
        eng.cache.check()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_long_decoding(dirs, dtype, name):
    """A short prompt, then hundreds of tokens one by one through many windows and pages, the recurrence carried all the way."""
    cfg, seed, page = CONFIGS[name]
    total = 330
    for key, strict, _ in variants(name, dtype):
        reqs = cases.requests_for(cfg["vocab"], [total], seed + 20)
        c, w = plain.read_model_dir(dirs[key])
        ref = {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()}
        eng = make_engine(dirs[key], dtype, page, -(-total // page) + 1, max_num_seqs=2)
        compare(run_steps(eng, cases.last_one_by_one(reqs, tail=total - 21)), ref, reqs, FP32_TOL if dtype == "float32" else BF16_TOL, strict)


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_float32_cuts_agree_closely(dirs, refs, name):
    reqs, _ = refs[name]
    eng = make_engine(dirs[name], "float32", CONFIGS[name][2], 128, max_num_seqs=8)
    a, b = run_steps(eng, cases.whole(reqs)), run_steps(eng, cases.portions(reqs))
    assert max(rel_err(b[k], a[k]) for k in a) < 1e-5


@pytest.mark.gpu
def test_long_portions_walk_the_recurrence_in_segments(dirs, refs):
    """A prompt of several hundred tokens in one step (the recurrence runs in segments with a second pass) against the same prompt
    in small portions (one walk per portion)."""
    cfg, seed, page = CONFIGS["C"]
    reqs = cases.requests_for(cfg["vocab"], [300, 129], seed + 30)
    c, w = plain.read_model_dir(dirs["C"])
    ref = {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()}
    eng = make_engine(dirs["C"], "float32", page, 64, max_num_seqs=2, max_num_batched_tokens=512)
    whole = run_steps(eng, [([(rid, toks, list(range(len(toks)))) for rid, toks in reqs.items()], list(reqs))])
    compare(whole, ref, reqs, FP32_TOL)
    agree(run_steps(eng, cases.portions(reqs)), whole, ref, 1e-5)


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=GPU)])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_llm(dirs, device, name):
    """Prompts of unequal length generate together through the scheduler (small token budget: prompts are cut into portions,
    the pool is small enough that requests wait; on the GPU decode steps replay from CUDA graphs); float32 must choose the
    plain implementation's tokens."""
    from iitj_llm_coopt_b200 import LLM, SamplingParams
    cfg, seed, page = CONFIGS[name]
    c, w = plain.read_model_dir(dirs[name])
    v = cfg["vocab"]
    prompts = [[5, 17, 3, v - 1, 9], [i % v for i in range(40, 77)], [v // 2], [i % v for i in range(20, 39)]]
    want = [plain.greedy(c, w, p, 8) for p in prompts]
    kernels = None
    if device == "cpu":
        from torch_kernels import TorchKernels
        kernels = TorchKernels()
    llm = LLM(dirs[name], dtype="float32", page_size=page, num_pages=128 // page, max_num_seqs=3, max_num_batched_tokens=24,
              device=device, kernels=kernels)
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert [o.token_ids for o in outs] == want


@pytest.mark.gpu
def test_trace_replay_program_and_command_line(dirs, tmp_path):
    """`bin/trace_run` as a subprocess on a Mamusun folder (mixed steps over a small pool), and the serving command line with
    greedy sampling: both against the plain implementation."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, seed, page = CONFIGS["A"]
    reqs, ref = cases.requests_for(cfg["vocab"], [3, 40, 17, 70], seed + 60), {}
    c, w = plain.read_model_dir(dirs["A"])
    steps, peak = cases.mixed(reqs, live=3, seed=4)
    out = tmp_path / "logits"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dirs["A"], "--dtype", "float32", "--out", str(out),
                           "--max-tokens", str(peak), "--max-requests", "3"], input="\n".join(cases.as_jsonl(steps)) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    done = {rid: 0 for rid in reqs}
    for i, (entries, _) in enumerate(steps):
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]).copy())
        r = 0
        for rid, toks, want in entries:
            if rid not in ref:
                ref[rid] = plain.forward(c, w, reqs[rid]).float()
            for j in want:
                assert rel_err(got[r], ref[rid][done[rid] + j]) < FP32_TOL
                r += 1
            done[rid] += len(toks)
    prompts = list(reqs.values())
    work, res_path = tmp_path / "w.jsonl", tmp_path / "res.json"
    work.write_text("\n".join(json.dumps({"id": f"p{i}", "prompt_token_ids": p, "max_tokens": 4 + i}) for i, p in enumerate(prompts)))
    proc = subprocess.run([sys.executable, "-m", "iitj_llm_coopt_b200.cli", "--model", dirs["A"], "--workload", str(work), "--out", str(res_path),
                           "--num-pages", "32", "--page-size", str(page), "--max-num-seqs", "3", "--max-num-batched-tokens", "48",
                           "--dtype", "float32", "--save-tokens"], cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(res_path.read_text())
    assert res["summary"]["completed"] == len(prompts) and res["summary"]["failed"] == 0
    for i, (p, rec) in enumerate(zip(prompts, res["requests"])):
        assert rec["token_ids"] == plain.greedy(c, w, p, 4 + i), i
