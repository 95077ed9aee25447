"""The Fomerax family through the engine's step function, cache manager and entry points, against the plain restatement
of tests/plain_fomerax.py: every way of cutting the same requests into steps (whole, the last tokens one by one, portions
down to two tokens, mixed batches over a pool so small that pages and slots are used again), the first tokens, long
decoding across many windows and pages, and greedy generation through `LLM.generate`.
CPU cases run the host logic with the plain-torch kernel double; `-m gpu` cases run the CUDA kernels.

bfloat16 and routed experts.  A token whose best router scores lie closer together than bfloat16 rounding moves them may
pick another expert than the float64 restatement does, and everything after it in the request then differs by far more
than rounding.  So in bfloat16 the configurations run with softer attention scales, once with their routed feed-forwards
replaced by dense ones of the same sizes (`soft_variant`: there the ways of cutting must also agree with one another) and
once as they are; both under bounds on the median and the ninth decile of the error.  float32 is compared at every
position, with the configurations as they are."""
import copy

import pytest
import torch

import plain_fomerax as plain
import replay_cases as cases
from fomerax_models import CONFIGS, write_model
from helpers import make_engine, rel_err, run_steps

FP32_TOL, BF16_TOL = 3e-4, 5e-2
# lengths around every window (10, 1, 33, 16, 70, 2) and page size (16, 8, 16, 4) of the configurations
LENGTHS = {"A": [1, 9, 10, 11, 33, 70], "B": [2, 31, 32, 33, 34, 35, 97, 130], "C": [3, 16, 17, 40, 75], "D": [7, 15, 16, 17, 69, 70, 71, 130]}

GPU = pytest.mark.gpu
CASES = [pytest.param("cpu", "float32", n, id=f"cpu-fp32-{n}") for n in "ABCD"] + \
        [pytest.param("cuda:0", dt, n, marks=GPU, id=f"gpu-{dt}-{n}") for dt in ("float32", "bfloat16") for n in "ABCD"]


def soft_variant(cfg, dense=True):
    """Attention scales a quarter as large (a peaked softmax magnifies bfloat16's rounding of queries and keys far beyond a
    rounding-sized tolerance) and, with `dense`, dense feed-forwards in place of the routed ones."""
    cfg = copy.deepcopy(cfg)
    for lay in cfg["layers"]:
        lay["mixer"]["scale"] *= 0.25
        if dense and lay["mlp"] is not None and lay["mlp"]["kind"] == "moe":
            lay["mlp"] = {"kind": "dense", "ff": lay["mlp"]["expert"]["ff"]}
    return cfg


def has_experts(name):
    return any(l["mlp"] is not None and l["mlp"]["kind"] == "moe" for l in CONFIGS[name][0]["layers"])


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for name, (cfg, seed, _) in CONFIGS.items():
        out[name] = write_model(cfg, str(tmp_path_factory.mktemp(f"fom_{name}")), seed)
        out[name + "-dense"] = write_model(soft_variant(cfg), str(tmp_path_factory.mktemp(f"fom_{name}_dense")), seed)
        out[name + "-soft"] = write_model(soft_variant(cfg, dense=False), str(tmp_path_factory.mktemp(f"fom_{name}_soft")), seed)
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
    """float32 (`strict`): every position within `tol`.  bfloat16: the median within `tol` and nine positions in ten
    within twice that: the configurations are ill-conditioned on purpose (peaked softmax, norms that bring a small branch
    back to full size), so single positions magnify bfloat16's rounding whatever the kernels do."""
    e = sorted(errors(rows, ref, reqs))
    if strict:
        assert e[-1] <= tol, e[-1]
    else:
        assert e[len(e) // 2] <= tol and e[int(0.9 * (len(e) - 1))] <= 2 * tol, (e[len(e) // 2], e[int(0.9 * (len(e) - 1))], e[-1])


def agree(rows, base, ref, tol):
    """Two ways of cutting the same requests give the same logits (relative to each request's largest logit)."""
    worst = max(((rows[k].float() - base[k].float()).abs().max() / ref[k[0]].abs().max()).item() for k in base)
    assert worst <= tol, worst


def variants(name, dtype):
    """(model key, compared at every position, whether different cuts must agree closely) for a configuration and type."""
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
    """A whole request one token a step: nothing before position 0 (a window that reaches before the start, a query
    temperature whose first period has not ended, a distance of zero)."""
    page = CONFIGS[name][2]
    for key, strict, _ in variants(name, dtype):
        reqs, ref = refs[key]
        rid, toks = max(reqs.items(), key=lambda kv: len(kv[1]) if len(kv[1]) <= 40 else 0)
        eng = make_engine(dirs[key], dtype, page, 16, device=device, max_num_seqs=2)
        rows = run_steps(eng, [([(rid, toks[i:i + 1], [0])], []) for i in range(len(toks))])
        compare(rows, ref, {rid: toks}, FP32_TOL if dtype == "float32" else BF16_TOL, strict)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_long_decoding(dirs, dtype, name):
    """A short prompt, then hundreds of tokens one by one through many windows, pages and temperature periods."""
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
    eng = make_engine(dirs[name], "float32", CONFIGS[name][2], 128, max_num_seqs=4)
    a, b = run_steps(eng, cases.whole(reqs)), run_steps(eng, cases.portions(reqs))
    assert max(rel_err(b[k], a[k]) for k in a) < 1e-5


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda:0", marks=GPU)])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_llm(dirs, device, name):
    """Prompts of unequal length generate together through the scheduler (small token budget: prompts are cut into
    portions, the pool is small enough that requests wait; on the GPU decode steps replay from CUDA graphs); float32 must
    choose the plain implementation's tokens."""
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
def test_command_line_serves_a_model_folder(dirs, tmp_path):
    """The serving command line on a Fomerax folder (continuous batching under a small token budget, float32, greedy): every
    request's ids equal the plain implementation's; and on a named shape of the family with random weights, sampled."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, seed, page = CONFIGS["B"]
    prompts = list(cases.requests_for(cfg["vocab"], [3, 40, 17, 70, 5], seed + 60).values())
    work, out = tmp_path / "w.jsonl", tmp_path / "res.json"
    work.write_text("\n".join(json.dumps({"id": f"p{i}", "prompt_token_ids": p, "max_tokens": 5 + i}) for i, p in enumerate(prompts)))
    proc = subprocess.run([sys.executable, "-m", "iitj_llm_coopt_b200.cli", "--model", dirs["B"], "--workload", str(work), "--out", str(out),
                           "--num-pages", "64", "--page-size", str(page), "--max-num-seqs", "3", "--max-num-batched-tokens", "48",
                           "--dtype", "float32", "--save-tokens"], cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(out.read_text())
    assert res["summary"]["completed"] == len(prompts) and res["summary"]["failed"] == 0
    c, w = plain.read_model_dir(dirs["B"])
    for i, (p, rec) in enumerate(zip(prompts, res["requests"])):
        assert rec["token_ids"] == plain.greedy(c, w, p, 5 + i), i
    proc = subprocess.run([sys.executable, "-m", "iitj_llm_coopt_b200.cli", "--shape", "fomerax-toy", "--random-seed", "5", "--workload",
                           "synthetic:10:4-300:3-20", "--out", str(out), "--num-pages", "128", "--max-num-seqs", "4",
                           "--max-num-batched-tokens", "64", "--save-tokens"], cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(out.read_text())
    assert res["summary"]["completed"] == 10 and res["summary"]["failed"] == 0
    assert all(len(r["token_ids"]) == r["output_tokens"] == r["max_tokens"] for r in res["requests"])
