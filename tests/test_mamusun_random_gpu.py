"""Mamusun configurations drawn at random from fixed seeds (layer orders and counts, the three mixers, head counts and groupings, key
and value sizes, rotated parts from two numbers to the whole head, scaled frequencies or none, windows from one token to longer than
the prompts or none, layers that borrow the keys and values of an earlier layer under a window of their own, recurrences of one to
many blocks and two to five taps, expert counts and choices, layers without a feed-forward, residual factors, widths and vocabularies
that are no multiples of 8, page sizes), each through the engine in float32 and bfloat16, whole, in portions and in mixed batches over
reused pages and slots, against the plain restatement.  Sizes that are multiples of 16 take the tensor-core attention in bfloat16, the
others the one-warp-per-row form; both are drawn.

The matrices are scaled by the inverse root of their input width, so scores and activations are of order one as in a trained model:
float32 is then compared at (nearly) every position (99 positions in 100 within 3e-4 and all within 1e-2 leaves room for a router's
close call), bfloat16 by its median and ninth decile, and the ways of cutting must agree with one another (in bfloat16 only without
routed layers, where a close call of the router moves a whole request)."""
import random

import pytest
import torch

import plain_mamusun as plain
import replay_cases as cases
from helpers import make_engine, run_steps
from mamusun_models import attention, config, dense, layer, make_tensors, moe, parallel, sink_attention, write_model
from test_mamusun_engine import agree, errors

pytestmark = pytest.mark.gpu

WINDOWS = [None, 1, 2, 7, 16, 17, 50, 64, 96, 128, 200, 1000]


def draw(seed):
    rng = random.Random(seed)
    width = rng.choice([64, 96, 100, 128, 192, 256, 384])
    layers, lenders = [], []
    for i in range(rng.randint(2, 7)):
        pick = rng.random()
        if pick < 0.4:
            if lenders and rng.random() < 0.4:
                src = rng.choice(lenders)
                o = layers[src]["mixer"]
                m = attention(o["kv_heads"] * rng.choice([1, 2, 4]), o["kv_heads"], o["dim"], o["vdim"], o["dim"] ** -0.5 * rng.choice([1.0, 2.0]),
                              window=rng.choice(WINDOWS), kv_from=src)
            else:
                kv, dim = rng.choice([1, 2, 3, 4]), rng.choice([8, 16, 32, 48, 64, 128])
                m = attention(kv * rng.choice([1, 2, 4, 8]), kv, dim, rng.choice([8, 16, 32, 40, 80, 96, 128]), dim ** -0.5 * rng.choice([1.0, 2.0]),
                              window=rng.choice(WINDOWS))
                lenders.append(i)
            kind = "attention"
        elif pick < 0.7:
            kv, dim = rng.choice([1, 2, 3, 8]), rng.choice([8, 16, 32, 64, 96, 128])
            scaling = rng.choice([None, (rng.choice([2.0, 8.0, 32.0]), rng.choice([16, 64, 1024]), rng.choice([32.0, 8.0]), rng.choice([1.0, 2.0]))])
            m = sink_attention(kv * rng.choice([1, 2, 4]), kv, dim, dim ** -0.5 * rng.choice([1.0, 2.0]), rng.choice([2, 4, 8, dim]),
                               base=rng.choice([100.0, 1e4, 5e5]), scaling=scaling)
            kind = "attention_2"
        else:
            kv, dim = rng.choice([1, 2, 3]), rng.choice([8, 16, 32, 64, 128])
            blocks = rng.choice([1, 2, 4, 8])
            scaling = rng.choice([None, (rng.choice([4.0, 8.0]), 1.0, rng.choice([2.0, 4.0]), rng.choice([16, 256]))])
            m = parallel(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([8, 16, 32, 64, 128]), dim ** -0.5 * rng.choice([1.0, 2.0]),
                         rng.choice(WINDOWS), rng.choice([2, 4, 8, dim]), blocks * rng.choice([3, 8, 16, 40, 64]), blocks, rng.choice([2, 3, 4, 5]),
                         base=rng.choice([100.0, 1e4]), scaling=scaling)
            kind = "parallel"
        pick = rng.random()
        if pick < 0.15:
            mlp = None
        elif pick < 0.55:
            mlp = dense(rng.choice([40, 64, 128, 384]))
        else:
            experts = rng.choice([1, 2, 4, 8, 12, 16])
            mlp = moe(experts, rng.randint(1, min(4, experts)), rng.choice([16, 32, 64, 128]), rng.choice([0.5, 1.0, 7.0]))
        layers.append(layer(kind, m, mlp))
    cfg = config(width, rng.choice([64, 131, 300, 1000]), rng.choice([1e-5, 1e-6]), rng.choice([1.0, 2.0, 3.0, 0.5]), layers)
    return cfg, rng.choice([4, 8, 16, 32])


def trained_like(cfg, seed):
    """Random tensors of the family's writer with every matrix scaled by the inverse root of its input width."""
    t = make_tensors(cfg, seed)
    for name, w in t.items():
        if w.dim() >= 2 and name != "embed" and not name.endswith(".conv"):
            f = w.float()
            t[name] = (f / f.std().clamp_min(1e-6) * w.shape[-1] ** -0.5).to(torch.bfloat16).contiguous()
    return t


@pytest.mark.parametrize("seed", range(500, 512))
def test_random_configuration(tmp_path, seed):
    cfg, page = draw(seed)
    d = write_model(cfg, str(tmp_path / "m"), seed, tensors=trained_like(cfg, seed))
    c, w = plain.read_model_dir(d)
    reqs = cases.requests_for(cfg["vocab"], [1, 19, 66, 150, 300], seed)
    ref = {rid: plain.forward(c, w, toks).float() for rid, toks in reqs.items()}
    mixed_steps, peak = cases.mixed(reqs, live=3, seed=seed, decode_tail=12)
    routed = any(l["mlp"] is not None and l["mlp"]["kind"] == "moe" for l in cfg["layers"])
    for dtype, tol in (("float32", 3e-4), ("bfloat16", 5e-2)):
        eng = make_engine(d, dtype, page, max(peak // page, 1), max_num_seqs=3, max_num_batched_tokens=peak)
        base = None
        for steps in (cases.whole(reqs), cases.portions(reqs), mixed_steps):
            rows = run_steps(eng, steps)
            eng.cache.check()
            e = sorted(errors(rows, ref, reqs))
            if dtype == "float32":
                assert e[int(0.99 * (len(e) - 1))] <= tol and e[-1] <= 1e-2, (seed, e[int(0.99 * (len(e) - 1))], e[-1])
            else:
                assert e[len(e) // 2] <= tol and e[int(0.9 * (len(e) - 1))] <= 3 * tol, (seed, e[len(e) // 2], e[int(0.9 * (len(e) - 1))])
            if base is not None and (dtype == "float32" or not routed):
                agree(rows, base, ref, tol if dtype == "float32" else 2e-2)
            base = base or rows
