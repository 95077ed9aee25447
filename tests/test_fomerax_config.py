"""Fomerax's configuration, its layers as data, its checkpoint names, and the trace replay's protocol on a Fomerax folder (CPU)."""
import copy
import io
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_fomerax as plain
from fomerax_models import CONFIGS, FOM_A, FOM_B, FOM_C, make_tensors, write_model

from iitj_llm_coopt_b200.config import ConfigError, load_config
from iitj_llm_coopt_b200.config.fomerax import FomeraxConfig
from iitj_llm_coopt_b200.models.decoder import cache_needs
from iitj_llm_coopt_b200.weights.loader import WeightError, expected_tensors


def test_layers_as_data(tmp_path):
    d = write_model(FOM_A, str(tmp_path / "m"), 1)
    arch, typed = load_config(d)
    assert arch.name == "Fomerax"
    spec = typed.model_spec()
    assert [c.cache for c in spec.order] == [0, 1, 2, 3] and all(c.write and c.state is None for c in spec.order)
    assert [l.arrangement for l in spec.layers] == ["sandwich_side", "sandwich_side", "sandwich_mixer_side", "sandwich_side"]
    needs = cache_needs(spec)
    # latent rows: one shared head of kv_rank + rot_dim numbers whose leading kv_rank are the values; the window is the layer's
    assert needs[0].kind == "paged_kv" and needs[0].shared_value
    assert (needs[0].kv_heads, needs[0].head_dim, needs[0].value_dim, needs[0].window) == (1, 32, 24, 10)
    assert (needs[1].kv_heads, needs[1].head_dim, needs[1].value_dim, needs[1].window) == (2, 16, 24, 0)
    assert (needs[2].head_dim, needs[2].value_dim, needs[2].window) == (56, 40, 1)
    m0, m1, m3 = (spec.layers[i].part("mixer") for i in (0, 1, 3))
    assert m0.kind == "latent_attention" and dict(m0.options)["q_rank"] == 20 and m0.softmax_scale == 0.5
    assert m0.position.pairing == "interleaved" and m0.position.rotary_dim == 8 and dict(m0.position.scaling)["factor"] == 4.0
    assert m1.kind == "gated_attention" and dict(m1.options)["q_temp"] == (0.3, 7) and dict(m1.options)["softcap"] == 6.0
    assert dict(m3.options)["q_temp"] is None and dict(m3.options)["softcap"] == 0.0
    f0, f1 = spec.layers[0].part("feed_forward"), spec.layers[1].part("feed_forward")
    assert (f0.kind, f0.experts, f0.experts_per_token, f0.inner) == ("routed_glu", 5, 2, 20)
    assert (f1.kind, f1.activation, f1.inner) == ("glu", "gelu_tanh", 48)
    sides = [spec.layers[i].part("token_input") for i in range(4)]
    assert [(s.dim, s.offset, s.table_width) for s in sides] == [(8, 0, 32), (8, 8, 32), (8, 16, 32), (8, 24, 32)]
    assert spec.tie_embeddings and spec.embedding.kind == "table_side"
    b = FomeraxConfig.from_dict(FOM_B).model_spec()
    assert b.embedding.kind == "table" and [l.arrangement for l in b.layers] == ["sandwich"] * 3
    assert cache_needs(b)[0].window == 0 and b.layers[0].part("mixer").position.scaling == ()
    assert FomeraxConfig.from_dict(FomeraxConfig.from_dict(FOM_C).to_dict()).model_spec() == FomeraxConfig.from_dict(FOM_C).model_spec()


def test_checkpoint_names_are_the_family_s(tmp_path):
    for name, (cfg, seed, _) in CONFIGS.items():
        d = write_model(cfg, str(tmp_path / name), seed)
        arch, typed = load_config(d)
        want = expected_tensors(arch, arch.model_spec(typed))
        have = make_tensors(cfg, seed)
        assert set(want) == set(have)
        assert all(tuple(want[k][0]) == tuple(have[k].shape) for k in want)


@pytest.mark.parametrize("change,text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["token_side"].pop("dim"), "dim"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0].update(type="mamba"), "not known"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["layers"][1]["mlp"].pop("ff"), "ff"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "router takes"),
])
def test_bad_configurations_are_refused(change, text):
    cfg = copy.deepcopy(FOM_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        FomeraxConfig.from_dict(cfg)


def test_scaled_frequencies_of_the_position_part():
    """The rotation part's frequencies and amplitude against the plain formula, for ramps that start inside, before and
    behind the pairs, and a ramp of zero length."""
    from iitj_llm_coopt_b200.parts.position import rope_amplitude, yarn_frequencies
    for dims, base, sc in ((8, 1000.0, (4.0, 16, 8.0, 1.0)), (32, 20000.0, (8.0, 1024, 32.0, 1.0)), (4, 10000.0, (16.0, 64, 4.0, 2.0)),
                           (6, 300.0, (2.0, 8, 2.0, 0.5)), (16, 50.0, (3.0, 4096, 1.0, 1.0)), (12, 1e6, (40.0, 32, 64.0, 32.0))):
        scaling = {"factor": sc[0], "original": sc[1], "fast": sc[2], "slow": sc[3]}
        want, amp = plain.yarn_frequencies(dims, base, scaling)
        cfg = copy.deepcopy(FOM_A)
        m = cfg["layers"][0]["mixer"]
        m["rot_dim"], m["rot"] = dims, {"dims": dims, "base": base, "scaling": scaling}
        pos = FomeraxConfig.from_dict(cfg).model_spec().layers[0].part("mixer").position
        assert pos.scaling_dict()["type"] == "yarn" and (pos.rotary_dim, pos.theta) == (dims, base)
        got = yarn_frequencies(pos.rotary_dim, pos.theta, pos.scaling_dict())
        assert torch.allclose(got.double(), want, rtol=1e-6, atol=0)
        assert math.isclose(rope_amplitude(pos.scaling_dict()), amp, rel_tol=1e-12)
        assert len(set(want.tolist())) == dims // 2               # the pairs' frequencies differ


def test_missing_and_unexpected_tensors_are_listed(tmp_path):
    from helpers import make_engine
    t = make_tensors(FOM_A, 1)
    t["l0.mlp.e5.up"] = t["l0.mlp.e4.up"].clone()               # the layer has five experts: e0 .. e4
    t["l2.norm2"] = t["l2.norm1"].clone()                       # the layer has no feed-forward
    del t["l2.mix.dq.norm"], t["l1.mix.g"], t["side.embed"], t["l3.side.norm"]
    d = write_model(FOM_A, str(tmp_path / "m"), 1, tensors=t)
    with pytest.raises(WeightError) as e:
        make_engine(d, "float32", device="cpu")
    assert e.value.missing == ["l1.mix.g", "l2.mix.dq.norm", "l3.side.norm", "side.embed"]
    assert e.value.unexpected == ["l0.mlp.e5.up", "l2.norm2"]


def test_trace_replay_protocol(tmp_path):
    """bin/trace_run's program on a Fomerax folder (CPU kernel double): files only for steps that want something, a `done`
    line after every step, a request left out of a step that goes on later, two state slots that three requests share."""
    from iitj_llm_coopt_b200 import replay
    from torch_kernels import TorchKernels
    cfg, seed, page = CONFIGS["A"]
    d = write_model(cfg, str(tmp_path / "m"), seed)
    c, w = plain.read_model_dir(d)
    a, b = list(range(3, 40)), list(range(90, 111))
    lines = [json.dumps(x) for x in (
        {"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [16]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[17:19], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[2:], "want": [0, 18]}, {"id": "a", "tokens": a[19:20], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [20]}, {"id": "a", "tokens": a[20:], "want": [16]}], "end": ["a", "c"]})]
    out = io.StringIO()
    args = replay.parse_args(["--model", d, "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128",
                              "--max-requests", "2", "--device", "cpu"])
    assert replay.run(args, lines, out=out, kernels=TorchKernels()) == 0
    assert out.getvalue().split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(tmp_path / "o")) == ["0.f32", "2.f32", "3.f32"]
    ra, rb = plain.forward(c, w, a), plain.forward(c, w, b)
    got = {s: np.fromfile(tmp_path / "o" / f"{s}.f32", dtype="<f4").reshape(-1, cfg["vocab"]) for s in (0, 2, 3)}
    want = {0: [ra[16]], 2: [rb[2], rb[20], ra[19]], 3: [rb[20], ra[36]]}
    for s, rows in want.items():
        ref = torch.stack(rows).float().numpy()
        assert np.abs(got[s] - ref).max() <= 1e-4 * np.abs(ref).max()
