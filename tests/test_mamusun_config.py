"""Mamusun's configuration and checkpoint names, without a device: what the file's keys become (layers as data, cache entries, windows
that cover a borrowing layer, rotation laws), which files are refused, and that the loader finds every tensor the test writer names."""
import copy
import math

import pytest
import torch

import plain_mamusun as plain
from iitj_llm_coopt_b200.config import ConfigError
from iitj_llm_coopt_b200.config.mamusun import MamusunConfig
from iitj_llm_coopt_b200.config.registry import architecture_for, load_config
from iitj_llm_coopt_b200.models.decoder import cache_needs, model_parameter_specs
from iitj_llm_coopt_b200.parts.position import rope_inverse_frequencies, yarn_frequencies
from iitj_llm_coopt_b200.weights.loader import WeightError, checkpoint_index, expected_tensors, load_parameters
from mamusun_models import CONFIGS, make_tensors, write_model


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_writer_s_names_are_the_loader_s(tmp_path, name):
    cfg, seed, _ = CONFIGS[name]
    d = write_model(cfg, str(tmp_path / name), seed)
    arch, typed = load_config(d)
    assert arch.name == "Mamusun" and typed.to_dict() == cfg
    spec = arch.model_spec(typed)
    want = expected_tensors(arch, spec)
    index = checkpoint_index(d)
    assert set(want) == set(index)
    assert all(tuple(index[n][1]) == tuple(want[n][0]) for n in want)
    params = load_parameters(d, arch, typed, spec, torch.float32, device="cpu")
    assert set(params) == set(model_parameter_specs(spec))


def test_layers_become_cache_entries_and_calls():
    cfg, _, _ = CONFIGS["B"]
    spec = MamusunConfig.from_dict(cfg).model_spec()
    needs = cache_needs(spec)
    order = spec.order
    # layer 0 lends to layer 2 (window 23) and to layer 4 (no window): its pages keep everything
    assert order[2].cache == order[0].cache == order[4].cache and not order[2].write and not order[4].write and order[0].write
    assert needs[order[0].cache].kind == "paged_kv" and needs[order[0].cache].window == 0
    # the parallel layer: pages for its left side with the left window, a record of [taps, channels] for its right side
    par = order[1]
    assert needs[par.cache].window == 16 and needs[par.state].kind == "state" and needs[par.state].state_shape == (2, 40)
    assert len(needs) == spec.cache_entries() == 4
    a = MamusunConfig.from_dict(CONFIGS["A"][0]).model_spec()
    na = cache_needs(a)
    assert na[a.order[1].cache].window == 10 and a.order[3].cache == a.order[1].cache
    wider = copy.deepcopy(CONFIGS["A"][0])
    wider["layers"][3]["mixer"]["mask"]["size"] = 33
    w = MamusunConfig.from_dict(wider).model_spec()
    assert cache_needs(w)[w.order[1].cache].window == 33           # the lender keeps what its widest reader sees
    assert dict(w.layers[1].part("mixer").options)["cache_window"] == 33 and w.layers[1].part("mixer").window == 10


def test_rotation_laws_agree_with_the_plain_ones():
    for dims, base, sc in ((48, 20000.0, {"factor": 8.0, "low": 1.0, "high": 2.0, "original": 256}), (8, 50.0, {"factor": 8.0, "low": 1.0, "high": 2.0, "original": 16})):
        want, _ = plain.stretched_frequencies(dims, base, sc)
        got = rope_inverse_frequencies(dims, base, {"type": "llama3", "factor": sc["factor"], "low_freq_factor": sc["low"],
                                                    "high_freq_factor": sc["high"], "original_max_position_embeddings": sc["original"]})
        assert torch.allclose(got.double(), want, rtol=1e-6)
        assert not torch.allclose(want, plain.plain_frequencies(dims, base))
    sc = {"factor": 16.0, "original": 1024, "fast": 16.0, "slow": 2.0}
    want, amp = plain.ramped_frequencies(64, 500000.0, sc)
    assert torch.allclose(yarn_frequencies(64, 500000.0, sc).double(), want, rtol=1e-6) and abs(amp - (0.1 * math.log(16.0) + 1.0)) < 1e-12


def broken(change):
    cfg = copy.deepcopy(CONFIGS["A"][0])
    change(cfg)
    return cfg


@pytest.mark.parametrize("change", [
    lambda c: c.pop("postln_alpha"),
    lambda c: c["norm"].pop("eps"),
    lambda c: c["layers"][0].update(type="attention_3"),
    lambda c: c["layers"][1]["mixer"].update(heads=3),                       # heads that do not group
    lambda c: c["layers"][3]["mixer"].update(kv_from=2),                     # borrows from a layer that is no attention layer
    lambda c: c["layers"][3]["mixer"].update(kv_from=3),                     # ... or from itself
    lambda c: c["layers"][3]["mixer"].update(dim=16),                        # other key size than the lender
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][0]["mixer"].update(vdim=8),                        # values are the keys
    lambda c: c["layers"][2]["mixer"]["right"].update(blocks=5),
    lambda c: c["layers"][2]["mixer"]["left"]["rot"]["scaling"].pop("low"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=6),
    lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"),
    lambda c: c["layers"][0]["mlp"].update(kind="glu"),
    lambda c: c["layers"][1]["mixer"]["mask"].update(size=0),
])
def test_refused_configurations(change):
    with pytest.raises(ConfigError):
        MamusunConfig.from_dict(broken(change))


def test_registry_and_weight_errors(tmp_path):
    cfg, seed, _ = CONFIGS["C"]
    assert architecture_for(cfg).name == "Mamusun"
    tensors = make_tensors(cfg, seed)
    del tensors["l0.mix.right.lam"]
    tensors["l1.mix.left.out"] = tensors["l1.mix.left.out"][:-1].contiguous()
    tensors["l0.mix.k"] = tensors["l0.mix.left.k"].clone()
    d = write_model(cfg, str(tmp_path / "bad"), seed, tensors=tensors)
    arch, typed = load_config(d)
    with pytest.raises(WeightError) as e:
        load_parameters(d, arch, typed, arch.model_spec(typed), torch.float32, device="cpu")
    assert e.value.missing == ["l0.mix.right.lam"] and e.value.unexpected == ["l0.mix.k"] and [n for n, *_ in e.value.wrong_shape] == ["l1.mix.left.out"]
