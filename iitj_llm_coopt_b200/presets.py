"""Named model shapes: the config.json of a model folder, as data, for runs with random weights.

Each entry holds exactly the keys a config.json of that model would hold; nothing in the engine reads a size
from here (the typed configuration is built from the dict as it would be from a file).  The benchmark, the
command line (`--shape NAME --random-seed S` in place of `--model DIR`) and the tests use them.
"""
from __future__ import annotations

import copy

_LLAMA3_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                   "original_max_position_embeddings": 8192}

LLAMA_3_1_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_SCALING),
    "tie_word_embeddings": False, "max_position_embeddings": 131072, "eos_token_id": 128001,
}
LLAMA_3_2_3B = dict(LLAMA_3_1_8B, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
                    head_dim=128, tie_word_embeddings=True, rope_scaling=dict(_LLAMA3_SCALING, factor=32.0))
LLAMA_3_2_1B = dict(LLAMA_3_2_3B, hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, head_dim=64)

# the two tiny test shapes (they differ in every size and option)
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "vocab_size": 256, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "eos_token_id": 0,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "vocab_size": 320, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": dict(_LLAMA3_SCALING, original_max_position_embeddings=64),
    "tie_word_embeddings": True, "max_position_embeddings": 512, "eos_token_id": [1, 2],
}
# a small shape for trying a benchmark out in seconds
TOY = dict(LLAMA_3_1_8B, hidden_size=512, intermediate_size=1408, num_hidden_layers=2, num_attention_heads=8,
           num_key_value_heads=2, head_dim=64, vocab_size=4096)



def lifusun_shape(width, inner, heads, kv_heads, head_dim, vocab, blocks, chunk=64, taps=4, retention_heads=None,
                  retention_value_dim=None) -> dict:
    """A Lifusun config.json of `blocks` groups of four layers (retention, attention with keys and values of its own,
    retention, attention that borrows them), with the layer sizes of a Llama of the same width: for runs with random
    weights beside that Llama."""
    rh = retention_heads or heads
    rv = retention_value_dim or head_dim
    mlp = {"kind": "dense", "ff": inner}
    layers = []
    for b in range(blocks):
        ret = {"heads": rh, "dim": head_dim, "vdim": rv, "rot": {"dims": head_dim, "base": 1000000.0},
               "decay": [1.0 - 2.0 ** (-5 - 7 * h / max(rh - 1, 1)) for h in range(rh)]}
        att = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
               "conv": taps, "mask": {"size": chunk}}
        layers += [{"type": "retention", "mixer": dict(ret), "mlp": dict(mlp)},
                   {"type": "attention", "mixer": dict(att), "mlp": dict(mlp)},
                   {"type": "retention", "mixer": dict(ret), "mlp": dict(mlp)},
                   {"type": "attention", "mixer": dict(att, kv_from=4 * b + 1), "mlp": dict(mlp)}]
    return {"architecture": "Lifusun", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "layers": layers}


# Lifusun at the layer sizes of the Llama shapes above (8 layers each; a Llama cut to 8 layers stands beside them)
LIFUSUN_8B = lifusun_shape(4096, 14336, 32, 8, 128, 128256, blocks=2)
LIFUSUN_3B = lifusun_shape(3072, 8192, 24, 8, 128, 128256, blocks=2)
LIFUSUN_1B = lifusun_shape(2048, 8192, 32, 8, 64, 128256, blocks=2)
LIFUSUN_TOY = lifusun_shape(512, 1408, 8, 2, 64, 4096, blocks=1)

def rodapel_shape(width, inner, heads, kv_heads, head_dim, vocab, blocks, window=4096, kv_rank=512, rot_dim=64, experts=8,
                  identity=2, top=2, wkv_head=64, decay_rank=64) -> dict:
    """A Rodapel config.json of `blocks` groups of four layers (windowed attention with a dense feed-forward, then latent
    attention, wkv and windowed attention with routed ones), with the layer sizes of a Llama of the same width: for runs
    with random weights beside that Llama.  A routed layer holds `experts` experts of half the dense inner width, of
    which a token uses `top`: as much arithmetic per token as the dense layer, `experts` / 2 times its weights."""
    att = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "mask": {"size": window}}
    lat = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank,
           "scale": (head_dim + rot_dim) ** -0.5, "rot": {"dims": rot_dim, "base": 1000000.0}}
    rec = {"heads": width // wkv_head, "dim": wkv_head, "decay_rank": decay_rank}
    dense = {"kind": "dense", "ff": inner, "limit": 7.0}
    routed = {"kind": "moe", "expert": {"ff": inner // 2, "limit": 7.0}, "router": {"experts": experts, "identity": identity, "top": top}}
    layers = []
    for _ in range(blocks):
        layers += [{"type": "attention", "mixer": dict(att), "mlp": dict(dense)},
                   {"type": "latent_attention", "mixer": copy.deepcopy(lat), "mlp": copy.deepcopy(routed)},
                   {"type": "wkv", "mixer": dict(rec), "mlp": copy.deepcopy(routed)},
                   {"type": "attention", "mixer": dict(att), "mlp": copy.deepcopy(routed)}]
    return {"architecture": "Rodapel", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "layers": layers}


# Rodapel at the layer sizes of the Llama shapes above (8 layers each)
RODAPEL_8B = rodapel_shape(4096, 14336, 32, 8, 128, 128256, blocks=2)
RODAPEL_3B = rodapel_shape(3072, 8192, 24, 8, 128, 128256, blocks=2)
RODAPEL_1B = rodapel_shape(2048, 8192, 32, 8, 64, 128256, blocks=2)
RODAPEL_TOY = rodapel_shape(512, 1408, 8, 2, 64, 4096, blocks=1, window=256, kv_rank=128, rot_dim=32, experts=4, identity=1)


def fomerax_shape(width, inner, heads, kv_heads, head_dim, vocab, blocks, window=1024, kv_rank=512, rot_dim=64, q_rank=1536,
                  experts=8, top=2, side_dim=256) -> dict:
    """A Fomerax config.json of `blocks` groups of four layers (windowed latent attention with a dense feed-forward, biased
    attention with routed ones, latent attention with routed ones, biased attention with a dense one), every layer with a
    token input of `side_dim` columns, at the layer sizes of a Llama of the same width: for runs with random weights beside
    the Rodapel and the Llama of that size.  A routed layer holds `experts` experts of half the dense inner width."""
    lat = {"heads": heads, "dim": head_dim, "rot_dim": rot_dim, "vdim": head_dim, "kv_rank": kv_rank, "q_rank": q_rank,
           "scale": (head_dim + rot_dim) ** -0.5, "mask": {"size": window},
           "rot": {"dims": rot_dim, "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "softcap": 50.0,
           "q_temp": {"coef": 0.1, "every": 8192}}
    dense = {"kind": "dense", "ff": inner}
    routed = {"kind": "moe", "expert": {"ff": inner // 2}, "router": {"experts": experts, "top": top}}
    layers = []
    for _ in range(blocks):
        layers += [{"type": "latent_attention", "mixer": copy.deepcopy(lat), "mlp": dict(dense)},
                   {"type": "attention", "mixer": copy.deepcopy(att), "mlp": copy.deepcopy(routed)},
                   {"type": "latent_attention", "mixer": copy.deepcopy(lat), "mlp": copy.deepcopy(routed)},
                   {"type": "attention", "mixer": copy.deepcopy(att), "mlp": dict(dense)}]
    return {"architecture": "Fomerax", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "token_side": {"dim": side_dim},
            "layers": layers}


# Fomerax at the layer sizes of the Llama shapes above (8 layers each)
FOMERAX_8B = fomerax_shape(4096, 14336, 32, 8, 128, 128256, blocks=2)
FOMERAX_3B = fomerax_shape(3072, 8192, 24, 8, 128, 128256, blocks=2, q_rank=1024)
FOMERAX_1B = fomerax_shape(2048, 8192, 32, 8, 64, 128256, blocks=2, q_rank=768, side_dim=128)
FOMERAX_TOY = fomerax_shape(512, 1408, 8, 2, 64, 4096, blocks=1, window=128, kv_rank=128, rot_dim=32, q_rank=192, experts=4, side_dim=32)

def mamusun_shape(width, inner, heads, kv_heads, head_dim, vocab, blocks, window=1024, experts=8, top=2, lru_blocks=16, taps=4,
                  alpha=2.0) -> dict:
    """A Mamusun config.json of `blocks` groups of four layers (sink attention with a dense feed-forward, window attention with
    routed ones, window attention beside a gated recurrence with a dense one, window attention on the second layer's keys and
    values with routed ones) at the layer sizes of a Llama of the same width: for runs with random weights beside the Rodapel and
    the Llama of that size.  A routed layer holds `experts` experts of half the dense inner width; the recurrence is as wide as
    the model."""
    sink = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5,
            "rot": {"dims": head_dim, "base": 500000.0, "scaling": {"factor": 16.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
    att = {"heads": heads, "kv_heads": kv_heads, "dim": head_dim, "vdim": head_dim, "scale": head_dim ** -0.5, "mask": {"size": window}}
    left = dict(att, rot={"dims": head_dim // 2, "base": 50000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 2.0, "original": 8192}})
    par = {"left": left, "right": {"width": width, "blocks": lru_blocks, "conv": taps}}
    dense = {"kind": "dense", "ff": inner}
    routed = {"kind": "moe", "expert": {"ff": inner // 2, "limit": 7.0}, "router": {"experts": experts, "top": top}}
    layers = []
    for b in range(blocks):
        layers += [{"type": "attention_2", "mixer": copy.deepcopy(sink), "mlp": dict(dense)},
                   {"type": "attention", "mixer": copy.deepcopy(att), "mlp": copy.deepcopy(routed)},
                   {"type": "parallel", "mixer": copy.deepcopy(par), "mlp": dict(dense)},
                   {"type": "attention", "mixer": dict(copy.deepcopy(att), kv_from=4 * b + 1), "mlp": copy.deepcopy(routed)}]
    return {"architecture": "Mamusun", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "postln_alpha": alpha, "layers": layers}


# Mamusun at the layer sizes of the Llama shapes above (8 layers each)
MAMUSUN_8B = mamusun_shape(4096, 14336, 32, 8, 128, 128256, blocks=2)
MAMUSUN_3B = mamusun_shape(3072, 8192, 24, 8, 128, 128256, blocks=2, lru_blocks=12)
MAMUSUN_1B = mamusun_shape(2048, 8192, 32, 8, 64, 128256, blocks=2, lru_blocks=8)
MAMUSUN_TOY = mamusun_shape(512, 1408, 8, 2, 64, 4096, blocks=1, window=128, experts=4, lru_blocks=4)

# name -> (label used in reports, config.json dict)
SHAPES = {
    "8b": ("llama-3.1-8b-shape-random", LLAMA_3_1_8B),
    "3b": ("llama-3.2-3b-shape-random", LLAMA_3_2_3B),
    "1b": ("llama-3.2-1b-shape-random", LLAMA_3_2_1B),
    "tinyA": ("llama-tiny-a-shape-random", TINY_A),
    "tinyB": ("llama-tiny-b-shape-random", TINY_B),
    "toy": ("llama-toy-shape-random", TOY),
    "lifusun-8b": ("lifusun-8b-layers-random", LIFUSUN_8B),
    "lifusun-3b": ("lifusun-3b-layers-random", LIFUSUN_3B),
    "lifusun-1b": ("lifusun-1b-layers-random", LIFUSUN_1B),
    "lifusun-toy": ("lifusun-toy-layers-random", LIFUSUN_TOY),
    "rodapel-8b": ("rodapel-8b-layers-random", RODAPEL_8B),
    "rodapel-3b": ("rodapel-3b-layers-random", RODAPEL_3B),
    "rodapel-1b": ("rodapel-1b-layers-random", RODAPEL_1B),
    "rodapel-toy": ("rodapel-toy-layers-random", RODAPEL_TOY),
    "fomerax-8b": ("fomerax-8b-layers-random", FOMERAX_8B),
    "fomerax-3b": ("fomerax-3b-layers-random", FOMERAX_3B),
    "fomerax-1b": ("fomerax-1b-layers-random", FOMERAX_1B),
    "fomerax-toy": ("fomerax-toy-layers-random", FOMERAX_TOY),
    "mamusun-8b": ("mamusun-8b-layers-random", MAMUSUN_8B),
    "mamusun-3b": ("mamusun-3b-layers-random", MAMUSUN_3B),
    "mamusun-1b": ("mamusun-1b-layers-random", MAMUSUN_1B),
    "mamusun-toy": ("mamusun-toy-layers-random", MAMUSUN_TOY),
}


def shape_config(name: str) -> dict:
    """A fresh copy of the config.json dict of shape `name`."""
    if name not in SHAPES:
        raise KeyError(f"shape {name!r} is not known; known: {', '.join(sorted(SHAPES))}")
    return copy.deepcopy(SHAPES[name][1])
