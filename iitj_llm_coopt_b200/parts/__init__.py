"""The part registries: a spec record names its part by `kind`, a registry per family of parts maps the kind to
the class.

Adding a part means writing a class with the interface described in parts/base.py and registering it here (or
from outside with the `register_*` functions); the model builder (models/decoder.py) looks the classes up by the
family an arrangement declares for each of its part names and by the `kind` of the part's spec record.
"""
from __future__ import annotations

from .base import ParamSpec, Part, StepPlan, StepShape
from .block import (Arrangement, BranchNormBlock, BranchNormMixerBlock, PostNormDepthBlock, PostNormDepthMixerBlock, PreNormBlock,
                    PreNormMixerBlock, SandwichBlock, SandwichMixerBlock, SandwichMixerSideBlock, SandwichSideBlock)
from .embedding import Embedding, NormedEmbedding, OutputHead, SideTableEmbedding
from .feed_forward import GLU, ClampedGLU, PolyNormMLP, RoutedGLU, SwiGLU
from .gated_attention import GatedAttention
from .latent_attention import LatentAttention
from .lru import GatedLRU
from .mixer import PagedAttention
from .parallel import ParallelMixer
from .retention import Retention
from .stream_mix import DepthAverage
from .talking_attention import TalkingAttention
from .token_input import GatedTableInput
from .wkv import WKV
from .norm import OnePlusRMSNorm, RMSNorm, ScalarGainRMSNorm
from .position import NoPosition, RotaryEmbedding, rope_inverse_frequencies

NORMS = {"rmsnorm": RMSNorm, "rmsnorm_scalar": ScalarGainRMSNorm, "rmsnorm_one_plus": OnePlusRMSNorm}
POSITION_ENCODINGS = {"rope": RotaryEmbedding, "none": NoPosition}
MIXERS = {"attention": PagedAttention, "talking_attention": TalkingAttention, "retention": Retention,
          "latent_attention": LatentAttention, "gated_attention": GatedAttention, "wkv": WKV, "gated_lru": GatedLRU,
          "parallel": ParallelMixer}
FEED_FORWARDS = {"swiglu": SwiGLU, "glu": GLU, "clamped_glu": ClampedGLU, "routed_glu": RoutedGLU, "poly_norm_mlp": PolyNormMLP}
ARRANGEMENTS = {"prenorm": PreNormBlock, "prenorm_mixer": PreNormMixerBlock, "branchnorm": BranchNormBlock,
                "branchnorm_mixer": BranchNormMixerBlock, "sandwich": SandwichBlock, "sandwich_mixer": SandwichMixerBlock,
                "sandwich_side": SandwichSideBlock, "sandwich_mixer_side": SandwichMixerSideBlock,
                "postnorm_depth": PostNormDepthBlock, "postnorm_depth_mixer": PostNormDepthMixerBlock}
EMBEDDINGS = {"table": Embedding, "table_norm": NormedEmbedding, "table_side": SideTableEmbedding}
TOKEN_INPUTS = {"gated_table": GatedTableInput}
STREAM_MIXES = {"depth_average": DepthAverage}
HEADS = {"linear": OutputHead}

# family name (what an arrangement's PARTS declares for a part name) -> registry
FAMILIES = {"norm": NORMS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS, "position": POSITION_ENCODINGS,
            "embedding": EMBEDDINGS, "head": HEADS, "token_input": TOKEN_INPUTS, "stream_mix": STREAM_MIXES}


def register_norm(kind, cls):
    NORMS[kind] = cls


def register_position_encoding(kind, cls):
    POSITION_ENCODINGS[kind] = cls


def register_mixer(kind, cls):
    MIXERS[kind] = cls


def register_feed_forward(kind, cls):
    FEED_FORWARDS[kind] = cls


def register_arrangement(kind, cls):
    ARRANGEMENTS[kind] = cls


def register_embedding(kind, cls):
    EMBEDDINGS[kind] = cls


def register_head(kind, cls):
    HEADS[kind] = cls


def register_token_input(kind, cls):
    TOKEN_INPUTS[kind] = cls


def register_stream_mix(kind, cls):
    STREAM_MIXES[kind] = cls
