"""The engine's kernel set: thin, checked wrappers around the sm_100a CUDA library.

`load()` builds `csrc/` on first use, loads the shared library with ctypes and returns the
one `Kernels` object the parts call into.  There is no other implementation: without a
CUDA device of compute capability 10.x, or without a working build, `load()` raises.

Every wrapper takes torch tensors that live on the GPU, checks dtype, shape and layout,
and launches on torch's current stream.  Matrix products in float32 always run this
library's FMA kernel.  In bfloat16 they run this library's tcgen05 kernels where those are
the faster ones (every product of a decode step of up to 32 tokens; the fused SwiGLU product
up to 128 tokens and, on the CTA-pair kernel, from 640 tokens), else cuBLAS through torch
(`torch.mm`), the library the reference's engine uses for them (engine/model.py:194,
F.linear); `gemm_policy` holds the measurements behind the choice.
"""
from __future__ import annotations

import ctypes
import math
import os
import threading

import numpy as np
import torch

from ..csrc import build as _build

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    # name: argtypes (all return int)
    "llm_check_device": [],
    "llm_set_pdl": [_c_int],
    "llm_abi_version": [],
    "llm_embed": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_add_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int,
                        _c_float, _c_int, ctypes.c_longlong, _c_void_p],
    "llm_rope_table": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
    "llm_rope_store": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int,
                       _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, ctypes.c_longlong, _c_void_p],
    "llm_silu_mul": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "llm_scale_f32": [_c_void_p, _c_float, ctypes.c_longlong, _c_void_p],
    "llm_sum_parts": [_c_void_p, _c_void_p, _c_int, _c_int, ctypes.c_longlong, _c_void_p],
    "llm_attention_generic": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                              _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_attention_bf16_supported": [_c_int, _c_int, _c_int],
    "llm_attention_prefill_bf16": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_attention_decode_bf16": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                  _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_decode_bf16_fused": [_c_void_p, _c_int, ctypes.c_longlong, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                        _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_decode_tma_supported": [_c_int, _c_int, _c_int, _c_int],
    "llm_attention_decode_bf16_tma": [_c_void_p, _c_int, _c_void_p, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p, _c_int,
                                      _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                                      _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_decode_bf16_fused_tma": [_c_void_p, _c_int, ctypes.c_longlong, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                                            ctypes.c_longlong, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                            _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                            _c_float, _c_int, _c_int, _c_void_p],
    "llm_attention_tcgen05_supported": [_c_int, _c_int, _c_int, _c_int],
    "llm_attention_prefill_tcgen05": [_c_void_p, _c_int, _c_int, _c_void_p, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p,
                                      _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                                      _c_void_p, _c_void_p, _c_void_p],
    "llm_attention_tcgen05_status": [],
    "llm_gemm_f32": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                     _c_void_p],
    "llm_gemm_bf16_token_tile": [_c_int],
    "llm_gemm_bf16": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                      _c_int, _c_int, _c_int, _c_void_p],
    "llm_gemm_bf16_status": [],
    "llm_gemm_bf16_wait_probe": [_c_int, _c_void_p],
    "llm_gemm_bf16_pair": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                           _c_void_p, _c_void_p],
    "llm_gemm_bf16_pair_scratch": [_c_int],
    "llm_gemm_bf16_pair_status": [],
    "llm_gather_tokens": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p],
    "llm_sample_scratch_floats": [_c_int, _c_int],
    "llm_sample": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "llm_attention_decode_status": [],
    "llm_conv_norm_store": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                            _c_void_p, _c_void_p, _c_void_p, _c_void_p, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_talking_attention": [_c_void_p, _c_int, _c_void_p, ctypes.c_longlong, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p,
                              _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                              _c_int, _c_int, _c_int, _c_float, _c_void_p],
    "llm_talking_attention_mma_supported": [_c_int, _c_int, _c_int, _c_int, _c_int, ctypes.c_longlong],
    "llm_talking_attention_mma": [_c_void_p, _c_int, _c_void_p, ctypes.c_longlong, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p,
                                  _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_float, _c_void_p],
    "llm_retention_scan": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                           _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p,
                           ctypes.c_longlong, _c_void_p, _c_int, _c_int, _c_void_p],
    "llm_retention_headnorm_gate": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                    _c_void_p],
    "llm_norm_add": [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p,
                     _c_void_p, _c_void_p],
    "llm_rmsnorm_rows": [_c_void_p, ctypes.c_longlong, _c_void_p, ctypes.c_longlong, _c_void_p, _c_int, _c_int, _c_int, _c_float,
                         _c_void_p],
    "llm_glu_act": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "llm_token_side_gate": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "llm_glu_clamped": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_float, _c_float, _c_void_p],
    "llm_latent_prepare": [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_float, _c_void_p, _c_void_p,
                           _c_void_p, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "llm_headnorm_store": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, ctypes.c_longlong, _c_int,
                           _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "llm_attention_flat": [_c_void_p, _c_int, _c_void_p, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int,
                           _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                           _c_float, _c_void_p, _c_float, _c_int, _c_void_p, _c_void_p],
    "llm_attention_flat_mma_supported": [_c_int, _c_int, _c_int, _c_int, _c_int, ctypes.c_longlong],
    "llm_attention_flat_mma_heads_per_block": [_c_int, _c_int],
    "llm_attention_flat_mma_smem": [_c_int, _c_int, _c_int],
    "llm_attention_flat_mma": [_c_void_p, _c_int, _c_void_p, ctypes.c_longlong, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int,
                               _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                               _c_float, _c_void_p, _c_float, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "llm_qk_prepare": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p,
                       ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_float, _c_void_p],
    "llm_post_norm": [_c_void_p, _c_void_p, _c_int, _c_float, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_void_p,
                      _c_void_p, _c_int, ctypes.c_longlong, _c_int, _c_int, _c_void_p],
    "llm_branch_mean": [_c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_float, _c_void_p, _c_int, _c_int, _c_void_p],
    "llm_poly_norm": [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "llm_lru_segment": [],
    "llm_lru_conv": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                     _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "llm_lru_gates": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int,
                      _c_int, _c_int, _c_int, _c_void_p],
    "llm_lru_step": [_c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                     _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                     _c_void_p],
    "llm_lru_scan": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
                     _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "llm_gemm_grouped_tile_rows": [],
    "llm_gemm_grouped": [_c_void_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, _c_void_p, _c_void_p, _c_void_p,
                         ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, _c_int,
                         _c_void_p, _c_int, _c_int, _c_float, _c_float, _c_void_p, _c_void_p, _c_void_p],
    "llm_route_topk": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "llm_moe_plan": [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p,
                     _c_void_p, _c_void_p],
    "llm_gather_rows": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "llm_moe_combine": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                        _c_void_p],
    "llm_token_shift": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int,
                        _c_void_p],
    "llm_wkv_decay": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p],
    "llm_wkv_scan": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int,
                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p],
}

# The library's health words in the order llm_sample copies them out (csrc/common.cuh): which kernel, and what its codes mean.
HEALTH_WORDS = (
    ("tcgen05 matrix product", "a bounded wait ran out (1 producer, 2 MMA issuer, 3 epilogue)"),
    ("CTA-pair matrix product", "a bounded wait ran out (1 producer, 2 MMA issuer, 3 epilogue, 4 drained accumulator, "
                                "5 other clusters' partial sums)"),
    ("tcgen05 prefill attention", "a bounded wait ran out (1 to 8), or a key's score lay more than 2^100 above all keys of "
                                  "the tiles before it (9: beyond what the one-pass softmax can mend; IITJ_ATTN_ONE_PASS=0 runs two passes "
                                  "everywhere)"),
    ("decode attention", "keys_per_split * max_splits did not cover an item's keys (6), or a bounded wait for keys and "
                         "values ran out (7)"),
)


def _ptr(t):
    return None if t is None else t.data_ptr()


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _check(t, name, dtype=None, dims=None):
    # the usual case in one expression (this runs several times per kernel launch); the messages are made below
    if type(t) is torch.Tensor and t.is_cuda and t.is_contiguous() and (dims is None or t.dim() == dims) and \
            (dtype is None or (t.dtype is dtype if type(dtype) is torch.dtype else t.dtype in dtype)):
        return
    _need(isinstance(t, torch.Tensor), f"{name}: expected a tensor")
    _need(t.is_cuda, f"{name}: tensor is on {t.device}, the kernels run on the GPU only")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list)) else t.dtype == dtype
        _need(ok, f"{name}: dtype {t.dtype} not accepted (want {dtype})")
    if dims is not None:
        _need(t.dim() == dims, f"{name}: expected {dims} dims, got shape {tuple(t.shape)}")
    _need(t.is_contiguous(), f"{name}: tensor must be contiguous")


class PartialSums:
    """The result of a matrix product that was split along k and whose partial sums are still to be added:
    `parts` [splits, tokens, n] float32 (in this library's scratch: valid until the next split product on the
    stream), `out` the tensor the sum belongs in.  `Kernels.add_rmsnorm` and `Kernels.rope_store` take it in
    place of the tensor and add the parts while they read; `sum()` adds them into `out` by a kernel of its own."""

    def __init__(self, kernels, parts, out):
        self.k, self.parts, self.out = kernels, parts, out
        self.shape, self.dtype = out.shape, out.dtype

    @property
    def splits(self) -> int:
        return self.parts.shape[0]

    @property
    def stride(self) -> int:
        return self.parts.shape[1] * self.parts.shape[2]

    def sum(self):
        return self.k.sum_parts(self.parts, self.out)


def materialize(x):
    """The tensor of `x`, which may be a PartialSums."""
    return x.sum() if isinstance(x, PartialSums) else x


class AttentionPlan:
    """How one step's tokens are handed to the tensor-core attention kernels: requests that
    bring one token go to the split-key decode kernel (`items`: their token rows), the rest
    are cut into tiles of 64 queries for the prefill kernel (`tiles`: first token row, rows,
    position of the first row, request).

    It is also the step plan of the attention mixer (parts/base.py, StepPlan): `arrays` are the lists the
    step function copies to the device with its own index arrays, `bind` receives them back as device
    tensors, `graph_key` is what a captured graph freezes of the plan."""

    graph_key = ()
    arrays: dict = {}

    def bind(self, views: dict) -> None:
        self.items = views.get("items")
        self.tiles = views["tiles"].view(-1, 4) if "tiles" in views else None
        self.big_tiles = views["big_tiles"].view(-1, 4) if "big_tiles" in views else None

    TILE = 64
    SPLIT_RULE = os.environ.get("IITJ_DECODE_SPLIT", "auto")    # "equal": always the rule for equal contexts (measurements)
    FORCE_KPS = int(os.environ.get("IITJ_DECODE_KPS", "0"))     # keys per split, whatever the rule says (measurements)

    def __init__(self, query_lens, seq_lens, device, items=None, tiles=None, total_tokens=None):
        self.decode_pos = []
        item_rows, tile_rows, big_rows, row = [], [], [], 0
        if total_tokens is not None and total_tokens == len(query_lens):      # one token each: all decode items
            item_rows, self.decode_pos, query_lens = list(range(total_tokens)), [t - 1 for t in seq_lens], ()
        for b, (n, total) in enumerate(zip(query_lens, seq_lens)):
            if n == 1:
                item_rows.append(row)
                self.decode_pos.append(total - 1)
            else:
                for s in range(0, n, self.TILE):
                    tile_rows.append((row + s, min(self.TILE, n - s), total - n + s, b))
                for s in range(0, n, 2 * self.TILE):        # 128-query tiles of the tcgen05 kernel
                    big_rows.append((row + s, min(2 * self.TILE, n - s), total - n + s, b))
            row += n
        # shortest contexts first: the prefill kernels walk these lists from their ends, so that the tiles with the most
        # keys start first and the short ones fill the gaps at the end of the launch
        big_rows.sort(key=lambda r: r[2] + r[1])
        tile_rows.sort(key=lambda r: r[2] + r[1])
        self.big_rows, self.big_tiles = big_rows, None
        self.n_items, self.n_tiles = len(item_rows), len(tile_rows)
        self.items, self.tiles = items, tiles
        self.context_bound = None     # an upper bound of the contexts that fixes the split choice (captured graphs)
        if self.items is None and item_rows:
            self.items = torch.tensor(item_rows, dtype=torch.int32).to(device)
        if self.tiles is None and tile_rows:
            self.tiles = torch.tensor(tile_rows, dtype=torch.int32).to(device)
        self.item_rows, self.tile_rows = item_rows, tile_rows
        self._splits: dict = {}

    def split(self, kv_heads: int, window: int, sm_count: int, head_dim: int = 128, bound: int | None = None):
        """(keys per split, most splits of any item).

        The decode kernel runs one CTA per (item, key/value head, split of that item's keys); an item with
        fewer keys than `keys per split` has one CTA, a long one several.  `resident` CTAs run at a time (2 per
        SM at head size 128, 4 at 64).  Candidates (the longest context cut into 1 .. 64 parts) are scored in
        units of keys, a CTA costing its keys plus 192:
          * contexts of about equal length (the shortest at least three quarters of the longest): waves of
            `resident` CTAs times the cost of one, which favours cuts that fill whole waves; the best wins;
          * unequal contexts (continuous batching: one 16k-token context beside thirty short ones): the longer
            of the longest CTA times the waves that the CTAs of more than half its length need, and the cost
            of all CTAs together shared out over `resident`; the coarsest cut within 5 % of the best wins.  So
            a long context among short ones is cut into many CTAs instead of keeping one SM busy while the
            others idle.
        `bound` replaces the longest context by an upper bound (captured graphs use one so that the choice
        stays the same while contexts grow); the other contexts are taken as grown by as much."""
        key = (kv_heads, window, head_dim, bound)
        if key not in self._splits:
            spans = []
            for pos in self.decode_pos:
                lo = max(0, pos - window + 1) if window > 0 else 0
                spans.append(pos - (lo // self.TILE) * self.TILE + 1)
            longest = max(spans) if bound is None else max(bound, max(spans))
            resident = sm_count * (2 if head_dim > 64 else 4)
            grown = longest - max(spans)
            equal = 4 * (min(spans) + grown) >= 3 * longest or self.SPLIT_RULE == "equal"
            arr = None if equal else np.asarray(spans, dtype=np.int64) + grown
            keys = 0 if equal else int(arr.sum()) * kv_heads
            pairs = self.n_items * kv_heads
            scored, seen = [], set()
            for n in range(1, 65):
                kps = -(-(-(-longest // n)) // self.TILE) * self.TILE
                if n > 1 and kps < 256:
                    break
                if kps in seen:
                    continue
                seen.add(kps)
                if equal:
                    cost = -(-pairs * -(-longest // kps) // resident) * (kps + 192)
                else:
                    ctas = int((-(-arr // kps)).sum()) * kv_heads
                    long_ctas = int(((arr + kps // 2) // kps).sum()) * kv_heads
                    cost = max(max(1, -(-long_ctas // resident)) * (min(kps, longest) + 192), (keys + 192 * ctas) / resident)
                scored.append((cost, kps))
            least = min(c for c, _ in scored)
            kps = next(k for c, k in scored if c <= (least if equal else 1.05 * least))
            if self.FORCE_KPS:
                kps = self.FORCE_KPS
            self._splits[key] = (kps, max((s - 1) // kps + 1 for s in ([longest] if bound is not None else spans)))
        return self._splits[key]


def attention_plan(meta, device) -> AttentionPlan:
    plan = getattr(meta, "attention_plan", None)
    if plan is None:
        plan = AttentionPlan(meta.query_lens, meta.seq_lens_host, device)
        meta.attention_plan = plan
    return plan


class Kernels:
    """Checked entry points of libllm_kernels.so.  One instance per process (see `load`)."""

    def __init__(self, library_path: str):
        self.library_path = library_path
        self.lib = ctypes.CDLL(library_path)
        self.lib.llm_last_error.restype = ctypes.c_char_p
        for name, args in _SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.argtypes = args
            fn.restype = _c_int
        self.launches = 0  # kernels of this library launched so far (the bench reports it)
        # IITJ_GEMM_BACKEND=cublas|tcgen05 forces one matrix-product path, IITJ_GEMM_SMALL_TOKENS moves the
        # SwiGLU boundary, IITJ_PDL=0 switches programmatic dependent launch off (all for measurements)
        self.gemm_backend = os.environ.get("IITJ_GEMM_BACKEND", "auto")
        self.gemm_small_tokens = int(os.environ.get("IITJ_GEMM_SMALL_TOKENS", "128"))
        self.gemm_plain_tokens = int(os.environ.get("IITJ_GEMM_PLAIN_TOKENS", "128"))   # plain products: tcgen05 up to here
        self.gemm_pair_mode = os.environ.get("IITJ_GEMM_PAIR", "swiglu")   # off | swiglu | all
        self.defer_sums = os.environ.get("IITJ_DEFER_SUMS", "1") == "1"     # k-split sums added by the reading kernel
        self.swiglu_half_tokens = int(os.environ.get("IITJ_SWIGLU_HALF_TOKENS", "64"))  # half-tile SwiGLU product up to here
        self.swiglu_half_smem_kb = int(os.environ.get("IITJ_SWIGLU_HALF_KB", "100"))
        self.fuse_decode = os.environ.get("IITJ_FUSE_DECODE", "1") != "0"   # rope + cache write inside decode attention
        self.decode_tma = os.environ.get("IITJ_DECODE_TMA", "1") != "0"     # decode attention fetches keys and values by TMA
        self.attention_splits = os.environ.get("IITJ_ATTN_SPLITS")         # forces the key splits of prefill attention
        self.attention_tcgen05 = os.environ.get("IITJ_ATTN_TCGEN05", "1") == "1"
        self.flat_mma = os.environ.get("IITJ_FLAT_MMA", "1") != "0"                     # tensor-core attention over flat pages
        self.talking_mma = os.environ.get("IITJ_TALKING_MMA", "1") != "0"               # tensor-core talking attention for prompt portions
        self.lru_step = os.environ.get("IITJ_LRU_STEP", "1") != "0"                      # one-launch recurrence for steps of single tokens
        self.retention_blocks = int(os.environ.get("IITJ_RETENTION_BLOCKS", "0"))        # blocks the retention walk aims at (0: its own rule)
        self.retention_segments = int(os.environ.get("IITJ_RETENTION_SEGMENTS", "0"))    # 1: never in segments, 2: always
        if os.environ.get("IITJ_PDL", "1") == "0":
            self.lib.llm_set_pdl(0)
        self._scratch_bufs: dict = {}
        self._pair_counters: dict = {}
        self._linear_plans: dict = {}    # (tokens, n, k, swiglu) -> (kernel, k-splits, shared memory, half-tile form)
        self.scratch_generation = 0
        self._sm_count = None
        self._device_index = None

    @property
    def sm_count(self) -> int:
        if self._sm_count is None:
            self._sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        return self._sm_count

    def _scratch(self, name, floats, device):
        """Grow-only float32 scratch (split-attention partials); contents never outlive a call."""
        buf = self._scratch_bufs.get((name, device))
        if buf is None or buf.numel() < floats:
            buf = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=device)
            self._scratch_bufs[(name, device)] = buf
            self.scratch_generation += 1
        return buf

    def _scratch_bf16(self, name, elements, device):
        """Grow-only bfloat16 scratch (grown to powers of two, so that token counts that creep up reallocate rarely)."""
        buf = self._scratch_bufs.get((name, device))
        if buf is None or buf.numel() < elements:
            buf = torch.empty(1 << max(elements - 1, 1 << 16).bit_length(), dtype=torch.bfloat16, device=device)
            self._scratch_bufs[(name, device)] = buf
            self.scratch_generation += 1
        return buf[:elements]

    # ---- plumbing --------------------------------------------------------------------
    def _call(self, name, *args):
        rc = getattr(self.lib, name)(*args)
        if rc != 0:
            raise KernelError(f"{name} failed ({rc}): {self.lib.llm_last_error().decode()}")
        self.launches += 1

    def _stream(self):
        """The raw handle of the current CUDA stream (inside a graph capture: the capturing stream)."""
        if self._device_index is None:
            self._device_index = torch.cuda.current_device()
        return torch._C._cuda_getCurrentRawStream(self._device_index)

    def set_pdl(self, on: bool) -> bool:
        """Programmatic dependent launch for all later launches of this library; returns the old setting."""
        return bool(self.lib.llm_set_pdl(1 if on else 0))

    def check_device(self):
        rc = self.lib.llm_check_device()
        if rc != 0:
            raise KernelError(self.lib.llm_last_error().decode())

    def plan_attention(self, shape) -> AttentionPlan:
        """The attention mixer's plan of a step (`shape`: parts.base.StepShape).  For a step that may run from a
        captured graph the split choice of decode attention is fixed by an upper bound of the contexts, in steps of
        512 tokens (the graph is captured anew when the batch outgrows the bound), and a step whose prompt portions
        reach contexts from LONG_PREFILL on is kept apart (its prefill attention launches key splits and a merge)."""
        plan = AttentionPlan(shape.query_lens, shape.seq_lens, shape.device, items=False, tiles=False,
                             total_tokens=shape.num_tokens)
        long_prefill = False
        if shape.graphable:
            if plan.n_items:
                plan.context_bound = (max(plan.decode_pos) + 512) // 512 * 512
            long_prefill = not shape.decode_shaped and any(n > 1 and end >= self.LONG_PREFILL
                                                           for n, end in zip(shape.query_lens, shape.seq_lens))
        plan.graph_key = (plan.context_bound, long_prefill)
        plan.arrays = {}
        if plan.n_items:
            plan.arrays["items"] = plan.item_rows
        if plan.n_tiles:
            plan.arrays["tiles"] = np.asarray(plan.tile_rows, dtype=np.int64).reshape(-1)
            plan.arrays["big_tiles"] = np.asarray(plan.big_rows, dtype=np.int64).reshape(-1)
        return plan

    # ---- row-wise kernels ------------------------------------------------------------
    def embed(self, ids, table, out, scale: float = 1.0):
        """out[t] = scale * table[ids[t]] as float32 (the residual stream)."""
        _check(ids, "embed.ids", torch.int32, 1)
        _check(table, "embed.table", tuple(DTYPE_CODE), 2)
        _check(out, "embed.out", torch.float32, 2)
        _need(out.shape == (ids.shape[0], table.shape[1]), "embed.out: wrong shape")
        self._call("llm_embed", _ptr(ids), _ptr(table), DTYPE_CODE[table.dtype], _ptr(out), ids.shape[0],
                   table.shape[1], table.shape[0], float(scale), self._stream())
        return out

    def add_rmsnorm(self, residual, delta, weight, eps: float, out, rows=None):
        """residual += delta (when given, and rows is None); out = rmsnorm(residual[rows]) * weight."""
        _check(residual, "add_rmsnorm.residual", torch.float32, 2)
        width = residual.shape[1]
        _check(out, "add_rmsnorm.out", tuple(DTYPE_CODE), 2)
        _check(weight, "add_rmsnorm.weight", tuple(DTYPE_CODE), 1)
        _need(weight.shape[0] == width and out.shape[1] == width, "add_rmsnorm: widths differ")
        splits, stride = 0, 0
        if isinstance(delta, PartialSums) and (delta.splits > 8 or delta.stride % 4):
            delta = delta.sum()
        if isinstance(delta, PartialSums):
            _need(tuple(delta.shape) == tuple(residual.shape), "add_rmsnorm.delta: shape differs from residual")
            splits, stride, delta = delta.splits, delta.stride, delta.parts
        elif delta is not None:
            _check(delta, "add_rmsnorm.delta", out.dtype, 2)
            _need(delta.shape == residual.shape, "add_rmsnorm.delta: shape differs from residual")
        if rows is not None:
            _check(rows, "add_rmsnorm.rows", torch.int32, 1)
            _need(out.shape[0] == rows.shape[0], "add_rmsnorm.out: one row per entry of rows")
        else:
            _need(out.shape[0] == residual.shape[0], "add_rmsnorm.out: shape differs from residual")
        self._call("llm_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(rows), _ptr(weight),
                   DTYPE_CODE[weight.dtype], _ptr(out), DTYPE_CODE[out.dtype], out.shape[0], width, float(eps),
                   splits, stride, self._stream())
        return out

    def rope_tables(self, positions, inv_freq, cos, sin, amplitude: float = 1.0):
        """cos[t, i] = amplitude * cos(positions[t] * inv_freq[i]) and sin likewise, float32 [tokens, rotary_dim/2]."""
        _check(positions, "rope_tables.positions", torch.int32, 1)
        _check(inv_freq, "rope_tables.inv_freq", torch.float32, 1)
        _check(cos, "rope_tables.cos", torch.float32, 2)
        _check(sin, "rope_tables.sin", torch.float32, 2)
        _need(cos.shape == (positions.shape[0], inv_freq.shape[0]) and sin.shape == cos.shape, "rope_tables: wrong table shape")
        self._call("llm_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), positions.shape[0],
                   inv_freq.shape[0], float(amplitude), self._stream())
        return cos, sin

    def rope_store(self, qkv, positions, inv_freq, slots, cache_layer, heads, kv_heads, head_dim, rotary_dim,
                   tables=None):
        """Rotate q (in place) and k, store k and v of every token in its cache slot.

        cache_layer: [pages, 2, kv_heads, page_size, head_dim]; slots may be None (rotate only).
        tables: (cos, sin) of `rope_tables` for these positions, else the angles are evaluated here.
        `qkv` may be a PartialSums: its parts are added on the way (all dims rotated, head_dim % 8 == 0),
        else summed first.  Returns the tensor that holds the rotated queries."""
        parts = None
        if isinstance(qkv, PartialSums):
            if rotary_dim == head_dim and head_dim % 8 == 0 and qkv.splits <= 8:
                parts, qkv = qkv, qkv.out
            else:
                qkv = qkv.sum()
        _check(qkv, "rope_store.qkv", tuple(DTYPE_CODE), 2)
        _check(positions, "rope_store.positions", torch.int32, 1)
        tokens = qkv.shape[0]
        _need(qkv.shape[1] == (heads + 2 * kv_heads) * head_dim, "rope_store.qkv: width is not (heads+2*kv_heads)*head_dim")
        _need(positions.shape[0] == tokens, "rope_store.positions: one per token")
        if rotary_dim:
            _check(inv_freq, "rope_store.inv_freq", torch.float32, 1)
            _need(inv_freq.shape[0] == rotary_dim // 2, "rope_store.inv_freq: rotary_dim/2 entries")
        page_size = 1
        if slots is not None:
            _check(slots, "rope_store.slots", torch.int32, 1)
            _need(slots.shape[0] == tokens, "rope_store.slots: one per token")
            _check(cache_layer, "rope_store.cache", qkv.dtype, 5)
            _need(cache_layer.shape[1] == 2 and cache_layer.shape[2] == kv_heads and cache_layer.shape[4] == head_dim,
                  f"rope_store.cache: shape {tuple(cache_layer.shape)} does not fit kv_heads/head_dim")
            page_size = cache_layer.shape[3]
        cos = sin = None
        if tables is not None and rotary_dim:
            cos, sin = tables
            _check(cos, "rope_store.cos", torch.float32, 2)
            _check(sin, "rope_store.sin", torch.float32, 2)
            _need(cos.shape == (tokens, rotary_dim // 2) and sin.shape == cos.shape, "rope_store: wrong table shape")
        self._call("llm_rope_store", _ptr(qkv), _ptr(positions), _ptr(inv_freq) if rotary_dim else None, _ptr(cos), _ptr(sin),
                   _ptr(slots), _ptr(cache_layer) if slots is not None else None, DTYPE_CODE[qkv.dtype], tokens,
                   heads, kv_heads, head_dim, rotary_dim, page_size, _ptr(parts.parts) if parts is not None else None,
                   parts.splits if parts is not None else 0, parts.stride if parts is not None else 0, self._stream())
        return qkv

    def silu_mul(self, gu, act):
        _check(gu, "silu_mul.gu", tuple(DTYPE_CODE), 2)
        _check(act, "silu_mul.act", gu.dtype, 2)
        _need(gu.shape[1] == 2 * act.shape[1] and gu.shape[0] == act.shape[0], "silu_mul: shapes do not fit")
        self._call("llm_silu_mul", _ptr(gu), _ptr(act), DTYPE_CODE[gu.dtype], act.shape[0], act.shape[1],
                   self._stream())
        return act

    # ---- attention -------------------------------------------------------------------
    def attention(self, qkv, cache_layer, meta, out, heads, kv_heads, head_dim, window: int = 0,
                  scale: float = 0.0):
        """Causal attention of every token in `qkv` (query heads first in each row) over the
        paged keys and values of its request.  `meta` carries block_table [B, W],
        token_request [T] and positions [T] as int32 device tensors."""
        _check(qkv, "attention.qkv", tuple(DTYPE_CODE), 2)
        _check(cache_layer, "attention.cache", qkv.dtype, 5)
        _check(out, "attention.out", qkv.dtype, 2)
        tokens = qkv.shape[0]
        _need(qkv.shape[1] >= heads * head_dim, "attention.qkv: row too narrow")
        _need(out.shape == (tokens, heads * head_dim), "attention.out: wrong shape")
        _need(cache_layer.shape[1] == 2 and cache_layer.shape[2] == kv_heads and cache_layer.shape[4] == head_dim,
              f"attention.cache: shape {tuple(cache_layer.shape)} does not fit kv_heads/head_dim")
        _check(meta.block_table, "attention.block_table", torch.int32, 2)
        _check(meta.token_request, "attention.token_request", torch.int32, 1)
        _check(meta.positions, "attention.positions", torch.int32, 1)
        _need(meta.token_request.shape[0] == tokens and meta.positions.shape[0] == tokens,
              "attention: one token_request and one position per token")
        if not scale:
            scale = 1.0 / math.sqrt(head_dim)
        page_size = cache_layer.shape[3]
        if qkv.dtype == torch.bfloat16 and self.lib.llm_attention_bf16_supported(heads, kv_heads, head_dim):
            plan = attention_plan(meta, qkv.device)
            if plan.n_tiles and self.attention_tcgen05 and \
                    cache_layer.shape[0] * 2 * kv_heads * page_size < (1 << 31) and \
                    self.lib.llm_attention_tcgen05_supported(heads, kv_heads, head_dim, page_size):     # (TMA coordinates are 32-bit)
                if plan.big_tiles is None:
                    plan.big_tiles = torch.tensor(plan.big_rows, dtype=torch.int32).to(qkv.device)
                splits = self.prefill_key_splits(plan.big_rows, heads, kv_heads, int(window))
                part_o = part_ml = None
                if splits > 1:
                    n = len(plan.big_rows) * heads * splits * 128
                    part_o = self._scratch("attn.tc_part_o", n * head_dim, qkv.device)
                    part_ml = self._scratch("attn.tc_part_ml", n * 2, qkv.device)
                self._call("llm_attention_prefill_tcgen05", _ptr(qkv), qkv.shape[1], tokens, _ptr(cache_layer),
                           cache_layer.shape[0], _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.big_tiles),
                           len(plan.big_rows), _ptr(out), out.shape[1], heads, kv_heads, head_dim, page_size, int(window),
                           float(scale), splits, _ptr(part_o), _ptr(part_ml), self._stream())
                if splits > 1:
                    self.launches += 1
            elif plan.n_tiles:
                self._call("llm_attention_prefill_bf16", _ptr(qkv), qkv.shape[1], _ptr(cache_layer),
                           _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.tiles), plan.n_tiles, _ptr(out),
                           out.shape[1], heads, kv_heads, head_dim, page_size, int(window), float(scale), self._stream())
            if plan.n_items:
                kps, splits = plan.split(kv_heads, int(window), self.sm_count, head_dim, getattr(plan, 'context_bound', None))
                part_o = part_ml = None
                if splits > 1:
                    part_o = self._scratch("attn.part_o", plan.n_items * heads * splits * head_dim, qkv.device)
                    part_ml = self._scratch("attn.part_ml", plan.n_items * heads * splits * 2, qkv.device)
                if self._decode_by_tma(cache_layer, heads, kv_heads, head_dim):
                    self._call("llm_attention_decode_bf16_tma", _ptr(qkv), qkv.shape[1], _ptr(cache_layer), cache_layer.shape[0],
                               _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.items), plan.n_items,
                               _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o), _ptr(part_ml), _ptr(out),
                               out.shape[1], heads, kv_heads, head_dim, page_size, int(window), float(scale), kps, splits,
                               self._stream())
                else:
                    self._call("llm_attention_decode_bf16", _ptr(qkv), qkv.shape[1], _ptr(cache_layer),
                               _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.items), plan.n_items,
                               _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o), _ptr(part_ml), _ptr(out),
                               out.shape[1], heads, kv_heads, head_dim, page_size, int(window), float(scale), kps, splits,
                               self._stream())
                if splits > 1:
                    self.launches += 1      # the merge kernel
            return out
        self._call("llm_attention_generic", _ptr(qkv), qkv.shape[1], _ptr(cache_layer), _ptr(meta.block_table),
                   meta.block_table.shape[1], _ptr(meta.token_request), _ptr(meta.positions), _ptr(out),
                   out.shape[1], DTYPE_CODE[qkv.dtype], tokens, heads, kv_heads, head_dim, page_size,
                   int(window), float(scale), self._stream())
        return out

    def _decode_by_tma(self, cache_layer, heads, kv_heads, head_dim) -> bool:
        """True if decode attention fetches this cache layer's keys and values by TMA: a page size of 8 to 64 tokens, and
        a layer whose rows (pages x 2 x kv_heads x page_size) fit TMA's 32-bit coordinates; else the copying kernel runs."""
        pages, page_size = cache_layer.shape[0], cache_layer.shape[3]
        return bool(self.decode_tma and pages * 2 * kv_heads * page_size < (1 << 31) and
                    self.lib.llm_attention_decode_tma_supported(heads, kv_heads, head_dim, page_size))

    def can_fuse_decode(self, qkv, meta, cache_layer, heads, kv_heads, head_dim) -> bool:
        """True if `attention_decode_fused` takes this step: every token is a single decoded token, the qkv
        product was left as at most eight partial sums, bfloat16 cache, a shape of the tensor-core kernel."""
        if not (self.fuse_decode and isinstance(qkv, PartialSums) and 1 <= qkv.splits <= 8 and qkv.stride % 4 == 0):
            return False
        if cache_layer is None or cache_layer.dtype != torch.bfloat16 or qkv.out.dtype != torch.bfloat16:
            return False
        if not self.lib.llm_attention_bf16_supported(heads, kv_heads, head_dim):
            return False
        plan = attention_plan(meta, cache_layer.device)
        return plan.n_tiles == 0 and plan.n_items == qkv.out.shape[0]

    def attention_decode_fused(self, qkv, tables, slots, cache_layer, meta, out, heads, kv_heads, head_dim,
                               window: int = 0, scale: float = 0.0):
        """Decode attention straight from the qkv product's partial sums (`can_fuse_decode` holds): adds the
        parts, rotates queries and keys with `tables` (cos, sin of `rope_tables`; every dim rotated), stores each
        token's key and value at `slots`, attends over the paged cache.  One kernel (and the merge of key
        splits) in place of rope_store + attention."""
        cos, sin = tables
        tokens = qkv.out.shape[0]
        _check(qkv.parts, "attention_decode_fused.parts", torch.float32, 3)
        _check(cos, "attention_decode_fused.cos", torch.float32, 2)
        _check(sin, "attention_decode_fused.sin", torch.float32, 2)
        _check(slots, "attention_decode_fused.slots", torch.int32, 1)
        _check(cache_layer, "attention_decode_fused.cache", torch.bfloat16, 5)
        _check(out, "attention_decode_fused.out", torch.bfloat16, 2)
        _need(qkv.out.shape[1] == (heads + 2 * kv_heads) * head_dim, "attention_decode_fused: qkv width is not (heads+2*kv_heads)*head_dim")
        _need(cos.shape == (tokens, head_dim // 2) and sin.shape == cos.shape, "attention_decode_fused: tables must be [tokens, head_dim/2]")
        _need(slots.shape[0] == tokens and out.shape == (tokens, heads * head_dim), "attention_decode_fused: one slot and one output row per token")
        _need(cache_layer.shape[1] == 2 and cache_layer.shape[2] == kv_heads and cache_layer.shape[4] == head_dim,
              f"attention_decode_fused.cache: shape {tuple(cache_layer.shape)} does not fit kv_heads/head_dim")
        _need(meta.token_request.shape[0] == tokens and meta.positions.shape[0] == tokens,
              "attention_decode_fused: one token_request and one position per token")
        if not scale:
            scale = 1.0 / math.sqrt(head_dim)
        plan = attention_plan(meta, out.device)
        _need(plan.n_tiles == 0 and plan.n_items == tokens, "attention_decode_fused: every token must be a single decoded token")
        kps, splits = plan.split(kv_heads, int(window), self.sm_count, head_dim, getattr(plan, 'context_bound', None))
        part_o = part_ml = None
        if splits > 1:
            part_o = self._scratch("attn.part_o", plan.n_items * heads * splits * head_dim, out.device)
            part_ml = self._scratch("attn.part_ml", plan.n_items * heads * splits * 2, out.device)
        if self._decode_by_tma(cache_layer, heads, kv_heads, head_dim):
            self._call("llm_attention_decode_bf16_fused_tma", _ptr(qkv.parts), qkv.splits, qkv.stride, _ptr(cos), _ptr(sin),
                       _ptr(slots), _ptr(cache_layer), cache_layer.shape[0], _ptr(meta.block_table), meta.block_table.shape[1],
                       _ptr(plan.items), plan.n_items, _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o),
                       _ptr(part_ml), _ptr(out), out.shape[1], heads, kv_heads, head_dim, cache_layer.shape[3], int(window),
                       float(scale), kps, splits, self._stream())
        else:
            self._call("llm_attention_decode_bf16_fused", _ptr(qkv.parts), qkv.splits, qkv.stride, _ptr(cos), _ptr(sin), _ptr(slots),
                       _ptr(cache_layer), _ptr(meta.block_table), meta.block_table.shape[1], _ptr(plan.items), plan.n_items,
                       _ptr(meta.token_request), _ptr(meta.positions), _ptr(part_o), _ptr(part_ml), _ptr(out), out.shape[1],
                       heads, kv_heads, head_dim, cache_layer.shape[3], int(window), float(scale), kps, splits, self._stream())
        if splits > 1:
            self.launches += 1      # the merge kernel
        return out


    # ---- mixers with state: short convolution, talking-heads attention, retention ------------------------
    @staticmethod
    def _page_size_of(cache_layer, kv_heads, head_dim, value_dim) -> int:
        per_token = kv_heads * (head_dim + value_dim)
        _need(cache_layer.dim() == 2 and cache_layer.shape[1] % per_token == 0,
              f"cache: a page of {tuple(cache_layer.shape)} is not key plane + value plane of {kv_heads} heads of {head_dim} + {value_dim}")
        return cache_layer.shape[1] // per_token

    def conv_norm_store(self, u, bias, taps_w, q_gain, k_gain, state, state_slots, token_request, cu_seqlens, q_out,
                        cache_layer, slots, heads, kv_heads, head_dim, value_dim, eps):
        """Bias, short causal convolution over time, norms, and the store of keys and values (csrc/short_conv.cu).

        u [T, C] is the fused projection: query channels, then (when `cache_layer` is given) key and value channels.
        bias [C], taps_w [C, taps], q_gain, k_gain: float32 (bias / taps_w None: no bias / one tap).  state
        [slots, taps - 1, C] float32 holds every request's last projected rows and is brought up to date.  Writes the
        normed queries to q_out [T, heads * head_dim] and, at `slots`, normed keys and values into cache_layer
        [pages, kv_heads * page * (head_dim + value_dim)]."""
        _check(u, "conv_norm_store.u", tuple(DTYPE_CODE), 2)
        tokens, channels = u.shape
        own = cache_layer is not None
        _need(channels == heads * head_dim + (kv_heads * (head_dim + value_dim) if own else 0), "conv_norm_store.u: wrong width")
        taps = 1
        if taps_w is not None:
            _check(taps_w, "conv_norm_store.taps", torch.float32, 2)
            _need(taps_w.shape[0] == channels, "conv_norm_store.taps: one row per channel")
            taps = taps_w.shape[1]
        if bias is not None:
            _check(bias, "conv_norm_store.bias", torch.float32, 1)
            _need(bias.shape[0] == channels, "conv_norm_store.bias: one per channel")
        _check(q_gain, "conv_norm_store.q_gain", torch.float32, 1)
        _need(q_gain.shape[0] == heads * head_dim, "conv_norm_store.q_gain: one per query channel")
        _check(q_out, "conv_norm_store.q_out", u.dtype, 2)
        _need(q_out.shape == (tokens, heads * head_dim), "conv_norm_store.q_out: wrong shape")
        for name, t in (("state_slots", state_slots), ("token_request", token_request), ("cu_seqlens", cu_seqlens)):
            _check(t, "conv_norm_store." + name, torch.int32, 1)
        requests = state_slots.shape[0]
        _need(token_request.shape[0] == tokens and cu_seqlens.shape[0] == requests + 1, "conv_norm_store: index arrays do not fit")
        if taps > 1:
            _check(state, "conv_norm_store.state", torch.float32, 3)
            _need(tuple(state.shape[1:]) == (taps - 1, channels), "conv_norm_store.state: [slots, taps - 1, channels]")
        page_size, page_stride = 1, 0
        if own:
            _check(cache_layer, "conv_norm_store.cache", u.dtype, 2)
            _check(k_gain, "conv_norm_store.k_gain", torch.float32, 1)
            _need(k_gain.shape[0] == kv_heads * head_dim, "conv_norm_store.k_gain: one per key channel")
            _check(slots, "conv_norm_store.slots", torch.int32, 1)
            _need(slots.shape[0] == tokens, "conv_norm_store.slots: one per token")
            page_size, page_stride = self._page_size_of(cache_layer, kv_heads, head_dim, value_dim), cache_layer.shape[1]
        self._call("llm_conv_norm_store", _ptr(u), _ptr(bias), _ptr(taps_w), taps, _ptr(q_gain), _ptr(k_gain) if own else None,
                   _ptr(state) if taps > 1 else None, _ptr(state_slots), _ptr(token_request), _ptr(cu_seqlens), _ptr(q_out),
                   _ptr(cache_layer) if own else None, _ptr(slots) if own else None, page_stride, page_size,
                   DTYPE_CODE[u.dtype], tokens, requests, heads, kv_heads, head_dim, value_dim, float(eps), self._stream())
        if taps > 1:
            self.launches += 1      # the state's own kernel
        return q_out

    def talking_attention(self, q, cache_layer, meta, talk, slopes, out, heads, kv_heads, head_dim, value_dim, chunk, scale,
                          tiles=None):
        """Attention with a distance bias (slopes [heads]) and heads mixed before the softmax (talk [heads, heads]),
        over the keys of the query's own chunk (`chunk` 0: all earlier keys); csrc/talking_attention.cu.  `tiles`
        [n, 4] int32 (first token row, rows up to 16, position of the first row, request) cuts the step's tokens into
        runs of one request: with them, bfloat16 and sizes it takes, the tensor-core form runs (csrc/talking_attention_mma.cu)."""
        _check(q, "talking_attention.q", tuple(DTYPE_CODE), 2)
        _check(cache_layer, "talking_attention.cache", q.dtype, 2)
        _check(out, "talking_attention.out", q.dtype, 2)
        _check(talk, "talking_attention.talk", torch.float32, 2)
        _check(slopes, "talking_attention.slopes", torch.float32, 1)
        tokens = q.shape[0]
        _need(q.shape[1] == heads * head_dim and out.shape == (tokens, heads * value_dim), "talking_attention: q / out shapes do not fit")
        _need(tuple(talk.shape) == (heads, heads) and slopes.shape[0] == heads, "talking_attention: talk [heads, heads], slopes [heads]")
        _check(meta.block_table, "talking_attention.block_table", torch.int32, 2)
        _check(meta.token_request, "talking_attention.token_request", torch.int32, 1)
        _check(meta.positions, "talking_attention.positions", torch.int32, 1)
        _need(meta.token_request.shape[0] == tokens and meta.positions.shape[0] == tokens,
              "talking_attention: one token_request and one position per token")
        page_size = self._page_size_of(cache_layer, kv_heads, head_dim, value_dim)
        if tiles is not None and q.dtype == torch.bfloat16 and self.talking_mma and \
                self.lib.llm_talking_attention_mma_supported(heads, kv_heads, head_dim, value_dim, int(chunk), cache_layer.shape[1]):
            _check(tiles, "talking_attention.tiles", torch.int32, 2)
            _need(tiles.shape[1] == 4, "talking_attention.tiles: [n, 4]")
            self._call("llm_talking_attention_mma", _ptr(q), q.shape[1], _ptr(cache_layer), cache_layer.shape[1],
                       kv_heads * page_size * head_dim, _ptr(meta.block_table), meta.block_table.shape[1], _ptr(tiles),
                       tiles.shape[0], _ptr(talk), _ptr(slopes), _ptr(out), out.shape[1], heads, kv_heads, head_dim, value_dim,
                       page_size, int(chunk), float(scale), self._stream())
            return out
        self._call("llm_talking_attention", _ptr(q), q.shape[1], _ptr(cache_layer), cache_layer.shape[1],
                   kv_heads * page_size * head_dim, _ptr(meta.block_table), meta.block_table.shape[1], _ptr(meta.token_request),
                   _ptr(meta.positions), _ptr(talk), _ptr(slopes), _ptr(out), out.shape[1], DTYPE_CODE[q.dtype], tokens,
                   heads, kv_heads, head_dim, value_dim, page_size, int(chunk), float(scale), self._stream())
        return out

    def retention(self, proj, tables, rotary_dim, decay, state, state_slots, cu_seqlens, o, heads, head_dim, value_dim,
                  k_scale, write: bool = True, longest: int = 0):
        """The retention scan (csrc/retention.cu): proj [T, >= 2*heads*head_dim + heads*value_dim] holds q, k, v of all
        heads; tables = (cos, sin) [T, rotary_dim / 2] float32 or None; decay [heads] float32; state
        [slots, heads, value_dim, head_dim] float32 (S transposed) is read and, with `write`, left at the step's last token;
        o [T, heads * value_dim] float32.  `longest`: the most tokens one request brings, if the caller knows it (a
        long portion is then walked in segments side by side and mended in a second pass)."""
        _check(proj, "retention.proj", tuple(DTYPE_CODE), 2)
        tokens = proj.shape[0]
        _need(proj.shape[1] >= 2 * heads * head_dim + heads * value_dim, "retention.proj: row too narrow")
        _check(decay, "retention.decay", torch.float32, 1)
        _check(state, "retention.state", torch.float32, 4)
        _need(decay.shape[0] == heads and tuple(state.shape[1:]) == (heads, value_dim, head_dim), "retention: decay / state shapes do not fit")
        _check(state_slots, "retention.state_slots", torch.int32, 1)
        _check(cu_seqlens, "retention.cu_seqlens", torch.int32, 1)
        _need(cu_seqlens.shape[0] == state_slots.shape[0] + 1, "retention.cu_seqlens: requests + 1 entries")
        _check(o, "retention.o", torch.float32, 2)
        _need(o.shape == (tokens, heads * value_dim), "retention.o: wrong shape")
        cos = sin = None
        half = rotary_dim // 2
        if half:
            cos, sin = tables
            _check(cos, "retention.cos", torch.float32, 2)
            _check(sin, "retention.sin", torch.float32, 2)
            _need(cos.shape == (tokens, half) and sin.shape == cos.shape, "retention: tables must be [tokens, rotary_dim / 2]")
        requests = state_slots.shape[0]
        seg, seg_floats = None, 0
        if longest >= 256:
            seg_floats = requests * min(32, -(-longest // 128)) * heads * value_dim * head_dim
            if seg_floats <= (1 << 28):        # (a GiB of scratch at most; beyond that the walk stays whole)
                seg = self._scratch("retention.segments", seg_floats, proj.device)
        rc = self.lib.llm_retention_scan(_ptr(proj), proj.shape[1], _ptr(cos), _ptr(sin), half, _ptr(decay), _ptr(state),
                                         _ptr(state_slots), _ptr(cu_seqlens), _ptr(o), DTYPE_CODE[proj.dtype], tokens, requests,
                                         heads, head_dim, value_dim, float(k_scale), 1 if write else 0, int(longest), _ptr(seg),
                                         seg_floats if seg is not None else 0,
                                         _ptr(self._scratch("retention.rotated", tokens * heads * 2 * head_dim, proj.device)),
                                         self.retention_blocks, self.retention_segments, self._stream())
        if rc < 0:
            raise KernelError(f"llm_retention_scan failed ({rc}): {self.lib.llm_last_error().decode()}")
        self.launches += 2 if rc <= 1 else 3          # rotation, walk (and its second pass)
        return o

    def headnorm_gate(self, o, proj, gate_col, out, heads, value_dim, eps):
        """out = (each head of o divided by its root mean square) * silu(proj[:, gate_col : gate_col + heads * value_dim])."""
        _check(o, "headnorm_gate.o", torch.float32, 2)
        _check(proj, "headnorm_gate.proj", tuple(DTYPE_CODE), 2)
        _check(out, "headnorm_gate.out", proj.dtype, 2)
        tokens = o.shape[0]
        _need(o.shape == (tokens, heads * value_dim) and out.shape == o.shape and proj.shape[0] == tokens and
              gate_col + heads * value_dim <= proj.shape[1], "headnorm_gate: shapes do not fit")
        self._call("llm_retention_headnorm_gate", _ptr(o), proj.data_ptr() + gate_col * proj.element_size(), proj.shape[1],
                   _ptr(out), DTYPE_CODE[proj.dtype], tokens, heads, value_dim, float(eps), self._stream())
        return out

    # ---- branch norms, gated feed-forwards with clamps, routed experts ------------------------------------------
    def norm_add(self, residual, branch, weight, eps, cast_out=None, accumulate: bool = True, next_weight=None, next_out=None):
        """residual (+)= rmsnorm(branch) * weight with float32 statistics (csrc/branch_norm.cu); `cast_out`: a copy of the new
        residual in another type (what the next sub-layer reads).  `accumulate` False writes the normed rows instead.
        With `next_weight` and `next_out` the new residual rows are normed too: next_out = rmsnorm(residual) * next_weight."""
        _check(residual, "norm_add.residual", torch.float32, 2)
        _check(branch, "norm_add.branch", tuple(DTYPE_CODE), 2)
        _check(weight, "norm_add.weight", tuple(DTYPE_CODE), 1)
        tokens, width = residual.shape
        _need(tuple(branch.shape) == (tokens, width) and weight.shape[0] == width, "norm_add: shapes differ")
        if cast_out is not None:
            _check(cast_out, "norm_add.cast_out", tuple(DTYPE_CODE), 2)
            _need(cast_out.shape == residual.shape, "norm_add.cast_out: shape differs from residual")
        typed = cast_out if cast_out is not None else next_out
        if next_out is not None:
            _check(next_out, "norm_add.next_out", tuple(DTYPE_CODE), 2)
            _check(next_weight, "norm_add.next_weight", weight.dtype, 1)
            _need(next_out.shape == residual.shape and next_weight.shape[0] == width and next_out.dtype == typed.dtype,
                  "norm_add.next_out: shape or type differs")
        else:
            _need(next_weight is None, "norm_add: a second gain without a place for its rows")
        self._call("llm_norm_add", _ptr(residual), _ptr(branch), DTYPE_CODE[branch.dtype], _ptr(weight), DTYPE_CODE[weight.dtype],
                   _ptr(cast_out), DTYPE_CODE[typed.dtype] if typed is not None else 0, tokens, width, float(eps),
                   1 if accumulate else 0, _ptr(next_weight), _ptr(next_out), self._stream())
        return residual

    def rmsnorm_rows(self, x, weight, eps, out):
        """out[t] = x[t] * rsqrt(mean(x[t]^2) + eps) * weight for rows of the engine's type; x and out may be column ranges of
        wider matrices (rows with strides of their own, unit stride inside a row)."""
        _need(x.dim() == 2 and out.dim() == 2 and x.dtype in DTYPE_CODE and out.dtype == x.dtype and x.is_cuda and out.is_cuda,
              "rmsnorm_rows: two matrices of one of the engine's types on the device")
        _need(x.stride(1) == 1 and out.stride(1) == 1 and tuple(out.shape) == tuple(x.shape), "rmsnorm_rows: rows must be dense and alike")
        _check(weight, "rmsnorm_rows.weight", torch.float32, 1)
        _need(weight.shape[0] == x.shape[1], "rmsnorm_rows.weight: one gain per column")
        self._call("llm_rmsnorm_rows", x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), _ptr(weight), DTYPE_CODE[x.dtype],
                   x.shape[0], x.shape[1], float(eps), self._stream())
        return out

    GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}

    def glu_act(self, gu, act, activation: str):
        """act = f(gate) * up from gu [T, 2 * inner] (gate columns, then up columns); f is "silu" or "gelu_tanh"."""
        _check(gu, "glu_act.gu", tuple(DTYPE_CODE), 2)
        _check(act, "glu_act.act", gu.dtype, 2)
        _need(gu.shape[1] == 2 * act.shape[1] and gu.shape[0] == act.shape[0], "glu_act: shapes do not fit")
        _need(activation in self.GLU_ACTIVATIONS, f"glu_act: activation {activation!r} is not known")
        self._call("llm_glu_act", _ptr(gu), _ptr(act), DTYPE_CODE[gu.dtype], act.shape[0], act.shape[1],
                   self.GLU_ACTIVATIONS[activation], self._stream())
        return act

    def token_side_gate(self, gate, table, ids, offset: int, out):
        """out[t, d] = gelu_tanh(gate[t, d]) * table[ids[t], offset + d] (csrc/token_side.cu)."""
        _check(gate, "token_side_gate.gate", tuple(DTYPE_CODE), 2)
        _check(table, "token_side_gate.table", gate.dtype, 2)
        _check(out, "token_side_gate.out", gate.dtype, 2)
        _check(ids, "token_side_gate.ids", torch.int32, 1)
        _need(tuple(out.shape) == tuple(gate.shape) and ids.shape[0] == gate.shape[0], "token_side_gate: shapes do not fit")
        self._call("llm_token_side_gate", _ptr(gate), _ptr(table), _ptr(ids), _ptr(out), DTYPE_CODE[gate.dtype], gate.shape[0],
                   gate.shape[1], table.shape[1], int(offset), self._stream())
        return out

    def glu_clamped(self, gu, act, limit: float, slope: float):
        """act = g * sigmoid(slope * g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit); gu [T, 2 * inner]
        holds the gate columns, then the up columns."""
        _check(gu, "glu_clamped.gu", tuple(DTYPE_CODE), 2)
        _check(act, "glu_clamped.act", gu.dtype, 2)
        _need(gu.shape[1] == 2 * act.shape[1] and gu.shape[0] == act.shape[0], "glu_clamped: shapes do not fit")
        self._call("llm_glu_clamped", _ptr(gu), _ptr(act), DTYPE_CODE[gu.dtype], act.shape[0], act.shape[1], float(limit),
                   float(slope), self._stream())
        return act

    def linear_by_group(self, a, w, out, a_stride: int, out_stride: int, a_offset: int = 0, out_offset: int = 0, out_gate=None):
        """One product per group in one launch (csrc/gemm_grouped.cu): with w [groups, n, k] and rows = out.shape[0],
        out[:, out_offset + g * out_stride : ... + n] = A_g . w[g]^T, where row r of A_g starts at element
        a_offset + g * a_stride + r * a.shape[1] of `a` (a head's slice of a wider row, or a block of rows of its own).
        `out_gate`: float32, shaped like `out`; every result number is multiplied by the sigmoid of the number at its place."""
        _check(a, "linear_by_group.a", tuple(DTYPE_CODE), 2)
        _check(w, "linear_by_group.w", a.dtype, 3)
        _check(out, "linear_by_group.out", a.dtype, 2)
        groups, n, k = w.shape
        rows, lda = out.shape[0], a.shape[1]
        _need(a_offset + (groups - 1) * a_stride + (rows - 1) * lda + k <= a.numel(), "linear_by_group: a is too small")
        _need(out_offset + (groups - 1) * out_stride + n <= out.shape[1], "linear_by_group: out is too narrow")
        if out_gate is not None:
            _check(out_gate, "linear_by_group.out_gate", torch.float32, 2)
            _need(tuple(out_gate.shape) == tuple(out.shape), "linear_by_group.out_gate: shaped like out")
        self._call("llm_gemm_grouped", _ptr(a), lda, int(a_stride), int(a_offset), None, _ptr(w), _ptr(out), out.shape[1],
                   int(out_stride), int(out_offset), DTYPE_CODE[a.dtype], rows, n, k, groups, None, 0, 0, 0.0, 0.0, None,
                   _ptr(out_gate), self._stream())
        return out

    def route_topk(self, scores, correction, chosen, weights, sigmoid: bool = False, chosen_softmax: bool = False):
        """Router outputs [T, R] float32 -> chosen [T, top] int32 (the largest s + correction, descending; correction None: of
        s) and weights [T, top] float32 (their s), where s is the softmax over the outputs, or with `sigmoid` each output's
        sigmoid.  `chosen_softmax`: the outputs themselves are compared, plus `correction` as a bias that belongs to them, and
        the weights are the softmax over the chosen outputs alone; csrc/moe_route.cu."""
        _check(scores, "route_topk.scores", torch.float32, 2)
        if correction is not None:
            _check(correction, "route_topk.correction", torch.float32, 1)
        _check(chosen, "route_topk.chosen", torch.int32, 2)
        _check(weights, "route_topk.weights", torch.float32, 2)
        tokens, outputs = scores.shape
        _need((correction is None or correction.shape[0] == outputs) and chosen.shape[0] == tokens and
              tuple(weights.shape) == tuple(chosen.shape), "route_topk: shapes do not fit")
        self._call("llm_route_topk", _ptr(scores), _ptr(correction), _ptr(chosen), _ptr(weights), tokens, outputs, chosen.shape[1],
                   2 if chosen_softmax else 1 if sigmoid else 0, self._stream())

    def moe_tile_bound(self, rows: int, experts: int) -> int:
        """The most row tiles `moe_plan` can make of `rows` (token, choice) pairs over `experts` experts."""
        return -(-rows // self.lib.llm_gemm_grouped_tile_rows()) + experts

    # (token, choice) pairs from which a step's expert products run expert by expert on the dense product kernels
    # (IITJ_MOE_DENSE_ROWS; 0: never).  Measured at 8B layer sizes, 2,048 tokens of 2 choices over 8 experts: the grouped
    # kernel's mma.sync tiles reach 150 to 190 TFLOP/s, the dense products 1,000 and more.
    moe_dense_rows = int(os.environ.get("IITJ_MOE_DENSE_ROWS", "2048"))

    def moe_plan(self, chosen, experts: int, source, place, tiles, counts=None, weights=None, row_weight=None):
        """Sorts the (token, choice) pairs of `chosen` [T, top] by expert on the device: source [T * top] (token of each
        sorted row), place [T * top] (sorted row of each pair, -1 for a choice >= experts), tiles [bound + 1, 4] (count in
        front, then (expert, first row, rows) records).  With `weights` [T, top] and `row_weight` [T * top] float32 every
        pair's weight is also left beside its sorted row.  Returns what `moe_linear` and `moe_combine` take as `plan`."""
        _check(chosen, "moe_plan.chosen", torch.int32, 2)
        for name, t in (("source", source), ("place", place)):
            _check(t, "moe_plan." + name, torch.int32, 1)
            _need(t.shape[0] == chosen.numel(), f"moe_plan.{name}: one entry per (token, choice)")
        _check(tiles, "moe_plan.tiles", torch.int32, 2)
        bound = self.moe_tile_bound(chosen.numel(), experts)
        _need(tiles.shape[1] == 4 and tiles.shape[0] >= bound + 1, "moe_plan.tiles: [tile bound + 1, 4]")
        if counts is not None:
            _check(counts, "moe_plan.counts", torch.int32, 1)
            _need(counts.shape[0] >= experts, "moe_plan.counts: one per expert")
        if row_weight is not None:
            _check(weights, "moe_plan.weights", torch.float32, 2)
            _check(row_weight, "moe_plan.row_weight", torch.float32, 1)
            _need(tuple(weights.shape) == tuple(chosen.shape) and row_weight.shape[0] == chosen.numel(), "moe_plan: one weight per pair")
        self._call("llm_moe_plan", _ptr(chosen), chosen.numel(), chosen.shape[1], int(experts),
                   self.lib.llm_gemm_grouped_tile_rows(), _ptr(source), _ptr(place), _ptr(tiles), bound, _ptr(counts),
                   _ptr(weights) if row_weight is not None else None, _ptr(row_weight), self._stream())
        return {"source": source, "place": place, "tiles": tiles, "bound": bound, "counts": counts, "row_weight": row_weight}

    def gather_rows(self, x, plan, out, weighted: bool = False):
        """out[r] = x[plan source of r] for every sorted row r of `plan` (`moe_plan`): the experts' rows side by side; `weighted`:
        times the row's weight (the plan's `row_weight`)."""
        _check(x, "gather_rows.x", tuple(DTYPE_CODE), 2)
        _check(out, "gather_rows.out", x.dtype, 2)
        _need(out.shape[1] == x.shape[1] and out.shape[0] == plan["source"].shape[0], "gather_rows: shapes do not fit")
        _need(not weighted or plan.get("row_weight") is not None, "gather_rows: the plan holds no row weights")
        self._call("llm_gather_rows", _ptr(x), _ptr(plan["source"]), plan["tiles"].data_ptr() + 4, _ptr(out), DTYPE_CODE[x.dtype],
                   out.shape[0], x.shape[1], _ptr(plan["row_weight"]) if weighted else None, self._stream())
        return out

    def moe_linear(self, a, w, out, plan, gather: bool = False, glu=False, limit: float = 0.0, slope: float = 1.0):
        """out[r] = a[row of r] . w[expert of r]^T for every sorted row r of `plan`; with `gather` a's rows are tokens
        (read through plan["source"]), else sorted rows.  `glu`: w [E, 2n, k] holds gate rows then up rows and the gate is
        applied in the epilogue: True or "clamped" the clamped form (limit, slope), "silu_weighted" silu(w g) * (w u) with
        the plan's weight w of the row (the expert's product of the row times w)."""
        _check(a, "moe_linear.a", tuple(DTYPE_CODE), 2)
        _check(w, "moe_linear.w", a.dtype, 3)
        _check(out, "moe_linear.out", a.dtype, 2)
        experts, wn, k = w.shape
        n = wn // 2 if glu else wn
        _need(a.shape[1] == k and out.shape[1] == n and out.shape[0] == plan["source"].shape[0], "moe_linear: shapes do not fit")
        form = 0 if not glu else 2 if glu == "silu_weighted" else 1
        _need(form != 2 or plan.get("row_weight") is not None, "moe_linear: the plan holds no row weights")
        self._call("llm_gemm_grouped", _ptr(a), a.shape[1], 0, 0, _ptr(plan["source"]) if gather else None, _ptr(w), _ptr(out),
                   out.shape[1], 0, 0, DTYPE_CODE[a.dtype], 0, n, k, experts, _ptr(plan["tiles"]), plan["bound"],
                   form, float(limit), float(slope), _ptr(plan["row_weight"]) if form == 2 else None, None, self._stream())
        return out

    def moe_combine(self, y, plan, chosen, weights, x, experts: int, out):
        """out[t] = sum_j weights[t, j] * (y[sorted row of (t, j)], or x[t] where chosen[t, j] >= experts), j in order;
        weights None: all 1."""
        _check(x, "moe_combine.x", tuple(DTYPE_CODE), 2)
        _check(out, "moe_combine.out", x.dtype, 2)
        _check(chosen, "moe_combine.chosen", torch.int32, 2)
        if weights is not None:
            _check(weights, "moe_combine.weights", torch.float32, 2)
        _need(out.shape == x.shape and chosen.shape[0] == x.shape[0] and
              (weights is None or tuple(weights.shape) == tuple(chosen.shape)), "moe_combine: shapes do not fit")
        if y is not None:
            _check(y, "moe_combine.y", x.dtype, 2)
            _need(y.shape[1] == x.shape[1], "moe_combine.y: width differs")
        else:
            _need(experts == 0, "moe_combine: experts without outputs")
        self._call("llm_moe_combine", _ptr(y), _ptr(plan["place"]) if plan is not None else None, _ptr(chosen), _ptr(weights),
                   _ptr(x), _ptr(out), DTYPE_CODE[x.dtype], x.shape[0], x.shape[1], chosen.shape[1], int(experts), self._stream())
        return out

    # ---- attention over flat pages (independent key and value sizes, latent rows), wkv ---------------------------
    @staticmethod
    def _flat_page_size(cache_layer, kv_heads, key_dim, value_dim, shared_value) -> int:
        per_token = kv_heads * (key_dim if shared_value else key_dim + value_dim)
        _need(cache_layer.dim() == 2 and cache_layer.shape[1] % per_token == 0,
              f"cache: a page of {tuple(cache_layer.shape)} does not hold rows of {kv_heads} heads of {key_dim} (+ {value_dim})")
        return cache_layer.shape[1] // per_token

    def latent_prepare(self, qd, tables, rotary_dim, interleaved, gain, eps, q_out, cache_layer, slots, heads, dim, rot_dim, rank,
                       kv=None):
        """From the fused projection qd [T, heads * (dim + rot_dim) + rank + rot_dim]: the latent part normed (gain [rank]
        float32) and the shared key part rotated, stored together as one cache row per token at `slots` (None: no store);
        every head's rotated query part written to q_out [T, heads * (rank + rot_dim)] behind the place of its absorbed
        part.  tables = (cos, sin) float32 [T, rotary_dim / 2]; csrc/attention_flat.cu.  With `kv` [T, rank + rot_dim] (rows
        with a stride of their own: columns of another product) qd holds the queries alone."""
        _check(qd, "latent_prepare.qd", tuple(DTYPE_CODE), 2)
        _check(q_out, "latent_prepare.q_out", qd.dtype, 2)
        _check(gain, "latent_prepare.gain", torch.float32, 1)
        tokens = qd.shape[0]
        qw = heads * (dim + rot_dim)
        if kv is None:
            _need(qd.shape[1] == qw + rank + rot_dim, "latent_prepare.qd: wrong width")
            kv_ptr, ld_kv = qd.data_ptr() + qw * qd.element_size(), qd.shape[1]
        else:
            _need(kv.dim() == 2 and kv.dtype == qd.dtype and kv.is_cuda and kv.stride(1) == 1 and
                  tuple(kv.shape) == (tokens, rank + rot_dim) and qd.shape[1] == qw, "latent_prepare.kv: [tokens, rank + rot_dim] beside queries alone")
            kv_ptr, ld_kv = kv.data_ptr(), kv.stride(0)
        _need(gain.shape[0] == rank and tuple(q_out.shape) == (tokens, heads * (rank + rot_dim)), "latent_prepare: shapes do not fit")
        cos = sin = None
        if rotary_dim:
            cos, sin = tables
            _check(cos, "latent_prepare.cos", torch.float32, 2)
            _check(sin, "latent_prepare.sin", torch.float32, 2)
            _need(cos.shape == (tokens, rotary_dim // 2) and sin.shape == cos.shape, "latent_prepare: tables must be [tokens, rotary_dim / 2]")
        page_size, stride = 1, 0
        if slots is not None:
            _check(slots, "latent_prepare.slots", torch.int32, 1)
            _check(cache_layer, "latent_prepare.cache", qd.dtype, 2)
            _need(slots.shape[0] == tokens, "latent_prepare.slots: one per token")
            page_size, stride = self._flat_page_size(cache_layer, 1, rank + rot_dim, rank, True), cache_layer.shape[1]
        self._call("llm_latent_prepare", _ptr(qd), qd.shape[1], kv_ptr, ld_kv, _ptr(cos), _ptr(sin), int(rotary_dim), 1 if interleaved else 0,
                   _ptr(gain), float(eps), _ptr(q_out), _ptr(cache_layer) if slots is not None else None, _ptr(slots), stride,
                   page_size, DTYPE_CODE[qd.dtype], tokens, heads, dim, rot_dim, rank, self._stream())

    def headnorm_store(self, qkv, q_gain, k_gain, eps, cache_layer, slots, heads, kv_heads, dim, vdim):
        """qkv [T, heads * dim + kv_heads * (dim + vdim)]: every query head (in place) and key head divided by its root
        mean square and multiplied by a gain [dim] shared by all heads (None: no norm); keys and values stored at `slots`
        in a flat-page cache (None: no store)."""
        _check(qkv, "headnorm_store.qkv", tuple(DTYPE_CODE), 2)
        tokens = qkv.shape[0]
        _need(qkv.shape[1] == heads * dim + kv_heads * (dim + vdim), "headnorm_store.qkv: wrong width")
        for name, g in (("q_gain", q_gain), ("k_gain", k_gain)):
            if g is not None:
                _check(g, "headnorm_store." + name, torch.float32, 1)
                _need(g.shape[0] == dim, f"headnorm_store.{name}: one per head dim")
        _need((q_gain is None) == (k_gain is None), "headnorm_store: both gains or none")
        page_size, stride = 1, 0
        if slots is not None:
            _check(slots, "headnorm_store.slots", torch.int32, 1)
            _check(cache_layer, "headnorm_store.cache", qkv.dtype, 2)
            _need(slots.shape[0] == tokens, "headnorm_store.slots: one per token")
            page_size, stride = self._flat_page_size(cache_layer, kv_heads, dim, vdim, False), cache_layer.shape[1]
        self._call("llm_headnorm_store", _ptr(qkv), qkv.shape[1], _ptr(q_gain), _ptr(k_gain), float(eps),
                   _ptr(cache_layer) if slots is not None else None, _ptr(slots), stride, page_size, DTYPE_CODE[qkv.dtype], tokens,
                   heads, kv_heads, dim, vdim, self._stream())

    def flat_tokens_per_tile(self, heads: int, kv_heads: int) -> int:
        """Neighbouring tokens of one request that a block of the tensor-core attention over flat pages takes."""
        return 64 // self.lib.llm_attention_flat_mma_heads_per_block(heads, kv_heads)

    def flat_key_splits(self, requests: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, shared_value: bool,
                        longest: int) -> int:
        """Over how many blocks the keys of each decoded token are shared out: as many as fill the SMs once with the blocks an
        SM holds (two, or one where a block's shared memory leaves no room for a second), each with at least eight key tiles
        of 32."""
        per = self.lib.llm_attention_flat_mma_heads_per_block(heads, kv_heads)
        blocks = requests * kv_heads * -(-(heads // kv_heads) // per) * -(-value_dim // (64 if value_dim <= 64 else 128 if value_dim <= 128 else 256))
        resident = max(1, min(2, (227 * 1024) // max(self.lib.llm_attention_flat_mma_smem(key_dim, value_dim, 1 if shared_value else 0), 1)))
        return max(1, min(32, (resident * self.sm_count) // max(blocks, 1), longest // 256))

    def attention_flat(self, q, cache_layer, meta, out, heads, kv_heads, key_dim, value_dim, shared_value: bool = False,
                       window: int = 0, scale: float = 1.0, gate=None, plan=None, softcap: float = 0.0, slopes=None,
                       q_temp=None, sinks=None):
        """Attention of every token's query heads (the leading heads * key_dim numbers of q's rows) over the flat-page
        cache of its request: keys of key_dim, values of value_dim (`shared_value`: the leading value_dim numbers of the key
        rows), a sliding window (0: all earlier keys), optionally the output times sigmoid(gate) (gate [T, heads]: a number
        per head; [T, heads * value_dim]: per output number).  Score options: `softcap` c > 0 squashes the scaled score to
        c tanh(s / c); `slopes` [heads] float32 takes slope * (query position - key position) off; `q_temp` = (coef, every)
        multiplies the query at position p by 1 + coef ln(floor((p + 1) / every) + 1); `sinks` [heads] float32 puts exp(sink) of
        the head into every row's denominator, a term without key or value that is neither scaled nor masked."""
        _check(q, "attention_flat.q", tuple(DTYPE_CODE), 2)
        if sinks is not None:
            _check(sinks, "attention_flat.sinks", torch.float32, 1)
            _need(sinks.shape[0] == heads, "attention_flat.sinks: one per head")
        _check(cache_layer, "attention_flat.cache", q.dtype, 2)
        _check(out, "attention_flat.out", q.dtype, 2)
        tokens = q.shape[0]
        _need(q.shape[1] >= heads * key_dim and tuple(out.shape) == (tokens, heads * value_dim), "attention_flat: q / out shapes do not fit")
        _check(meta.block_table, "attention_flat.block_table", torch.int32, 2)
        _check(meta.token_request, "attention_flat.token_request", torch.int32, 1)
        _check(meta.positions, "attention_flat.positions", torch.int32, 1)
        _need(meta.token_request.shape[0] == tokens and meta.positions.shape[0] == tokens,
              "attention_flat: one token_request and one position per token")
        gate_cols = 1
        if gate is not None:
            _check(gate, "attention_flat.gate", torch.float32, 2)
            _need(gate.shape[0] == tokens and gate.shape[1] in (heads, heads * value_dim),
                  "attention_flat.gate: [tokens, heads] or [tokens, heads * value_dim]")
            gate_cols = gate.shape[1] // heads
        if slopes is not None:
            _check(slopes, "attention_flat.slopes", torch.float32, 1)
            _need(slopes.shape[0] == heads, "attention_flat.slopes: one per head")
        coef, every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
        _need(every >= 0 and softcap >= 0, "attention_flat: negative softcap or temperature period")
        page_size = self._flat_page_size(cache_layer, kv_heads, key_dim, value_dim, shared_value)
        tiles = plan.device_arrays.get("tiles") if plan is not None else None
        if tiles is not None and q.dtype == torch.bfloat16 and self.flat_mma and q.shape[1] % 8 == 0 and \
                self.lib.llm_attention_flat_mma_supported(heads, kv_heads, key_dim, value_dim, 1 if shared_value else 0, cache_layer.shape[1]):
            # prompt portions and decoded tokens alike on the tensor cores (csrc/attention_flat_mma.cu)
            splits = int(getattr(plan, "splits", 1))
            part_o = part_ml = None
            if splits > 1:
                part_o = self._scratch("flat.part_o", tokens * heads * splits * value_dim, q.device)
                part_ml = self._scratch("flat.part_ml", tokens * heads * splits * 2, q.device)
            self._call("llm_attention_flat_mma", _ptr(q), q.shape[1], _ptr(cache_layer), cache_layer.shape[1], _ptr(meta.block_table),
                       meta.block_table.shape[1], _ptr(tiles), tiles.shape[0] // 4, _ptr(gate), gate_cols, _ptr(out), out.shape[1],
                       tokens, heads, kv_heads, key_dim, value_dim, 1 if shared_value else 0, page_size, int(window), float(scale),
                       float(softcap), _ptr(slopes), coef, every, splits, _ptr(part_o), _ptr(part_ml), _ptr(sinks), self._stream())
            if splits > 1:
                self.launches += 1      # the merge kernel
            return out
        self._call("llm_attention_flat", _ptr(q), q.shape[1], _ptr(cache_layer), cache_layer.shape[1], _ptr(meta.block_table),
                   meta.block_table.shape[1], _ptr(meta.token_request), _ptr(meta.positions), _ptr(gate), gate_cols, _ptr(out),
                   out.shape[1], DTYPE_CODE[q.dtype], tokens, heads, kv_heads, key_dim, value_dim, 1 if shared_value else 0, page_size,
                   int(window), float(scale), float(softcap), _ptr(slopes), coef, every, _ptr(sinks), self._stream())
        return out

    def qk_prepare(self, proj, heads, kv_heads, dim, vdim, eps, cache_layer=None, slots=None, bias=None, norm: str = "none",
                   q_gain=None, k_gain=None, norm_first: bool = True, tables=None, rotary_dim: int = 0, interleaved: bool = False,
                   own_kv: bool = True, value_from_key: bool = False):
        """Between a grouped attention's fused projection and its attention kernel (csrc/qk_prepare.cu), per token:
        proj [T, heads * dim (+ kv_heads * dim (+ kv_heads * vdim))] gets `bias` (float32, one per column) added; the values
        are the keys at that point (`value_from_key`) or the v columns; queries and keys are normed (`norm` "head": every head
        by its root mean square with gains [dim] shared by the heads, or none; "row": all of q, and all of k, at once with
        gains of that size) and their leading `rotary_dim` numbers rotated by `tables` = (cos, sin) float32 [T, rotary_dim / 2],
        the norm first or the rotation first; queries go back in place, keys and values into the flat-page cache at `slots`
        (None: no store).  `own_kv` False: proj holds queries alone."""
        _check(proj, "qk_prepare.proj", tuple(DTYPE_CODE), 2)
        tokens = proj.shape[0]
        q_cols, k_cols = heads * dim, kv_heads * dim if own_kv else 0
        v_cols = kv_heads * vdim if own_kv and not value_from_key else 0
        _need(proj.shape[1] == q_cols + k_cols + v_cols, "qk_prepare.proj: wrong width")
        _need(norm in ("none", "head", "row"), "qk_prepare: norm is none, head or row")
        if bias is not None:
            _check(bias, "qk_prepare.bias", torch.float32, 1)
            _need(bias.shape[0] >= q_cols + k_cols, "qk_prepare.bias: one per query and key column")
            _need(v_cols == 0 or bias.shape[0] == proj.shape[1], "qk_prepare.bias: one per column")
        for name, g, n in (("q_gain", q_gain, dim if norm == "head" else q_cols), ("k_gain", k_gain, dim if norm == "head" else k_cols)):
            if g is not None:
                _check(g, "qk_prepare." + name, torch.float32, 1)
                _need(norm != "none" and g.shape[0] == n, f"qk_prepare.{name}: {n} gains")
        cos = sin = None
        if rotary_dim:
            cos, sin = tables
            _check(cos, "qk_prepare.cos", torch.float32, 2)
            _check(sin, "qk_prepare.sin", torch.float32, 2)
            _need(cos.shape == (tokens, rotary_dim // 2) and sin.shape == cos.shape, "qk_prepare: tables must be [tokens, rotary_dim / 2]")
        page_size, stride = 1, 0
        if slots is not None:
            _need(own_kv, "qk_prepare: a layer without keys of its own stores nothing")
            _check(slots, "qk_prepare.slots", torch.int32, 1)
            _check(cache_layer, "qk_prepare.cache", proj.dtype, 2)
            _need(slots.shape[0] == tokens, "qk_prepare.slots: one per token")
            page_size, stride = self._flat_page_size(cache_layer, kv_heads, dim, vdim, False), cache_layer.shape[1]
        self._call("llm_qk_prepare", _ptr(proj), proj.shape[1], _ptr(bias), _ptr(q_gain), _ptr(k_gain), _ptr(cos), _ptr(sin),
                   _ptr(cache_layer) if slots is not None else None, _ptr(slots), stride, page_size, DTYPE_CODE[proj.dtype], tokens,
                   heads, kv_heads, dim, vdim, {"none": 0, "head": 1, "row": 2}[norm], 1 if norm_first else 0, int(rotary_dim),
                   1 if interleaved else 0, 1 if own_kv else 0, 1 if value_from_key else 0, float(eps), self._stream())
        return proj

    # ---- norms behind the sum, depth average, normed branches, normed polynomial activation ---------------------
    def post_norm(self, x, branch, alpha: float, gain, eps: float, out, cast_out=None, history=None, mix=None):
        """y = rmsnorm(alpha * x + branch) * gain with float32 statistics (csrc/post_norm.cu); x, out float32 [T, w] (may be the
        same), gain float32 as it multiplies.  With `history` float32 [inputs, T, w] and `mix` float32 [inputs]: y becomes the
        history's last entry and `out` receives sum_j mix[j] * history[j].  `cast_out`: what `out` got, in another type."""
        _check(x, "post_norm.x", torch.float32, 2)
        _check(out, "post_norm.out", torch.float32, 2)
        _check(branch, "post_norm.branch", tuple(DTYPE_CODE), 2)
        _check(gain, "post_norm.gain", torch.float32, 1)
        tokens, width = x.shape
        _need(tuple(branch.shape) == (tokens, width) and tuple(out.shape) == (tokens, width) and gain.shape[0] == width,
              "post_norm: shapes differ")
        if cast_out is not None:
            _check(cast_out, "post_norm.cast_out", tuple(DTYPE_CODE), 2)
            _need(cast_out.shape == x.shape, "post_norm.cast_out: shape differs")
        inputs = 0
        if history is not None:
            _check(history, "post_norm.history", torch.float32, 3)
            _check(mix, "post_norm.mix", torch.float32, 1)
            inputs = mix.shape[0]
            _need(history.shape[0] >= inputs >= 1 and tuple(history.shape[1:]) == (tokens, width), "post_norm.history: [inputs, T, w]")
        self._call("llm_post_norm", _ptr(x), _ptr(branch), DTYPE_CODE[branch.dtype], float(alpha), _ptr(gain), float(eps), _ptr(out),
                   _ptr(cast_out), DTYPE_CODE[cast_out.dtype] if cast_out is not None else 0, _ptr(history), _ptr(mix), inputs,
                   tokens * width, tokens, width, self._stream())
        return out

    def branch_mean(self, branches, gains, scale: float, eps: float, out):
        """out (float32) = scale * sum_b rmsnorm(branches[b]) * gains[b], one to four branches of the engine's type."""
        _need(1 <= len(branches) <= 4 and len(gains) == len(branches), "branch_mean: one to four branches, a gain vector each")
        _check(out, "branch_mean.out", torch.float32, 2)
        for b, g in zip(branches, gains):
            _check(b, "branch_mean.branch", branches[0].dtype, 2)
            _check(g, "branch_mean.gain", torch.float32, 1)
            _need(b.shape == out.shape and g.shape[0] == out.shape[1], "branch_mean: shapes differ")
        _need(branches[0].dtype in DTYPE_CODE, "branch_mean: branches of one of the engine's types")
        n = len(branches)
        bp = (ctypes.c_void_p * n)(*[b.data_ptr() for b in branches])
        gp = (ctypes.c_void_p * n)(*[g.data_ptr() for g in gains])
        self._call("llm_branch_mean", ctypes.cast(bp, ctypes.c_void_p), ctypes.cast(gp, ctypes.c_void_p), n,
                   DTYPE_CODE[branches[0].dtype], float(scale), float(eps), _ptr(out), out.shape[0], out.shape[1], self._stream())
        return out

    def poly_norm(self, z, coef, eps: float, act):
        """act = a N(z) + b N(z^2) + c N(z^3) + e over every row of z, N dividing a row by its root mean square; coef float32 [4]."""
        _check(z, "poly_norm.z", tuple(DTYPE_CODE), 2)
        _check(act, "poly_norm.act", z.dtype, 2)
        _check(coef, "poly_norm.coef", torch.float32, 1)
        _need(act.shape == z.shape and coef.shape[0] == 4, "poly_norm: shapes do not fit")
        self._call("llm_poly_norm", _ptr(z), _ptr(coef), float(eps), _ptr(act), DTYPE_CODE[z.dtype], z.shape[0], z.shape[1], self._stream())
        return act

    # ---- gated linear recurrence ------------------------------------------------------------------------------------
    def lru(self, proj, y_col: int, x_col: int, width: int, bias_y, bias_x, taps_w, conv_bias, ra, ri, ra_bias, ri_bias, lam,
            decay_scale: float, state, state_slots, token_request, cu_seqlens, out, longest: int, write: bool = True):
        """A gated linear recurrence per channel with its short convolution (csrc/lru.cu): proj [T, ld] holds the gate branch's
        projection at columns [y_col, y_col + width) and the input branch's at [x_col, ...); state float32 [slots, taps, width]
        (row 0 the recurrence's state, then the last taps - 1 inputs of the convolution); out [T, width] of proj's type."""
        _check(proj, "lru.proj", tuple(DTYPE_CODE), 2)
        _check(out, "lru.out", proj.dtype, 2)
        tokens = proj.shape[0]
        _need(max(y_col, x_col) + width <= proj.shape[1] and tuple(out.shape) == (tokens, width), "lru: proj / out shapes do not fit")
        _check(taps_w, "lru.taps", torch.float32, 2)
        taps = taps_w.shape[1]
        _need(taps_w.shape[0] == width, "lru.taps: one row per channel")
        for name, t in (("bias_y", bias_y), ("bias_x", bias_x), ("conv_bias", conv_bias), ("ra_bias", ra_bias), ("ri_bias", ri_bias), ("lam", lam)):
            if t is not None:
                _check(t, "lru." + name, torch.float32, 1)
                _need(t.shape[0] == width, f"lru.{name}: one per channel")
        _need(ra_bias is not None and ri_bias is not None and lam is not None, "lru: gate biases and decay parameters are needed")
        _check(ra, "lru.ra", proj.dtype, 3)
        _check(ri, "lru.ri", proj.dtype, 3)
        blocks = ra.shape[0]
        _need(width % blocks == 0 and tuple(ra.shape) == (blocks, width // blocks, width // blocks) and ri.shape == ra.shape,
              "lru: gate matrices are [blocks, width / blocks, width / blocks]")
        _check(state, "lru.state", torch.float32, 3)
        _need(tuple(state.shape[1:]) == (taps, width), "lru.state: [slots, taps, width]")
        for name, t in (("state_slots", state_slots), ("token_request", token_request), ("cu_seqlens", cu_seqlens)):
            _check(t, "lru." + name, torch.int32, 1)
        requests = state_slots.shape[0]
        _need(token_request.shape[0] == tokens and cu_seqlens.shape[0] == requests + 1, "lru: index arrays do not fit")
        code = DTYPE_CODE[proj.dtype]
        if longest == 1 and self.lru_step:
            # single tokens: convolution, gates, recurrence and the state's update in one launch
            self._call("llm_lru_step", _ptr(proj), proj.shape[1], int(y_col), int(x_col), _ptr(bias_y), _ptr(bias_x), _ptr(taps_w),
                       _ptr(conv_bias), taps, _ptr(ra), _ptr(ri), _ptr(ra_bias), _ptr(ri_bias), _ptr(lam), float(decay_scale), _ptr(state),
                       _ptr(state_slots), _ptr(cu_seqlens), _ptr(out), code, requests, width, blocks, 1 if write else 0, self._stream())
            return out
        u = self._scratch("lru.u", tokens * width, proj.device)
        a = self._scratch("lru.a", tokens * width, proj.device)
        b = self._scratch("lru.b", tokens * width, proj.device)
        self._call("llm_lru_conv", _ptr(proj), proj.shape[1], int(x_col), _ptr(bias_x), _ptr(taps_w), _ptr(conv_bias), taps, _ptr(state),
                   _ptr(state_slots), _ptr(token_request), _ptr(cu_seqlens), _ptr(u), code, tokens, width, self._stream())
        self._call("llm_lru_gates", _ptr(u), _ptr(ra), _ptr(ri), _ptr(ra_bias), _ptr(ri_bias), _ptr(lam), float(decay_scale), _ptr(a),
                   _ptr(b), code, tokens, width, blocks, self._stream())
        seg = self.lib.llm_lru_segment()
        scratch = None
        if longest > seg:
            scratch = self._scratch("lru.segments", 2 * requests * -(-longest // seg) * width, proj.device)
            self.launches += 2
        self._call("llm_lru_scan", _ptr(a), _ptr(b), _ptr(proj), proj.shape[1], int(y_col), int(x_col), _ptr(bias_y), _ptr(bias_x), taps,
                   _ptr(state), _ptr(state_slots), _ptr(cu_seqlens), _ptr(out), code, requests, width, int(longest), 1 if write else 0,
                   _ptr(scratch), self._stream())
        return out

    def token_shift(self, x, mu, before, state_slots, token_request, cu_seqlens, out):
        """out [streams * T, width]: m_s = x + (x' - x) * mu_s, mu [streams * width] float32, x' the row before (a request's
        first row of the step: before[its state slot], float32 [slots, width]); csrc/wkv.cu."""
        _check(x, "token_shift.x", tuple(DTYPE_CODE), 2)
        _check(mu, "token_shift.mu", torch.float32, 1)
        _check(before, "token_shift.before", torch.float32, 2)
        _check(out, "token_shift.out", x.dtype, 2)
        tokens, width = x.shape
        streams = mu.shape[0] // width
        _need(mu.shape[0] == streams * width and tuple(out.shape) == (streams * tokens, width) and before.shape[1] == width,
              "token_shift: shapes do not fit")
        for name, t in (("state_slots", state_slots), ("token_request", token_request), ("cu_seqlens", cu_seqlens)):
            _check(t, "token_shift." + name, torch.int32, 1)
        _need(token_request.shape[0] == tokens and cu_seqlens.shape[0] == state_slots.shape[0] + 1, "token_shift: index arrays do not fit")
        self._call("llm_token_shift", _ptr(x), _ptr(mu), _ptr(before), _ptr(state_slots), _ptr(token_request), _ptr(cu_seqlens),
                   _ptr(out), DTYPE_CODE[x.dtype], tokens, width, streams, self._stream())
        return out

    def wkv_decay(self, low, w2, w0, out):
        """out[t, c] = exp(-exp(w2[c] . tanh(low[t]) + w0[c])), all float32."""
        for name, t, d in (("low", low, 2), ("w2", w2, 2), ("w0", w0, 1), ("out", out, 2)):
            _check(t, "wkv_decay." + name, torch.float32, d)
        tokens, rank = low.shape
        _need(w2.shape[1] == rank and w0.shape[0] == w2.shape[0] and tuple(out.shape) == (tokens, w2.shape[0]), "wkv_decay: shapes do not fit")
        self._call("llm_wkv_decay", _ptr(low), _ptr(w2), _ptr(w0), _ptr(out), tokens, w2.shape[0], rank, self._stream())
        return out

    def wkv_scan(self, rkvg, decay, u, gain, eps, state, state_slots, cu_seqlens, out, heads, dim, write: bool = True,
                 last_rows=None):
        """The wkv walk with head norm, gain and gate (csrc/wkv.cu): rkvg [4 * T, heads * dim] (the rows of r, then k, v, g), decay
        [T, heads * dim] float32, u [heads, dim], gain [heads * dim], state [slots, heads, dim, dim] float32 (read, and with
        `write` left at the step's last token).  last_rows = (x [T, width], before [slots, width]): each request's last row of
        x becomes its row in `before`."""
        _check(rkvg, "wkv_scan.rkvg", tuple(DTYPE_CODE), 2)
        _check(out, "wkv_scan.out", rkvg.dtype, 2)
        for name, t, d in (("decay", decay, 2), ("u", u, 2), ("gain", gain, 1), ("state", state, 4)):
            _check(t, "wkv_scan." + name, torch.float32, d)
        tokens, n = rkvg.shape[0] // 4, heads * dim
        _need(tuple(rkvg.shape) == (4 * tokens, n) and tuple(decay.shape) == (tokens, n) and tuple(out.shape) == (tokens, n) and
              tuple(u.shape) == (heads, dim) and gain.shape[0] == n and tuple(state.shape[1:]) == (heads, dim, dim),
              "wkv_scan: shapes do not fit")
        _check(state_slots, "wkv_scan.state_slots", torch.int32, 1)
        _check(cu_seqlens, "wkv_scan.cu_seqlens", torch.int32, 1)
        _need(cu_seqlens.shape[0] == state_slots.shape[0] + 1, "wkv_scan.cu_seqlens: requests + 1 entries")
        x = before = None
        width = 0
        if last_rows is not None:
            x, before = last_rows
            _check(x, "wkv_scan.x", rkvg.dtype, 2)
            _check(before, "wkv_scan.before", torch.float32, 2)
            width = x.shape[1]
            _need(x.shape[0] == tokens and before.shape[1] == width, "wkv_scan.last_rows: shapes do not fit")
        self._call("llm_wkv_scan", _ptr(rkvg), _ptr(decay), _ptr(u), _ptr(gain), float(eps), _ptr(state), _ptr(state_slots),
                   _ptr(cu_seqlens), _ptr(out), DTYPE_CODE[rkvg.dtype], tokens, state_slots.shape[0], heads, dim, 1 if write else 0,
                   _ptr(x), _ptr(before), width, self._stream())
        return out

    # ---- matrix products -------------------------------------------------------------
    def prefill_key_splits(self, big_rows, heads, kv_heads, window) -> int:
        """CTAs along the keys of each 128-query tile of the tcgen05 prefill attention.  The kernel is at its best
        with two heads per CTA and about 1.7 CTAs per SM; a short portion of a prompt against a long context has
        too few query tiles for that, so its keys are shared out.  This is the number of CTAs the launch provides
        per tile and head; the kernel uses as many of them as leave each about 16 key tiles of 128, by the tile's
        own context (a captured graph thus follows a prompt as it grows).
        Measured at 32 heads / 8 key-value heads: 512 queries over 16384 keys 260 -> 209 us with 4 splits, over
        32768 keys 510 -> 352 us; 128 queries over 16384 keys 254 -> 86 us."""
        if self.attention_splits is not None:
            return max(1, min(16, int(self.attention_splits)))
        longest = max(min(pos0 + rows, window + rows) if window > 0 else pos0 + rows for _, rows, pos0, _ in big_rows)
        if longest < self.LONG_PREFILL:               # no tile would use a second split: no merge kernel either
            return 1
        group = heads // kv_heads
        pair_ctas = len(big_rows) * kv_heads * ((group + 1) // 2)
        splits = max(1, min(16, round(1.7 * self.sm_count / pair_ctas)))
        if pair_ctas * splits < self.sm_count:        # too few even so: the kernel then runs one head per CTA
            splits = max(1, min(16, self.sm_count // (len(big_rows) * heads)))
        return splits

    # Context from which a query tile's keys may be shared out over two CTAs (24 key tiles of 128).  A step's
    # captured graph freezes whether its prefill attention launches splits at all, so the step function keeps
    # shorter and longer contexts apart in its graph keys.
    LONG_PREFILL = 3072

    def linear(self, x, weight, out, swiglu: bool = False, defer: bool = False):
        """out = x . weight^T; with swiglu, weight holds gate rows then up rows and
        out = silu(x . gate^T) * (x . up^T).  With `defer` the result may come back as a PartialSums (the product
        was split along k and the caller's next kernel adds the parts); else `out`."""
        _check(x, "linear.x", tuple(DTYPE_CODE), 2)
        _check(weight, "linear.weight", x.dtype, 2)
        _check(out, "linear.out", (x.dtype, torch.float32), 2)
        n = weight.shape[0] // 2 if swiglu else weight.shape[0]
        _need(x.shape[1] == weight.shape[1], f"linear: x has {x.shape[1]} columns, weight {weight.shape[1]}")
        _need(out.shape == (x.shape[0], n), f"linear.out: shape {tuple(out.shape)}, want {(x.shape[0], n)}")
        if x.shape[0] == 0:
            return out
        if x.dtype == torch.float32:
            self._call("llm_gemm_f32", _ptr(x), _ptr(weight), _ptr(out), x.shape[0], n, x.shape[1], x.shape[1],
                       weight.shape[1], n, 1 if swiglu else 0, self._stream())
            return out
        # bfloat16: this library's tcgen05 kernel where it is the faster one, else cuBLAS through torch
        tokens, k = x.shape
        # which kernel, and how it is cut, depends on the shape alone: decided once per shape
        pkey = (tokens, n, k, swiglu)
        plan = self._linear_plans.get(pkey)
        if plan is None:
            policy = self.gemm_policy(tokens, n, k, swiglu)
            if policy == "tcgen05":
                if swiglu and tokens <= self.swiglu_half_tokens and n % 64 == 0:
                    # decode batches: 64 gate + 64 up rows per CTA, twice the CTAs (two per SM), no k-split and no kernel
                    # after it.  Against the whole tile (128 + 128 rows, one CTA per SM, 112 CTAs at the 8B shape) a decode
                    # step at 4096-token contexts: batch 16 / 32 at the 8B shape 4.61 -> 4.57 / 5.98 -> 5.93 ms, batch 32 / 64
                    # at the 3B shape 4.43 -> 4.31 / 7.54 -> 7.42 ms, at the 1B shape 1.97 -> 1.88 / 3.11 -> 3.03 ms; level at
                    # batch 64 of the 8B shape and at batch 128, where the whole tile stays
                    plan = ("tcgen05", 1, self.swiglu_half_smem_kb, True)
                else:
                    plan = ("tcgen05",) + tuple(self.gemm_plan(tokens, n, k, swiglu)) + (False,)
            else:
                plan = (policy, 1, 0, False)
            if len(self._linear_plans) > 8192:
                self._linear_plans.clear()
            self._linear_plans[pkey] = plan
        policy, splits, smem_kb, half = plan
        if policy == "tcgen05":
            if half:
                return self.gemm_tcgen05(x, weight, out, True, 1, smem_kb, half=True)
            return self.gemm_tcgen05(x, weight, out, swiglu, splits, smem_kb, defer=defer and not swiglu and self.defer_sums)
        if policy == "pair":
            return self.gemm_pair(x, weight, out, swiglu)
        if swiglu:
            # the [tokens, 2 * inner] intermediate lives in this library's grow-only scratch: a step allocates nothing
            gu = self._scratch_bf16("gemm.gate_up", tokens * weight.shape[0], x.device).view(tokens, weight.shape[0])
            torch.mm(x, weight.t(), out=gu)
            return self.silu_mul(gu, out)
        if out.dtype == torch.float32:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            torch.mm(x, weight.t(), out=out)
        return out

    def gemm_tcgen05(self, x, weight, out, swiglu: bool = False, splits: int = 1, smem_kb: int = 0, defer: bool = False,
                     half: bool = False):
        """out = x . weight^T on this library's tcgen05 kernel (bfloat16 in, bfloat16 or float32 out).  With `defer`
        and more than one split the partial sums are returned as a PartialSums instead of being added here.
        `half`: the SwiGLU product of at most 128 tokens with 64 gate and 64 up rows per CTA (unsplit, n % 64 == 0)."""
        _check(x, "gemm.x", torch.bfloat16, 2)
        _check(weight, "gemm.weight", torch.bfloat16, 2)
        _check(out, "gemm.out", (torch.bfloat16, torch.float32), 2)
        tokens, k = x.shape
        n = weight.shape[0] // 2 if swiglu else weight.shape[0]
        _need(weight.shape[1] == k and out.shape == (tokens, n), "gemm: shapes do not fit")
        splits = max(1, min(int(splits), -(-k // 64)))
        scratch = None
        if splits > 1:
            scratch = self._scratch("gemm.partials", splits * tokens * weight.shape[0], x.device)
        defer = bool(defer and splits > 1 and not swiglu)
        self._call("llm_gemm_bf16", _ptr(x), _ptr(weight), _ptr(out), 1 if out.dtype == torch.float32 else 0, tokens,
                   n, k, out.shape[1], 1 if swiglu else 0, splits, _ptr(scratch), int(smem_kb), 1 if defer else 0,
                   1 if half else 0, self._stream())
        if defer:
            return PartialSums(self, scratch[:splits * tokens * n].view(splits, tokens, n), out)
        if splits > 1:
            self.launches += 1
        return out

    def sum_parts(self, parts, out):
        """out = the sum over the first dimension of `parts` [splits, tokens, n] float32, added in split order."""
        _check(parts, "sum_parts.parts", torch.float32, 3)
        _check(out, "sum_parts.out", tuple(DTYPE_CODE), 2)
        _need(tuple(parts.shape[1:]) == tuple(out.shape), "sum_parts: shapes do not fit")
        self._call("llm_sum_parts", _ptr(parts), _ptr(out), DTYPE_CODE[out.dtype], parts.shape[0], out.numel(), self._stream())
        return out

    def scale_(self, x, scale: float):
        """x *= scale, float32, in place."""
        _check(x, "scale_.x", torch.float32)
        self._call("llm_scale_f32", _ptr(x), float(scale), x.numel(), self._stream())
        return x

    def gemm_pair(self, x, weight, out, swiglu: bool = False, tail_split: bool = True):
        """out = x . weight^T on this library's persistent CTA-pair tcgen05 kernel (many tokens).  With
        `tail_split` the tiles of the last, partly filled round are cut along k over all clusters."""
        _check(x, "gemm.x", torch.bfloat16, 2)
        _check(weight, "gemm.weight", torch.bfloat16, 2)
        _check(out, "gemm.out", (torch.bfloat16, torch.float32), 2)
        tokens, k = x.shape
        n = weight.shape[0] // 2 if swiglu else weight.shape[0]
        _need(weight.shape[1] == k and out.shape == (tokens, n), "gemm: shapes do not fit")
        partials = counters = None
        if tail_split:
            partials = self._scratch("gemm.pair.partials", self.lib.llm_gemm_bf16_pair_scratch(0), x.device)
            counters = self._pair_counters.get(x.device)
            if counters is None:      # zeroed once; every launch leaves them zero again
                counters = torch.zeros(self.lib.llm_gemm_bf16_pair_scratch(1), dtype=torch.int32, device=x.device)
                self._pair_counters[x.device] = counters
        self._call("llm_gemm_bf16_pair", _ptr(x), _ptr(weight), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                   tokens, n, k, out.shape[1], 1 if swiglu else 0, _ptr(partials), _ptr(counters), self._stream())
        return out

    # Which kernel multiplies: "tcgen05" (this library) or "cublas".  `gemm_backend` may force one.
    def gemm_policy(self, tokens, n, k, swiglu) -> str:
        """"tcgen05" (one CTA per tile, weights on the 128-row side), "pair" (persistent CTA pairs, tokens on
        the 256-row side) or "cublas".  Measured on B200 at the 8B shapes, in CUDA graphs with cold weights:
        up to 32 tokens the tcgen05 product with two or three CTAs per SM and up to eight k-splits matches
        or beats cuBLAS for every shape of the model (and its weight prefetch overlaps the kernel before
        it); from there to 128 tokens it is 5-17 % behind by itself, but its k-split sums are added by the
        kernels that read them and the decode attention takes them with the rotation fused in, so the whole
        decode step is 3-5 % faster with it (batch 48 / 64 / 128 at 8192-token contexts: 12.4 -> 11.8, 15.3 ->
        14.9, 27.7 -> 26.9 ms); beyond 128 tokens cuBLAS wins (batch 192: 14.6 against 15.2 ms).  The fused
        SwiGLU form holds up to 128 tokens.  From about 640 tokens the pair kernel's fused
        SwiGLU product beats cuBLAS plus a separate activation kernel (2048 tokens: 330 against 365 us).  Its
        plain products stay about 7 % behind cuBLAS, which halves its operand traffic with multicast loads
        that this library does not use, so those stay on cuBLAS (IITJ_GEMM_PAIR=all moves them over)."""
        if k % 8:
            return "cublas"
        if self.gemm_backend != "auto":
            return self.gemm_backend
        if tokens <= (self.gemm_small_tokens if swiglu else min(self.gemm_plain_tokens, self.gemm_small_tokens)):
            return "tcgen05"
        if tokens >= 640 and (self.gemm_pair_mode == "all" or (swiglu and self.gemm_pair_mode == "swiglu")):
            return "pair"
        return "cublas"

    def gemm_plan(self, tokens, n, k, swiglu) -> tuple:
        """(k-splits, shared memory per CTA in KiB) for the tcgen05 product.

        Products with many feature tiles (the LM head) run unsplit with three CTAs per SM.  Products with
        few tiles are split along k until about two CTAs per SM are in flight (at most eight splits, at
        least four k-blocks each).  The SwiGLU product beyond the half-tile form's token count (see linear) runs
        unsplit with the whole shared memory as its ring."""
        tile = self.lib.llm_gemm_bf16_token_tile(tokens)
        tiles = -(-n // 128) * -(-tokens // tile)
        k_blocks = -(-k // 64)
        if tokens > 256 or n % 4:
            return 1, 0
        if tiles >= 2 * self.sm_count:
            return 1, 66
        if swiglu and tokens > 8:
            return 1, 0
        splits = max(1, min(8, round(2 * self.sm_count / tiles), k_blocks // 4))
        return splits, 100

    def gemm_splits(self, tokens, n, k, swiglu) -> int:
        return self.gemm_plan(tokens, n, k, swiglu)[0]

    def gemm_status(self) -> int:
        """0, or a code if a tcgen05 GEMM gave up waiting on one of its barriers since the last call."""
        return self.lib.llm_gemm_bf16_status()

    def wait_probe(self, polls: int = 2000) -> None:
        """Launches a kernel whose only act is a bounded wait that runs out after `polls` polls (an mbarrier nobody
        arrives on; nothing else is in flight); it leaves code 7 in the tcgen05 product's status word.  For tests of
        what the host makes of a kernel that gave up."""
        self._call("llm_gemm_bf16_wait_probe", int(polls), self._stream())

    def gemm_pair_status(self) -> int:
        """0, or a code if the CTA-pair GEMM gave up waiting on one of its barriers since the last call."""
        return self.lib.llm_gemm_bf16_pair_status()

    def attention_status(self) -> int:
        """0, or a code if the tcgen05 attention kernel gave up waiting on a barrier since the last call."""
        return self.lib.llm_attention_tcgen05_status()

    def decode_status(self) -> int:
        """0, or a code if a decode attention call since the last read was given too few splits for an item's keys."""
        return self.lib.llm_attention_decode_status()

    HEALTH_WORDS = len(HEALTH_WORDS)

    def check_health(self, codes=None) -> None:
        """Raises KernelError if a kernel of this library reported that it gave up (a bounded wait that ran out) or
        that a contract was broken since the last check; what such a kernel wrote cannot be used.  `codes`: the
        words as `sample(..., health=...)` copied them out; None reads them from the device now (which waits for
        the work in flight).  On a failure the device words are cleared and the CTA-pair product's tile counters,
        which a CTA that gave up may have left non-zero, are zeroed again, so the library can be used afterwards."""
        if codes is None:
            codes = [self.gemm_status(), self.gemm_pair_status(), self.attention_status(), self.decode_status()]
        codes = [int(c) for c in codes]
        if not any(codes):
            return
        self.gemm_status(), self.gemm_pair_status(), self.attention_status(), self.decode_status()   # read = clear
        for counters in self._pair_counters.values():
            counters.zero_()
        bad = [f"{name}: code {c >> 16} in block/item {c & 0xffff} ({meaning})"
               for c, (name, meaning) in zip(codes, HEALTH_WORDS) if c]
        raise KernelError("a kernel gave up, its output is not valid: " + "; ".join(bad))

    def gather_tokens(self, dst, src, rows):
        """dst[i] = src[rows[i]] where rows[i] >= 0 (int32 device tensors): the previous step's sampled ids
        become this step's input tokens without a trip to the host."""
        _check(dst, "gather_tokens.dst", torch.int32, 1)
        _check(src, "gather_tokens.src", torch.int32, 1)
        _check(rows, "gather_tokens.rows", torch.int32, 1)
        _need(rows.shape[0] == dst.shape[0], "gather_tokens: one source row per destination")
        self._call("llm_gather_tokens", _ptr(dst), _ptr(src), _ptr(rows), dst.shape[0], self._stream())

    # ---- sampling --------------------------------------------------------------------
    def sample(self, logits, temperature, keys, out, health=None):
        """out[r] = argmax of row r (temperature[r] <= 0) or a draw from softmax(row / T).  `health`: an int32 tensor
        of HEALTH_WORDS entries that receives the library's status words (see `check_health`)."""
        _check(logits, "sample.logits", torch.float32, 2)
        _check(out, "sample.out", torch.int32, 1)
        rows = logits.shape[0]
        _need(out.shape[0] == rows, "sample.out: one per row")
        if temperature is not None:
            _check(temperature, "sample.temperature", torch.float32, 1)
            _check(keys, "sample.keys", torch.int64, 1)
            _need(temperature.shape[0] == rows and keys.shape[0] == rows, "sample: one temperature and key per row")
        if health is not None:
            _check(health, "sample.health", torch.int32, 1)
            _need(health.shape[0] >= self.HEALTH_WORDS, "sample.health: too short")
        need = self.lib.llm_sample_scratch_floats(rows, logits.shape[1])
        scratch = self._scratch("sample.part", need, logits.device) if need else None
        self._call("llm_sample", _ptr(logits), logits.shape[1], _ptr(temperature), _ptr(keys), _ptr(out), rows,
                   logits.shape[1], _ptr(scratch), _ptr(health), self._stream())
        return out


_lock = threading.Lock()
_instance = None


def load() -> Kernels:
    """The process-wide kernel set; builds and loads the library on first call."""
    global _instance
    with _lock:
        if _instance is None:
            if not torch.cuda.is_available():
                raise KernelError("no CUDA device is visible: this engine runs on the GPU only "
                                  "(there is no CPU path)")
            k = Kernels(_build.library_path())
            k.check_device()
            _instance = k
        return _instance
