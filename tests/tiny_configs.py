"""The two tiny LFM2 configurations of the test-suite and helpers to make model folders.

They differ in every size and option: layer order and count, hidden size, heads and
groups (2 and 3 query heads per KV head), head size, feed-forward width (no power of
two), taps, conv bias, vocabulary, rope theta, eps, tied or untied head.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

TINY_A = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "num_hidden_layers": 4, "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 192, "block_auto_adjust_ff_dim": False, "block_multiple_of": 32,
    "conv_L_cache": 3, "conv_bias": False, "vocab_size": 256, "rope_theta": 10000.0,
    "norm_eps": 1e-5, "max_position_embeddings": 4096, "tie_embedding": True,
}

TINY_B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "num_hidden_layers": 6,
    "layer_types": ["full_attention", "conv", "full_attention", "conv", "conv", "full_attention"],
    "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "intermediate_size": 320, "block_auto_adjust_ff_dim": False, "block_multiple_of": 32,
    "conv_L_cache": 4, "conv_bias": True, "vocab_size": 384, "rope_theta": 1000000.0,
    "norm_eps": 1e-6, "max_position_embeddings": 4096, "tie_embedding": False,
}

TINY = {"A": TINY_A, "B": TINY_B}


def make_model_dir(path, config: dict, seed: int, preset: str = "unit",
                   dtype: torch.dtype = torch.float32, edit=None) -> Path:
    """Write config.json + model.safetensors with seeded random weights through the
    framework's own random-weights mode.  ``edit(tensors)`` may change tensors first."""
    from flyweight_b200.config import architecture_name, lookup
    from flyweight_b200.parts import Precision
    from flyweight_b200.weights import random_tensors, write_model_dir
    import flyweight_b200.models  # noqa: F401

    arch = lookup(architecture_name(config))
    typed = arch.config_class.from_dict(config)
    model = arch.model_class(typed, Precision("float32"), torch.device("cpu"))
    tensors = random_tensors(model.declare(), seed, preset, dtype, "cpu")
    if edit is not None:
        edit(tensors)
    return write_model_dir(path, typed.to_dict(), tensors, seed)


def _latent(heads, dim, rot_dim, vdim, kv_rank, base, scale, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "rot": {"base": base, "dims": rot_dim}, "scale": scale}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def _kemitar_layer(mixer, ff):
    return {"type": "latent_attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# Two tiny Kemitar configurations that differ in every size and option: head counts (1 to 20), plain /
# rotated / value widths that are all different, latent ranks (one odd), cache rows that need padding,
# layers that read the rows of a layer one or two places back, layers without a feed-forward, a pair
# table of one bucket, multipliers of 1, a width that is no multiple of 8.
KEMITAR_A = {
    "architecture": "Kemitar", "vocab": 211, "width": 80, "norm": {"eps": 1e-6},
    "embedding": {"scale": 3.0, "bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 5}},
    "layers": [
        _kemitar_layer(_latent(3, 24, 8, 16, 40, 1000.0, 0.3), 144),
        _kemitar_layer(_latent(5, 16, 8, 24, 40, 1000.0, 0.2, kv_from=0), None),
        _kemitar_layer(_latent(2, 8, 8, 40, 40, 1000.0, 0.5, kv_from=0), 112),
        _kemitar_layer(_latent(2, 8, 4, 8, 20, 50.0, 0.4), 96),
    ],
}

KEMITAR_B = {
    "architecture": "Kemitar", "vocab": 130, "width": 82, "norm": {"eps": 1e-5},
    "embedding": {"scale": 1.0, "bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 1}},
    "layers": [
        _kemitar_layer(_latent(1, 10, 6, 12, 37, 300000.0, 0.25), 50),
        _kemitar_layer(_latent(20, 16, 16, 8, 48, 10000.0, 0.18), None),
        _kemitar_layer(_latent(17, 12, 16, 4, 48, 10000.0, 0.22, kv_from=1), 200),
    ],
}

# One head count in every layer (the native step plan cuts a step's prompts into row tiles once for all
# layers), a cache row of 96 + 32 = 128 entries, a layer that reads the rows of the one before.
KEMITAR_C = {
    "architecture": "Kemitar", "vocab": 300, "width": 128, "norm": {"eps": 1e-5},
    "embedding": {"scale": 2.0, "bigram": {"buckets": 61, "mul_prev": 13, "mul_cur": 3}},
    "layers": [
        _kemitar_layer(_latent(4, 32, 32, 16, 96, 10000.0, 0.125), 256),
        _kemitar_layer(_latent(4, 16, 32, 32, 96, 10000.0, 0.15, kv_from=0), None),
        _kemitar_layer(_latent(4, 16, 16, 16, 40, 500.0, 0.2), 192),
    ],
}

# Twenty heads in every layer: more than one group of sixteen shares the cached row.
KEMITAR_D = {
    "architecture": "Kemitar", "vocab": 180, "width": 96, "norm": {"eps": 1e-5},
    "embedding": {"scale": 1.5, "bigram": {"buckets": 29, "mul_prev": 7, "mul_cur": 11}},
    "layers": [
        _kemitar_layer(_latent(20, 16, 16, 8, 48, 10000.0, 0.18), 128),
        _kemitar_layer(_latent(20, 8, 16, 16, 48, 10000.0, 0.2, kv_from=0), 160),
    ],
}

TINY.update({"KA": KEMITAR_A, "KB": KEMITAR_B, "KC": KEMITAR_C, "KD": KEMITAR_D})


def _chunk_attention(heads, kv_heads, dim, vdim, chunk, base, rot_dims, scale, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
             "rot": {"base": base, "dims": rot_dims}, "mask": {"size": chunk}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _experts(ff, experts, identity, top, groups=None, keep=None):
    router = {"experts": experts, "identity": identity, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


# Three tiny Diforax configurations that differ in every size and option: the order of the layers (a
# delta rule first, attention first), head counts and groups (1 to 4 query heads per key head), query
# and value sizes that differ both ways, partial and full rotation, chunks shorter than, equal to and
# longer than a page, a layer that reads another's keys under a chunk of its own, layers without a
# feed-forward, taps from 2 to 4, state sizes that fill no warp, routers with and without identity
# experts and groups, top 1.
DIFORAX_A = {
    "architecture": "Diforax", "vocab": 211, "width": 80, "norm": {"eps": 1e-5},
    "layers": [
        {**_delta(4, 2, 16, 24, 4), "mlp": _experts(48, 6, 2, 3, groups=4, keep=2)},
        {**_chunk_attention(6, 3, 32, 16, 48, 10000.0, 16, 0.2), "mlp": _dense(144)},
        {**_chunk_attention(6, 3, 32, 16, 37, 10000.0, 16, 0.3, kv_from=1), "mlp": None},
        {**_delta(2, 2, 8, 8, 2), "mlp": _dense(112)},
    ],
}

DIFORAX_B = {
    "architecture": "Diforax", "vocab": 130, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {**_chunk_attention(4, 1, 16, 48, 64, 500.0, 16, 0.25), "mlp": _experts(40, 5, 0, 1)},
        {**_delta(3, 1, 40, 20, 3), "mlp": None},
        {**_chunk_attention(2, 2, 64, 64, 100, 1000000.0, 32, 0.11), "mlp": _experts(24, 3, 3, 4, groups=3, keep=2)},
    ],
}

# Head sizes and group widths that the tensor-core attention kernels take, so that the bfloat16 path
# runs them: 128 channels, four query heads per key head.
DIFORAX_C = {
    "architecture": "Diforax", "vocab": 300, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        {**_chunk_attention(8, 2, 128, 128, 130, 10000.0, 64, 0.09), "mlp": _dense(256)},
        {**_delta(4, 2, 64, 128, 4), "mlp": _experts(64, 8, 0, 2, groups=2, keep=1)},
        {**_chunk_attention(8, 2, 128, 128, 70, 10000.0, 64, 0.07, kv_from=0), "mlp": _dense(192)},
    ],
}

# Models of one kind of mixer only: delta layers alone keep no pages at all (one query head per key head,
# one layer without a feed-forward); attention layers alone, one of them with neither rotation nor chunks
# (keys its configuration leaves out), the other reading its keys, with routers that leave `groups` out.
DIFORAX_D = {
    "architecture": "Diforax", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {**_delta(3, 3, 12, 20, 3), "mlp": _dense(80)},
        {**_delta(2, 1, 24, 16, 5), "mlp": None},
    ],
}
DIFORAX_E = {
    "architecture": "Diforax", "vocab": 160, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3},
         "mlp": _experts(32, 4, 1, 2)},
        {"type": "attention", "mixer": {"heads": 4, "scale": 0.2, "kv_from": 0, "mask": {"size": 33}},
         "mlp": _experts(16, 2, 0, 2)},
    ],
}

TINY.update({"DA": DIFORAX_A, "DB": DIFORAX_B, "DC": DIFORAX_C, "DD": DIFORAX_D, "DE": DIFORAX_E})


def _window_attention(heads, kv_heads, dim, vdim, scale, window=None, v_mix=False):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer}


def _pair(left, right):
    return {"type": "parallel", "mixer": {"left": left, "right": right}}


def _left(heads, kv_heads, dim, vdim, scale, rot=None, softcap=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        left["rot"] = rot
    if softcap is not None:
        left["softcap"] = softcap
    return left


def _linear(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


# Tiny Gukosun configurations that differ in every size and option: the order of the layers (a pair
# first, a window first), 1 to 4 query heads per key head, query and value sizes that differ both ways and
# sizes that are no multiple of 16, partial, full and no rotation with and without the scaling of long
# waves (the three bands all occur at these sizes), capped and uncapped scores, windows shorter than, equal
# to and longer than a page and a window of one, layers that mix values beside layers that do not, layers
# without a feed-forward, models with and without the token side input and the logit scale, decays from
# fast to almost none, and recurrent states that fill no warp.
GUKOSUN_A = {
    "architecture": "Gukosun", "vocab": 211, "width": 80, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "token_side": {"dim": 8},
    "layers": [
        {**_pair(_left(4, 2, 16, 24, 0.3, rot={"base": 10000.0, "dims": 8, "scaling":
                                               {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}, softcap=5.0),
                 _linear(3, 8, 20, (0.5, 0.9, 0.995))), "mlp": _dense(144)},
        {**_window_attention(6, 3, 32, 16, 0.2, window=37, v_mix=True), "mlp": _dense(112)},
        {**_window_attention(2, 1, 24, 24, 0.25), "mlp": None},
        {**_window_attention(6, 3, 32, 16, 0.3, window=70, v_mix=True), "mlp": _dense(96)},
        {**_pair(_left(2, 2, 32, 16, 0.2, rot={"base": 500.0, "dims": 32}, softcap=2.0),
                 _linear(1, 40, 12, (0.97,))), "mlp": None},
        {**_window_attention(6, 3, 32, 16, 0.3, window=1, v_mix=True), "mlp": _dense(96)},
    ],
}

GUKOSUN_B = {
    "architecture": "Gukosun", "vocab": 130, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {**_window_attention(4, 4, 16, 48, 0.25, window=64, v_mix=True), "mlp": _dense(160)},
        {**_pair(_left(3, 1, 20, 20, 0.22), _linear(2, 24, 24, (0.8, 0.999))), "mlp": _dense(120)},
        {**_window_attention(4, 4, 16, 48, 0.3, window=5, v_mix=True), "mlp": None},
        {**_window_attention(1, 1, 64, 32, 0.11, window=200), "mlp": _dense(64)},
    ],
}

# Head sizes and group widths that the tensor-core attention kernels take, so that the bfloat16 path
# runs them with a sink, a window and capped scores: 64 and 128 channels, four query heads per key head.
GUKOSUN_C = {
    "architecture": "Gukosun", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
    "token_side": {"dim": 16},
    "layers": [
        {**_window_attention(8, 2, 64, 64, 0.12, window=130, v_mix=True), "mlp": _dense(256)},
        {**_pair(_left(8, 2, 128, 128, 0.09, rot={"base": 10000.0, "dims": 64, "scaling":
                                                  {"factor": 8.0, "low": 1.0, "high": 2.0, "original": 128}}, softcap=10.0),
                 _linear(2, 64, 64, (0.9, 0.99))), "mlp": _dense(192)},
        {**_window_attention(8, 2, 64, 64, 0.1, window=70, v_mix=True), "mlp": _dense(256)},
        {**_pair(_left(4, 1, 64, 64, 0.12, rot={"base": 1000000.0, "dims": 64}),
                 _linear(4, 32, 32, (0.6, 0.9, 0.97, 0.999))), "mlp": _dense(128)},
    ],
}

# Models of one kind of layer only: pairs alone (pages of every key and a state, no window group), and
# windows alone (no state slots are needed; the first layer does not mix values, the second is the source).
GUKOSUN_D = {
    "architecture": "Gukosun", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "token_side": {"dim": 4},
    "layers": [
        {**_pair(_left(2, 1, 16, 16, 0.25, rot={"base": 100.0, "dims": 16}, softcap=50.0),
                 _linear(3, 12, 20, (0.7, 0.9, 0.99))), "mlp": _dense(80)},
        {**_pair(_left(3, 3, 8, 8, 0.35, rot={"base": 10000.0, "dims": 4}), _linear(2, 16, 8, (0.95, 0.5))), "mlp": None},
    ],
}
GUKOSUN_E = {
    "architecture": "Gukosun", "vocab": 160, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.25,
    "layers": [
        {**_window_attention(4, 2, 16, 32, 0.3, window=33), "mlp": _dense(96)},
        {**_window_attention(2, 2, 32, 16, 0.2, window=64, v_mix=True), "mlp": _dense(64)},
        {**_window_attention(2, 2, 32, 16, 0.2, v_mix=True), "mlp": _dense(64)},
    ],
}

TINY.update({"GA": GUKOSUN_A, "GB": GUKOSUN_B, "GC": GUKOSUN_C, "GD": GUKOSUN_D, "GE": GUKOSUN_E})


def _ramp(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _conv_attention(heads, kv_heads, dim, vdim, scale, conv=None, chunk=None, rot=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:
        mixer["conv"] = conv
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer}


def _gated_latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                                                  "kv_rank": kv_rank, "rot": rot, "scale": scale}}


def _table_experts(ff, limit, experts, top, shared=None):
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    return mlp


# Tiny Fobatar configurations that differ in every size and option: which layers repeat (the first two, one
# in the middle four times, the last two, none, all of them once), both orders of the two mixers and models of
# one mixer only, 1 to 4 query heads per key head, key and value sizes that differ both ways and sizes that are
# no multiple of 16, 1 to 4 taps, chunks shorter than, equal to and longer than a page and a chunk of one,
# attention without chunks, partial, full and no rotation with and without the ramp (whose three bands all
# occur), latent rows of 32 to 128 entries, one to all experts per token, with and without the shared expert,
# layers without a feed-forward, limits below and above 1, and the constants on the embedding and on the
# residual sums present, absent and equal to 1.
FOBATAR_A = {
    "architecture": "Fobatar", "vocab": 211, "width": 80, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
    "residual_mult": 0.7, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {**_conv_attention(4, 2, 16, 24, 0.3, conv=4, chunk=37, rot={"base": 10000.0, "dims": 8, "scaling": _ramp(4.0, 64, 8.0, 1.0)}),
         "mlp": _table_experts(48, 1.5, 5, 2, shared=(40, 2.5))},
        {**_gated_latent(3, 8, 8, 20, 24, 0.25, 500.0, _ramp(2.0, 32, 4.0, 0.5)), "mlp": _table_experts(32, 3.0, 3, 1)},
        {**_conv_attention(2, 1, 24, 24, 0.2, conv=2, chunk=64), "mlp": None},
        {**_gated_latent(2, 16, 4, 8, 40, 0.2, 100.0), "mlp": _table_experts(16, 0.75, 4, 4, shared=(8, 1.0))},
    ],
}

FOBATAR_B = {
    "architecture": "Fobatar", "vocab": 130, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "residual_mult": 1.0, "loop": {"start": 2, "stop": 3, "times": 4},
    "layers": [
        {**_gated_latent(4, 12, 6, 12, 20, 0.3, 10000.0, _ramp(8.0, 16, 2.0, 0.25)), "mlp": _table_experts(24, 2.0, 2, 2)},
        {**_gated_latent(1, 32, 16, 48, 64, 0.15, 1000000.0), "mlp": None},
        {**_conv_attention(3, 3, 20, 12, 0.22, conv=3, chunk=5, rot={"base": 300.0, "dims": 20}),
         "mlp": _table_experts(40, 0.5, 7, 3, shared=(56, 4.0))},
        {**_conv_attention(6, 2, 8, 16, 0.35, conv=1, rot={"base": 50.0, "dims": 4, "scaling": _ramp(3.0, 8, 1.5, 0.5)}),
         "mlp": _table_experts(24, 2.0, 2, 1, shared=(24, 2.0))},
    ],
}

# Sizes that the tensor-core kernels take, so that the bfloat16 path runs them: heads of 64 and 128 channels,
# four query heads per key head, latent rows of 64 and of 128 entries, expert widths in multiples of 8.
FOBATAR_C = {
    "architecture": "Fobatar", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
    "residual_mult": 0.25, "loop": {"start": 1, "stop": 4, "times": 2},
    "layers": [
        {**_conv_attention(8, 2, 64, 64, 0.12, conv=2, chunk=130, rot={"base": 1000000.0, "dims": 32, "scaling": _ramp(16.0, 256, 16.0, 2.0)}),
         "mlp": _table_experts(64, 1.0, 6, 2, shared=(96, 3.0))},
        {**_gated_latent(8, 32, 16, 32, 48, 0.125, 10000.0, _ramp(4.0, 64, 8.0, 1.0)), "mlp": _table_experts(32, 2.5, 4, 3)},
        {**_conv_attention(4, 1, 128, 128, 0.09, conv=4, chunk=70, rot={"base": 10000.0, "dims": 128}),
         "mlp": _table_experts(64, 1.0, 6, 2, shared=(96, 3.0))},
        {**_gated_latent(4, 64, 32, 64, 96, 0.1, 20000.0), "mlp": _table_experts(128, 6.0, 3, 2, shared=(64, 0.5))},
    ],
}

# One mixer only: latent layers alone (no state slots are needed; the constants are absent), and attention layers
# alone (a chunk of one token, a layer without chunks, every layer once through a loop of one pass).
FOBATAR_D = {
    "architecture": "Fobatar", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {**_gated_latent(2, 16, 8, 16, 24, 0.25, 100.0, _ramp(2.0, 16, 2.0, 1.0)), "mlp": _table_experts(80, 1.25, 3, 2, shared=(16, 1.25))},
        {**_gated_latent(3, 8, 2, 8, 12, 0.35, 10000.0), "mlp": None},
    ],
}
FOBATAR_E = {
    "architecture": "Fobatar", "vocab": 160, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
    "residual_mult": 1.5, "loop": {"start": 0, "stop": 3, "times": 1},
    "layers": [
        {**_conv_attention(4, 2, 16, 32, 0.3, conv=2, chunk=1), "mlp": _table_experts(96, 2.0, 8, 1)},
        {**_conv_attention(2, 2, 32, 16, 0.2, conv=3, chunk=33, rot={"base": 1000.0, "dims": 32, "scaling": _ramp(2.0, 48, 6.0, 0.5)}),
         "mlp": _table_experts(64, 1.0, 2, 2, shared=(32, 2.0))},
        {**_conv_attention(2, 2, 32, 16, 0.2, rot={"base": 1000.0, "dims": 16}), "mlp": _table_experts(64, 1.0, 2, 2, shared=(32, 2.0))},
    ],
}

TINY.update({"FA": FOBATAR_A, "FB": FOBATAR_B, "FC": FOBATAR_C, "FD": FOBATAR_D, "FE": FOBATAR_E})


def vocab_of(config: dict) -> int:
    return int(config.get("vocab_size", config.get("vocab")))
