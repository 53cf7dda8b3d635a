"""Named configurations: the dictionaries a ``config.json`` would hold.

The reference chooses a model by name from a registry of size dictionaries
(``Llama-3-8B``, ``Llama-3.2-1B`` ... yalis/external/config.py:755-951, with an
``-Instruct`` twin of each).  The same names are kept here as data for the
random-weights mode and the benchmark; a real checkpoint is run from its own
``config.json`` and never needs this file.  The two ``tiny-*`` entries are the
small test shapes (they differ in every size and option).
"""

from __future__ import annotations

from copy import deepcopy
from typing import Any, Dict

_LLAMA3_SCALING_8 = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                         original_max_position_embeddings=8192)
_LLAMA3_SCALING_32 = dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)


def _llama(hidden, layers, heads, kv_heads, inter, max_pos, scaling=None, tied=False, head_dim=None,
           vocab=128256, theta=500000.0, eps=1e-5) -> Dict[str, Any]:
    return dict(
        architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=hidden, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim or hidden // heads,
        intermediate_size=inter, vocab_size=vocab, max_position_embeddings=max_pos, rms_norm_eps=eps,
        rope_theta=theta, rope_scaling=scaling, tie_word_embeddings=tied, hidden_act="silu",
        attention_bias=False, mlp_bias=False, torch_dtype="bfloat16", bos_token_id=128000, eos_token_id=128001,
    )


_BASE: Dict[str, Dict[str, Any]] = {
    "Llama-3-8B": _llama(4096, 32, 32, 8, 14336, 8192),
    "Llama-3.1-8B": _llama(4096, 32, 32, 8, 14336, 131072, _LLAMA3_SCALING_8),
    "Llama-3-70B": _llama(8192, 80, 64, 8, 28672, 8192),
    "Llama-3.1-70B": _llama(8192, 80, 64, 8, 28672, 131072, _LLAMA3_SCALING_8),
    "Llama-3.1-405B": _llama(16384, 126, 128, 8, 53248, 131072, _LLAMA3_SCALING_8),
    "Llama-3.2-1B": _llama(2048, 16, 32, 8, 8192, 131072, _LLAMA3_SCALING_32, tied=True),
    "Llama-3.2-3B": _llama(3072, 28, 24, 8, 8192, 131072, _LLAMA3_SCALING_32, tied=True),
}

PRESETS: Dict[str, Dict[str, Any]] = {}
for _name, _cfg in _BASE.items():
    PRESETS[_name] = _cfg
    PRESETS[_name + "-Instruct"] = _cfg
PRESETS["Llama-3.3-70B-Instruct"] = _BASE["Llama-3.1-70B"]

# Test shapes. A: GQA x2, no scaling, untied. B: MQA x3 with an odd head count, llama3 scaling whose
# three regimes all occur among 16 frequencies, tied, other eps/theta.
PRESETS["tiny-A"] = dict(
    _llama(64, 2, 4, 2, 176, 128, None, tied=False, head_dim=16, vocab=256, theta=10000.0, eps=1e-5),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)
PRESETS["tiny-B"] = dict(
    _llama(96, 3, 3, 1, 256, 256,
           dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                original_max_position_embeddings=32),
           tied=True, head_dim=32, vocab=512, theta=500000.0, eps=1e-6),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)
# Head sizes 64 and 128: the shapes that the TMA- and tcgen05-based attention kernels are built for.
PRESETS["tiny-C"] = dict(
    _llama(136, 2, 4, 2, 208, 512,
           dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                original_max_position_embeddings=64),
           tied=False, head_dim=64, vocab=320, theta=10000.0, eps=1e-5),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)
PRESETS["tiny-D"] = dict(
    _llama(192, 2, 2, 1, 320, 512, None, tied=True, head_dim=128, vocab=272, theta=500000.0, eps=1e-6),
    torch_dtype="bfloat16", bos_token_id=None, eos_token_id=None)



# ---- Tirezen: layers of three kinds of mixer, some of them run several times -------------------------------

def _retention(heads, dim, vdim, decay, rot_dims, base, ff):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay),
                                           "rot": {"dims": rot_dims, "base": base}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _delta(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _parallel(left, right, left_scale, right_scale, ff):
    lh, lg, ld, lv, rot_dims, base, scale, cap = left
    rh, rg, rd, rv, conv, decay_rank, gate_rank = right
    return {"type": "parallel",
            "mixer": {"left": {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "rot": {"dims": rot_dims, "base": base},
                               "scale": scale, "softcap": cap},
                      "right": {"heads": rh, "kv_heads": rg, "dim": rd, "vdim": rv, "conv": conv,
                                "decay_rank": decay_rank, "gate_rank": gate_rank},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _tirezen(width, vocab, layers, loop=None, eps=1e-5) -> Dict[str, Any]:
    cfg = {"architecture": "Tirezen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def _tirezen_stack(width, vocab, groups, heads, dim, kv_heads, ff) -> Dict[str, Any]:
    """``groups`` times (delta, parallel, retention) at the sizes of a real model: head size ``dim`` everywhere."""
    layers = []
    for _ in range(groups):
        layers.append(_delta(heads, kv_heads, dim, dim, 4, ff))
        layers.append(_parallel((heads, kv_heads, dim, dim, dim, 10000.0, dim ** -0.5, 30.0),
                                (heads, kv_heads, dim, dim, 4, 64, 64), 1.0, 1.0, ff))
        layers.append(_retention(heads, dim, dim, [1.0 - 0.04 / (1 + i % 4) for i in range(heads)], dim, 10000.0, ff))
    return _tirezen(width, vocab, layers)


# Test shapes.  A: three passes over the first two layers, partial rotation, grouped heads, value sizes that differ
# from key sizes, a layer without feed-forward.  B: no loop, sizes that are multiples of nothing, one head, one pass.
# C: state matrices of 64 and 128 rows, a loop in the middle.
PRESETS["tirezen-tiny-A"] = _tirezen(64, 96, [
    _retention(2, 16, 24, [0.9, 0.97], 8, 100.0, 48),
    _parallel((4, 2, 16, 8, 12, 10000.0, 0.3, 5.0), (4, 2, 8, 16, 3, 8, 4), 0.7, 1.3, 80),
    _delta(4, 2, 12, 20, 2, None)], loop=(0, 2, 3))
PRESETS["tirezen-tiny-B"] = _tirezen(40, 50, [
    _delta(3, 3, 6, 10, 5, 24),
    _parallel((3, 1, 20, 36, 20, 500.0, 0.2, 30.0), (2, 1, 20, 6, 4, 5, 12), 1.0, 0.25, None),
    _retention(1, 40, 8, [0.99], 16, 200000.0, 56)], eps=1e-6)
PRESETS["tirezen-tiny-C"] = _tirezen(128, 160, [
    _delta(2, 1, 128, 64, 4, 96),
    _retention(2, 64, 128, [0.97, 0.995], 64, 10000.0, 96),
    _parallel((2, 2, 64, 64, 32, 10000.0, 0.125, 25.0), (2, 2, 64, 48, 4, 16, 16), 1.1, 0.6, 96)], loop=(1, 2, 2))
# D: no attention at all (nothing is kept in pages), every layer inside the loop, kv_heads below heads in the delta rule.
PRESETS["tirezen-tiny-D"] = _tirezen(48, 64, [
    _retention(3, 8, 12, [0.5, 0.9, 0.999], 4, 10.0, 32),
    _delta(4, 1, 16, 4, 3, 40)], loop=(0, 2, 2))
# E: a width and head sizes that are multiples of 2 or 3 only (no row starts on a 16-byte boundary), attention whose
# keys and values share a head size of 16 (the tensor-core kernel's smallest), six taps.
PRESETS["tirezen-tiny-E"] = _tirezen(36, 37, [
    _parallel((2, 1, 16, 16, 10, 300.0, 0.4, 8.0), (3, 3, 9, 3, 6, 3, 7), 0.9, 1.1, 30),
    _retention(2, 10, 7, [0.8, 0.95], 6, 50.0, None),
    _delta(2, 2, 5, 9, 6, 22)], loop=(1, 3, 2))
# Sizes that resemble a real model's layers (random weights, for the benchmark).
PRESETS["tirezen-1b"] = _tirezen_stack(2048, 32000, 5, 16, 128, 8, 8192)
PRESETS["tirezen-3b"] = _tirezen_stack(3072, 32000, 8, 24, 128, 8, 8192)


# ---- Vepivik: windowed attention and attention over a cached latent, routed feed-forwards ----------------------

def _moe(experts, top, ff, shared):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def _windowed(heads, kv_heads, dim, vdim, window, scale, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, window, scale, rot, mlp, kv_from=None):
    """``rot`` = (dims, base) or (dims, base, factor, original, fast, slow)."""
    r = {"dims": rot[0], "base": rot[1]}
    if len(rot) > 2:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2:]))
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
             "scale": scale, "rot": r}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _vepivik(width, vocab, layers, embedding_scale=1.0, eps=1e-5) -> Dict[str, Any]:
    return {"architecture": "Vepivik", "width": width, "vocab": vocab, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale}, "layers": layers}


def _vepivik_stack(width, vocab, groups, heads, kv_heads, dim, kv_rank, rot_dim, window, experts, top, ff, shared) -> Dict[str, Any]:
    """``groups`` times (attention, latent, latent reading the one before, attention) at the sizes of a real model."""
    rot = (rot_dim, 10000.0, 8.0, 4096, 32.0, 1.0)
    layers = []
    for _ in range(groups):
        at = len(layers)
        mlp = _moe(experts, top, ff, shared)
        layers.append(_windowed(heads, kv_heads, dim, dim, window, dim ** -0.5, mlp))
        layers.append(_latent(heads, dim, rot_dim, dim, kv_rank, 2 * window, (dim + rot_dim) ** -0.5, rot, mlp))
        layers.append(_latent(heads, dim, rot_dim, dim, kv_rank, 2 * window, (dim + rot_dim) ** -0.5, rot, mlp, kv_from=at + 1))
        layers.append(_windowed(heads, kv_heads, dim, dim, window, dim ** -0.5, mlp))
    return _vepivik(width, vocab, layers, embedding_scale=width ** 0.5)


_Y1 = (8, 100.0, 4.0, 32, 8.0, 2.0)
# Test shapes.  A: a reader with a wider window than the layer whose rows it reads, a rotation of fewer sizes than the
# rotated part has, a layer without feed-forward, one without a shared expert, a single choice.  B: sizes that are
# multiples of nothing (no row on a 16-byte boundary), one key head, one latent head, three of five experts.
# C: the head sizes of the tensor-core kernels, windows of one position and of a page, sixteen experts.
# D: every expert chosen, windows that never bind, as many key heads as heads, no embedding scale.
PRESETS["vepivik-tiny-A"] = _vepivik(64, 96, [
    _latent(2, 8, 8, 12, 24, 20, 0.3, _Y1, _moe(4, 2, 24, 40)),
    _windowed(4, 2, 12, 20, 9, 0.25, _moe(6, 1, 16, 16)),
    _latent(3, 12, 8, 8, 24, 33, 0.2, _Y1, None, kv_from=0),
    _windowed(2, 2, 16, 16, 16, 0.35, _moe(4, 3, 32, None)),
    _latent(2, 10, 6, 14, 16, 11, 0.28, (4, 50.0), _moe(4, 2, 24, 8))], embedding_scale=2.5)
PRESETS["vepivik-tiny-B"] = _vepivik(36, 50, [
    _windowed(3, 1, 10, 6, 5, 0.3, _moe(5, 3, 18, None)),
    _latent(1, 6, 4, 10, 14, 7, 0.4, (4, 20.0, 3.0, 16, 4.0, 0.5), _moe(3, 2, 10, 14)),
    _latent(3, 5, 4, 7, 14, 3, 0.35, (4, 20.0, 3.0, 16, 4.0, 0.5), _moe(5, 3, 18, 6), kv_from=1)],
    embedding_scale=0.7, eps=1e-6)
PRESETS["vepivik-tiny-C"] = _vepivik(128, 160, [
    _latent(4, 32, 32, 32, 64, 64, 0.12, (32, 10000.0, 2.0, 64, 16.0, 1.0), _moe(16, 4, 32, 64)),
    _windowed(4, 2, 64, 64, 1, 0.125, _moe(16, 4, 32, 64)),
    _windowed(2, 1, 64, 64, 64, 0.125, _moe(8, 2, 64, None)),
    _latent(8, 16, 32, 16, 64, 17, 0.15, (32, 10000.0, 2.0, 64, 16.0, 1.0), _moe(16, 4, 32, 64), kv_from=0)],
    embedding_scale=3.0)
PRESETS["vepivik-tiny-D"] = _vepivik(48, 64, [
    _windowed(2, 2, 8, 24, 4096, 0.3, _moe(2, 2, 20, 12)),
    _latent(2, 16, 2, 8, 20, 4096, 0.25, (2, 7.0), _moe(2, 2, 20, 12))], embedding_scale=1.0)
# Sizes that resemble a real model's layers (random weights, for the benchmark): about a billion weights of which
# a token uses a quarter; head size 128 so that the windowed attention runs on the tensor cores.
PRESETS["vepivik-1b"] = _vepivik_stack(2048, 32000, 4, 16, 8, 128, 256, 64, 1024, 16, 2, 2048, 2048)
PRESETS["vepivik-3b"] = _vepivik_stack(3072, 32000, 6, 24, 8, 128, 384, 64, 1024, 32, 4, 1536, 3072)


# ---- Pametar -------------------------------------------------------------------------------------------------------

def _pm_moe(experts, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}


def _pm_delta(heads, dim, decay_rank, mlp):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}, "mlp": mlp}


def _pm_latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, mlp):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"dims": rot_dim, "base": base}}}


def _pametar(width, vocab, streams, layers, loop=None, embedding_scale=1.0, bigram=(509, 31, 3), eps=1e-5) -> Dict[str, Any]:
    emb: Dict[str, Any] = {"scale": embedding_scale}
    if bigram is not None:
        emb["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    cfg = {"architecture": "Pametar", "width": width, "vocab": vocab, "streams": streams, "norm": {"eps": eps},
           "embedding": emb, "layers": layers}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def _pametar_stack(width, vocab, groups, streams, heads, dim, kv_rank, q_rank, rot_dim, delta_heads, delta_dim, experts, top, ff):
    """``groups`` times (generalized delta rule, latent attention) at the sizes of a real model, every layer with experts."""
    layers = []
    for _ in range(groups):
        mlp = _pm_moe(experts, top, ff, 1.0)
        layers.append(_pm_delta(delta_heads, delta_dim, 64, mlp))
        layers.append(_pm_latent(heads, dim, rot_dim, dim, kv_rank, q_rank, (dim + rot_dim) ** -0.5, 10000.0, mlp))
    return _pametar(width, vocab, streams, layers, embedding_scale=width ** 0.5, bigram=(32003, 1009, 31))


# Test shapes.  A: two copies of the stream, a looped pair of layers, a layer without feed-forward, one chosen expert.
# B: sizes that are multiples of nothing, one copy, three passes over one layer, every expert chosen.  C: sizes the
# tensor-core kernels take, four copies, no loop, no pair table.  D: the rule before attention and after, a loop that
# covers all layers, three copies, one head, as many latent sizes as query sizes.
PRESETS["pametar-tiny-A"] = _pametar(64, 96, 2, [
    _pm_latent(2, 8, 8, 12, 24, 20, 0.3, 100.0, _pm_moe(4, 2, 24, 2.0)),
    _pm_delta(2, 16, 8, _pm_moe(6, 1, 16, 1.0)),
    _pm_latent(3, 12, 4, 8, 16, 28, 0.2, 50.0, None),
    _pm_delta(4, 8, 4, _pm_moe(4, 3, 32, 0.7))], loop=(1, 3, 2), embedding_scale=2.5)
PRESETS["pametar-tiny-B"] = _pametar(36, 50, 1, [
    _pm_delta(3, 10, 5, _pm_moe(3, 3, 10, 1.3)),
    _pm_latent(1, 6, 2, 10, 14, 9, 0.4, 20.0, _pm_moe(5, 3, 18, 1.0)),
    _pm_delta(1, 20, 3, None)], loop=(0, 1, 3), embedding_scale=0.7, bigram=(7, 5, 11), eps=1e-6)
PRESETS["pametar-tiny-C"] = _pametar(128, 160, 4, [
    _pm_latent(4, 32, 32, 32, 64, 48, 0.12, 10000.0, _pm_moe(16, 4, 32, 1.5)),
    _pm_delta(2, 64, 16, _pm_moe(8, 2, 64, 1.0)),
    _pm_latent(8, 16, 16, 16, 128, 64, 0.15, 10000.0, _pm_moe(16, 4, 32, 0.5)),
    _pm_delta(4, 32, 8, _pm_moe(8, 2, 64, 1.0))], embedding_scale=3.0, bigram=None)
PRESETS["pametar-tiny-D"] = _pametar(48, 64, 3, [
    _pm_delta(2, 12, 6, _pm_moe(2, 1, 20, 1.0)),
    _pm_latent(1, 16, 6, 8, 20, 20, 0.25, 7.0, _pm_moe(2, 2, 20, 3.0)),
    _pm_delta(3, 8, 2, None)], loop=(0, 3, 2), embedding_scale=1.0, bigram=(64, 1, 1))
# Sizes that resemble a real model's layers (random weights, for the benchmark): the widths, expert counts and latent
# sizes of the Vepivik benchmark models, so that the two designs stand beside each other at equal size.
PRESETS["pametar-1b"] = _pametar_stack(2048, 32000, 8, 4, 16, 128, 256, 768, 64, 16, 128, 16, 2, 1280)
PRESETS["pametar-3b"] = _pametar_stack(3072, 32000, 12, 4, 24, 128, 384, 1024, 64, 24, 128, 32, 4, 1024)


# ---- Sazavik -------------------------------------------------------------------------------------------------------

def _sz_mixer(kind, heads, kv_heads, dim, vdim, size, scale, rot=None, q_temp=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size}, "scale": scale}
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    if q_temp is not None:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": kind, "mixer": mixer}


def _sz_dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _sz_layer(mixer, mlp):
    return {**mixer, "mlp": mlp}


def _sazavik(width, vocab, layers, softcap=30.0, eps=1e-5) -> Dict[str, Any]:
    cfg = {"architecture": "Sazavik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if softcap is not None:
        cfg["logit_softcap"] = softcap
    return cfg


def _sazavik_stack(width, vocab, groups, heads, kv_heads, dim, chunk, window, ff, experts, top, expert_ff, shared) -> Dict[str, Any]:
    """``groups`` times (half-split chunked attention + dense, windowed attention with distance bias + experts,
    interleaved chunked attention with sink and gate + dense, a reader of the windowed layer's keys + experts)."""
    layers = []
    for _ in range(groups):
        at = len(layers)
        moe = _moe(experts, top, expert_ff, shared)
        layers.append(_sz_layer(_sz_mixer("attention_2", heads, kv_heads, dim, dim, chunk, dim ** -0.5, rot=(dim // 2, 10000.0)),
                                _sz_dense(ff, 7.0)))
        layers.append(_sz_layer(_sz_mixer("attention_3", heads, kv_heads, dim, dim, window, dim ** -0.5, q_temp=(0.1, 1024)), moe))
        layers.append(_sz_layer(_sz_mixer("attention", heads, kv_heads, dim, dim, chunk, dim ** -0.5, rot=(dim, 500000.0)),
                                _sz_dense(ff, 7.0)))
        layers.append(_sz_layer(_sz_mixer("attention_3", heads, kv_heads, dim, dim, window, dim ** -0.5, q_temp=(0.1, 1024),
                                          kv_from=at + 1), moe))
    return _sazavik(width, vocab, layers)


# Test shapes.  A: all three mixers, a reader with a wider window than the layer whose keys it reads, a layer without
# feed-forward, an expert layer without a shared expert, chunks and windows that are multiples of nothing.  B: sizes
# that are multiples of nothing (no row on a 16-byte boundary), one key head, all heads turning whole, three of five
# experts, no soft cap.  C: the head sizes of the tensor-core kernels, a window of one position, a chunk of a page,
# sixteen experts, a query temperature that changes every few positions.  D: every expert chosen, masks that never
# bind, as many key heads as heads, key and value sizes apart.
PRESETS["sazavik-tiny-A"] = _sazavik(64, 96, [
    _sz_layer(_sz_mixer("attention_3", 4, 2, 12, 20, 9, 0.3, q_temp=(0.4, 5)), _moe(6, 2, 16, 24)),
    _sz_layer(_sz_mixer("attention", 4, 2, 16, 16, 11, 0.25, rot=(8, 100.0)), _sz_dense(40, 1.5)),
    _sz_layer(_sz_mixer("attention_3", 4, 2, 12, 20, 23, 0.3, q_temp=(0.7, 3), kv_from=0), None),
    _sz_layer(_sz_mixer("attention_2", 2, 1, 24, 8, 13, 0.2, rot=(10, 50.0)), _moe(4, 1, 24, None)),
    _sz_layer(_sz_mixer("attention", 3, 3, 10, 14, 7, 0.35, rot=(10, 30.0)), _sz_dense(24, 0.8))], softcap=12.0)
PRESETS["sazavik-tiny-B"] = _sazavik(36, 50, [
    _sz_layer(_sz_mixer("attention_2", 3, 1, 10, 6, 5, 0.3, rot=(10, 20.0)), _moe(5, 3, 18, 14)),
    _sz_layer(_sz_mixer("attention_3", 3, 3, 6, 10, 4, 0.4, q_temp=(1.5, 2)), _sz_dense(30, 3.0)),
    _sz_layer(_sz_mixer("attention", 2, 1, 14, 5, 3, 0.35, rot=(2, 7.0)), _moe(3, 2, 10, 6))], softcap=None, eps=1e-6)
PRESETS["sazavik-tiny-C"] = _sazavik(128, 160, [
    _sz_layer(_sz_mixer("attention", 4, 2, 64, 64, 16, 0.125, rot=(32, 10000.0)), _moe(16, 4, 32, 64)),
    _sz_layer(_sz_mixer("attention_3", 4, 4, 32, 32, 1, 0.18, q_temp=(0.3, 7)), _sz_dense(256, 2.5)),
    _sz_layer(_sz_mixer("attention_2", 8, 2, 16, 16, 40, 0.25, rot=(16, 1000.0)), _moe(8, 2, 64, None)),
    _sz_layer(_sz_mixer("attention_3", 2, 1, 128, 128, 50, 0.09, q_temp=(0.2, 16)), _sz_dense(128, 1.0)),
    _sz_layer(_sz_mixer("attention_3", 2, 1, 128, 128, 33, 0.09, q_temp=(0.6, 4), kv_from=3), _moe(16, 4, 32, 64))], softcap=20.0)
PRESETS["sazavik-tiny-D"] = _sazavik(48, 64, [
    _sz_layer(_sz_mixer("attention_2", 2, 2, 8, 24, 4096, 0.3, rot=(4, 9.0)), _moe(2, 2, 20, 12)),
    _sz_layer(_sz_mixer("attention", 2, 2, 16, 8, 4096, 0.25, rot=(16, 7.0)), _sz_dense(36, 50.0)),
    _sz_layer(_sz_mixer("attention_3", 4, 4, 8, 8, 4096, 0.3, q_temp=(0.5, 4096)), _moe(2, 2, 20, 12))], softcap=40.0)
# Sizes that resemble a real model's layers (random weights, for the benchmark): the widths, head counts and windows of
# the Vepivik benchmark models and, with half the layers dense, twice their experts, so that the two designs stand
# beside each other at about equal size (2.9 and 9.2 billion weights beside 2.6 and 8.5).
PRESETS["sazavik-1b"] = _sazavik_stack(2048, 32000, 4, 16, 8, 128, 2048, 1024, 4096, 32, 2, 1408, 2048)
PRESETS["sazavik-3b"] = _sazavik_stack(3072, 32000, 6, 24, 8, 128, 2048, 1024, 6144, 64, 4, 1024, 3072)


def preset(name: str) -> Dict[str, Any]:
    """A fresh copy of the named configuration dictionary."""
    for key in (name, name.split("/")[-1], name.split("/")[-1].replace("Meta-", "")):
        if key in PRESETS:
            return deepcopy(PRESETS[key])
    raise ValueError(f"{name!r} is not a supported config name (known: {', '.join(sorted(PRESETS))})")
