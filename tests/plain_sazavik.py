"""A plain, slow Sazavik: whole sequences, no cache, explicit loops, one function per mechanism.

The oracle of the Sazavik tests.  It shares no code with the package: it reads a model folder with its own
safetensors reader and computes every position from all tokens before it.  ``dtype`` is the arithmetic
(float64 in most tests).

Notation: T tokens, H query heads, G key/value heads, d key size, e value size, C chunk size, W window.
"""

from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


def read_folder(path):
    """(config dictionary, name -> float64 tensor) of a model folder."""
    with open(os.path.join(path, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = blob[8 + n + a:8 + n + b]
        kind = info["dtype"]
        if kind == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32).astype(np.float64)
        elif kind == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif kind == "I32":
            arr = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {kind}")
        tensors[name] = torch.from_numpy(arr.reshape(info["shape"]).copy())
    return config, tensors


# ---- norms -----------------------------------------------------------------------------------------------------

def rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def stream_norm(x, w, eps):
    """The norm of the stream: the stored weight lies around zero."""
    return rms(x, eps) * (1.0 + w)


def head_norm(x, w, eps):
    """The norm of a head: the stored weight is the scale."""
    return rms(x, eps) * w


# ---- positions -------------------------------------------------------------------------------------------------

def turn(x, positions, dims, base, interleaved):
    """x [T, heads, d]: the first ``dims`` sizes of every head turn by position * base^(-2i/dims); pair i is
    (2i, 2i + 1) when interleaved, else (i, i + dims/2)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        angle = positions.to(x.dtype) * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(angle)[:, None], torch.sin(angle)[:, None]
        out[:, :, a] = x[:, :, a] * c - x[:, :, b] * s
        out[:, :, b] = x[:, :, b] * c + x[:, :, a] * s
    return out


def query_temperature(positions, coef, every, dtype):
    """1 + coef ln(floor((p + 1) / every) + 1) per position."""
    return torch.tensor([1.0 + coef * math.log((int(p) + 1) // every + 1) for p in positions], dtype=dtype)


def visible(i, kind, size):
    """The positions j that position i sees: ``chunk``: those of its own chunk of ``size`` up to itself; ``window``:
    itself and the size - 1 before it."""
    if kind == "chunk":
        return range((i // size) * size, i + 1)
    return range(max(0, i - size + 1), i + 1)


def distance_slopes(H):
    return [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]


# ---- attention core --------------------------------------------------------------------------------------------

def attend(q, k, v, scale, mask_kind, mask_size, sink=None, slopes=None):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  ``sink`` [H]: exp(sink_h) joins the denominator.
    ``slopes`` [H]: slope_h * (i - j) is taken off the score."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for i in range(T):
        js = list(visible(i, mask_kind, mask_size))
        for h in range(H):
            g = h // (H // G)
            s = (k[js, g] @ q[i, h]) * scale
            if slopes is not None:
                s = s - slopes[h] * torch.tensor([float(i - j) for j in js], dtype=q.dtype)
            m = s.max()
            if sink is not None:
                m = torch.maximum(m, sink[h])
            e = torch.exp(s - m)
            denom = e.sum()
            if sink is not None:
                denom = denom + torch.exp(sink[h] - m)
            out[i, h] = (e / denom) @ v[js, g]
    return out


# ---- the three mixers ------------------------------------------------------------------------------------------

def _project(h, t, name, bias):
    y = h @ t[name].T
    return y + t[name + ".b"] if bias else y


def make_keys_values(h, t, prefix, m, kind, eps, positions):
    """What a layer caches: keys after norm (and rotation, where the mixer has one) and values."""
    T = h.shape[0]
    G, d, e = m["kv_heads"], m["dim"], m["vdim"]
    bias = kind == "attention_3"
    k = head_norm(_project(h, t, prefix + "k", bias).reshape(T, G, d), t[prefix + "k.norm"], eps)
    v = _project(h, t, prefix + "v", bias).reshape(T, G, e)
    if kind != "attention_3":
        k = turn(k, positions, m["rot"]["dims"], m["rot"]["base"], interleaved=(kind == "attention"))
    return k, v


def mixer(h, t, prefix, m, kind, eps, positions, kv=None):
    """One of the mixers ``attention`` (chunked, interleaved rotation, sink, gate), ``attention_2`` (chunked,
    half rotation) and ``attention_3`` (window, biases, query temperature, distance bias, gate).  ``kv``: keys and
    values of another layer to use instead of making them.  Returns (output, (keys, values))."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    bias = kind == "attention_3"
    q = head_norm(_project(h, t, prefix + "q", bias).reshape(T, H, d), t[prefix + "q.norm"], eps)
    if kv is None:
        kv = make_keys_values(h, t, prefix, m, kind, eps, positions)
    k, v = kv
    sink = slopes = None
    if kind == "attention_3":
        q = q * query_temperature(positions, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None, None]
        slopes = distance_slopes(H)
        mask = "window"
    else:
        q = turn(q, positions, m["rot"]["dims"], m["rot"]["base"], interleaved=(kind == "attention"))
        mask = "chunk"
        if kind == "attention":
            sink = t[prefix + "sink"]
    o = attend(q, k, v, m["scale"], mask, m["mask"]["size"], sink=sink, slopes=slopes).reshape(T, -1)
    if kind in ("attention", "attention_3"):
        o = o * torch.sigmoid(h @ t[prefix + "g"].T)
    return _project(o, t, prefix + "o", bias), kv


# ---- feed-forwards ---------------------------------------------------------------------------------------------

def dense_ff(h, t, prefix, limit):
    g = torch.clamp(h @ t[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ t[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ t[prefix + "down"].T


def silu_expert(h, t, prefix):
    z = h @ t[prefix + "gate"].T
    return (z * torch.sigmoid(z) * (h @ t[prefix + "up"].T)) @ t[prefix + "down"].T


def route(h, t, prefix, top):
    """(chosen experts [T, top], their sigmoid scores [T, top]); ties go to the smaller index."""
    s = torch.sigmoid(h @ t[prefix + "router"].T)
    ids, ws = [], []
    for row in s:
        order = sorted(range(len(row)), key=lambda e: (-float(row[e]), e))[:top]
        ids.append(order)
        ws.append([float(row[e]) for e in order])
    return ids, ws


def route_margins(h, t, prefix, top):
    """Per token, how far the last chosen logit lies above the first one left out (inf when every expert is chosen):
    where this is small, reduced precision may choose otherwise."""
    z = h @ t[prefix + "router"].T
    if top >= z.shape[1]:
        return torch.full((z.shape[0],), float("inf"), dtype=z.dtype)
    srt = torch.sort(z, dim=1, descending=True).values
    return srt[:, top - 1] - srt[:, top]


def moe_ff(h, t, prefix, mlp, margins=None):
    """Every token's input, times the chosen expert's score, goes through that expert; the shared expert is
    weighted by one sigmoid per token."""
    ids, ws = route(h, t, prefix, mlp["router"]["top"])
    if margins is not None:
        margins.append(route_margins(h, t, prefix, mlp["router"]["top"]))
    out = torch.zeros_like(h)
    for n in range(h.shape[0]):
        for e, w in zip(ids[n], ws[n]):
            out[n] += silu_expert((h[n] * w)[None], t, f"{prefix}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + silu_expert(h, t, prefix + "shared.") * torch.sigmoid(h @ t[prefix + "shared.sg"].T)
    return out


# ---- the model ---------------------------------------------------------------------------------------------------

def forward(config, tensors, tokens, dtype=torch.float64, taps=None, margins=None):
    """Logits [T, vocab] of one sequence.  ``taps``: a list that receives the stream after every layer.  ``margins``: a
    list that receives, per routed layer, every token's ``route_margins``."""
    t = {k: (v.to(dtype) if v.dtype.is_floating_point else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = stream_norm(t["embed"][torch.tensor(tokens)], t["embed.norm"], eps)
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        src = m.get("kv_from")
        y, kept[i] = mixer(stream_norm(x, t[p + "norm1"], eps), t, p + "mix.", m, kind, eps, positions,
                           kv=None if src is None else kept[src])
        x = x + stream_norm(y, t[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = stream_norm(x, t[p + "norm2"], eps)
            y = dense_ff(h, t, p + "mlp.", mlp["limit"]) if mlp["kind"] == "dense" else moe_ff(h, t, p + "mlp.", mlp, margins)
            x = x + stream_norm(y, t[p + "norm2b"], eps)
        if taps is not None:
            taps.append(x.clone())
    z = stream_norm(x, t["final.norm"], eps) @ t["head"].T
    cap = config.get("logit_softcap")
    return z if cap is None else cap * torch.tanh(z / cap)


def greedy(config, tensors, prompt, n_new, dtype=torch.float64):
    """The prompt's continuation by ``n_new`` tokens, each the arg-max of the logits at the last position."""
    tokens, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(config, tensors, tokens, dtype)[-1]))
        tokens.append(nxt)
        out.append(nxt)
    return out
