"""A plain, slow Pametar: whole sequences, no cache, explicit loops, one function per mechanism.

The oracle of the Pametar tests.  It shares no code with the package: it reads a model folder with its own
safetensors reader and computes every position from all tokens before it.  ``dtype`` is the arithmetic
(float64 in most tests).

Notation: T tokens, H heads, d plain query/key size, p rotated size, e value size, r latent size of keys and
values, S copies of the stream, E experts.
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


# ---- small pieces ---------------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def dynamic_tanh(x, t, name):
    """The layer norm of this design: no statistics, tanh(alpha x) w + b."""
    return torch.tanh(t[name + ".alpha"] * x) * t[name] + t[name + ".b"]


def embed_tokens(tokens, t, config):
    """Token rows times the scale, plus the row of the pair table that (previous token, token) hashes to; the
    first token of a sequence takes the table's last row."""
    e = config["embedding"]
    x = t["embed"][torch.tensor(tokens)] * e["scale"]
    big = e.get("bigram")
    if big is not None:
        rows = []
        for i, tok in enumerate(tokens):
            rows.append(big["buckets"] if i == 0 else (tokens[i - 1] * big["mul_prev"] + tok * big["mul_cur"]) % big["buckets"])
        x = x + t["bigram"][torch.tensor(rows)]
    return x


def rotate_half_pairs(x, positions, dims, base):
    """x [T, ..., n]: among the first ``dims`` sizes, size i is paired with size i + dims / 2 and the pair is
    turned by position * base^(-2 i / dims); the other sizes pass."""
    half = dims // 2
    out = x.clone()
    for ti, pos in enumerate(positions):
        for i in range(half):
            a = pos * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[ti, ..., i], x[ti, ..., i + half]
            out[ti, ..., i] = u * c - v * s
            out[ti, ..., i + half] = v * c + u * s
    return out


def causal_attention_with_sink(q, k, v, scale, sink):
    """q, k [T, H, n], v [T, H, e], sink [H]: softmax over j <= i whose denominator also holds exp(sink_h)."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for i in range(T):
        for h in range(H):
            s = (k[:i + 1, h] @ q[i, h]) * scale
            top = torch.maximum(s.max(), sink[h])
            w = torch.exp(s - top)
            out[i, h] = (w @ v[:i + 1, h]) / (w.sum() + torch.exp(sink[h] - top))
    return out


# ---- mixers ---------------------------------------------------------------------------------------

def latent_attention_mixer(h, t, prefix, m, eps):
    """Queries through a normed latent; keys and values from a normed latent of r sizes plus one rotated key part
    shared by all heads."""
    T = h.shape[0]
    H, d, p, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = list(range(T))
    cq = rms_norm(h @ t[prefix + "dq"].T, t[prefix + "dq.norm"], eps)
    q = (cq @ t[prefix + "uq"].T).reshape(T, H, d + p)
    down = h @ t[prefix + "dkv"].T
    c = rms_norm(down[:, :r], t[prefix + "dkv.norm"], eps)
    rot = m["rot"]
    k_rot = rotate_half_pairs(down[:, r:], positions, rot["dims"], rot["base"])                       # [T, p]
    q_rot = rotate_half_pairs(q[:, :, d:], positions, rot["dims"], rot["base"])                       # [T, H, p]
    k_plain = (c @ t[prefix + "uk"].T).reshape(T, H, d)
    v = (c @ t[prefix + "uv"].T).reshape(T, H, e)
    keys = torch.cat([k_plain, k_rot[:, None, :].expand(T, H, p)], dim=-1)
    queries = torch.cat([q[:, :, :d], q_rot], dim=-1)
    o = causal_attention_with_sink(queries, keys, v, m["scale"], t[prefix + "sink"])
    return o.reshape(T, H * e) @ t[prefix + "o"].T


def general_delta_rule(r, k, v, w, a, state=None):
    """r, k, v, w, a [T, H, d].  Per head, with the unit key u_t = k_t / sqrt(sum k_t^2 + 1e-6):
    S_t = diag(w_t) S_(t-1) - (a_t * u_t)(u_t^T S_(t-1)) + k_t v_t^T (decay and removal both read S_(t-1)),
    o_t = S_t^T r_t.  Returns (o [T, H, d], the last state [H, d, d]); ``state`` is S before the first token (zeros)."""
    T, H, d = r.shape
    u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    out = torch.zeros((T, H, d), dtype=r.dtype)
    last = torch.zeros((H, d, d), dtype=r.dtype)
    for hh in range(H):
        S = torch.zeros((d, d), dtype=r.dtype) if state is None else state[hh].clone()
        for i in range(T):
            seen = u[i, hh] @ S                                                       # u^T S_(t-1), one number per value column
            S = w[i, hh][:, None] * S - torch.outer(a[i, hh] * u[i, hh], seen) + torch.outer(k[i, hh], v[i, hh])
            out[i, hh] = S.T @ r[i, hh]
        last[hh] = S
    return out, last


def head_rms(o, eps):
    """Every head's vector divided by its root mean square (eps inside the root)."""
    return o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps)


def general_delta_mixer(h, t, prefix, m, eps):
    """The rule's inputs from the mixer's input, the rule, and the normed, scaled and gated read-out."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ t[prefix + "r"].T).reshape(T, H, d)
    k = (h @ t[prefix + "k"].T).reshape(T, H, d)
    v = (h @ t[prefix + "v"].T).reshape(T, H, d)
    low = torch.tanh(h @ t[prefix + "w1"].T) @ t[prefix + "w2"].T + t[prefix + "w0"]
    w = torch.exp(-math.exp(-0.5) * sigmoid(low)).reshape(T, H, d)
    a = sigmoid(h @ t[prefix + "a"].T + t[prefix + "a.b"]).reshape(T, H, d)
    out, _ = general_delta_rule(r, k, v, w, a)
    y = head_rms(out, eps).reshape(T, H * d) * t[prefix + "norm"] * sigmoid(h @ t[prefix + "g"].T)
    return y @ t[prefix + "o"].T


# ---- feed-forward ---------------------------------------------------------------------------------

def routing(h, router, top, scale):
    """Chosen experts [T, top] and their weights: the largest softmax scores times ``scale``, not renormalised."""
    z = h @ router.T
    z = z - z.max(dim=-1, keepdim=True).values
    s = torch.exp(z)
    s = s / s.sum(dim=-1, keepdim=True)
    weights, chosen = torch.topk(s, top, dim=-1)
    return chosen, weights * scale


def expert(h, t, prefix):
    g = h @ t[prefix + "gate"].T
    return ((g * sigmoid(g)) * (h @ t[prefix + "up"].T)) @ t[prefix + "down"].T


def mixture_of_experts(h, t, prefix, mlp):
    chosen, weights = routing(h, t[prefix + "router"], mlp["router"]["top"], mlp["router"]["scale"])
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for j, w in zip(chosen[i].tolist(), weights[i]):
            out[i] += w * expert(h[i:i + 1], t, f"{prefix}e{j}.")[0]
    return out


# ---- the layer arrangement ------------------------------------------------------------------------

def read_copies(streams, weights):
    """u = sum_s weights[s] x_s of the copies [S, T, width]."""
    return torch.einsum("s,stw->tw", weights, streams)


def write_copies(streams, mix, out, y):
    """All copies at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y."""
    return torch.einsum("sr,stw->rtw", mix, streams) + out[:, None, None] * y[None]


def sublayer(streams, t, layer_prefix, q, run):
    """One sub-layer (q = 1: mixer, 2: feed-forward) between the copies of the stream [S, T, width]: h = norm(read),
    y = run(h) * scale * sigmoid(W_g h + b_g), write."""
    hc = f"{layer_prefix}hc{q}."
    h = dynamic_tanh(read_copies(streams, t[hc + "in"]), t, f"{layer_prefix}norm{q}")
    y = run(h) * t[f"{layer_prefix}ls{q}"]
    y = y * sigmoid(h @ t[f"{layer_prefix}rg{q}"].T + t[f"{layer_prefix}rg{q}.b"])
    return write_copies(streams, t[hc + "mix"], t[hc + "out"], y)


def layer_order(config):
    """Indices of the layers in the order they run; a looped range runs ``times`` times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def forward(config, t, tokens, dtype=torch.float64, taps=None):
    """Logits [T, vocab] of a whole sequence.  ``taps``, a list, receives the sum of the streams after every layer run."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in t.items()}
    eps = config["norm"]["eps"]
    x = embed_tokens(list(tokens), t, config)
    streams = x[None].repeat(config.get("streams", 1), 1, 1)
    for li in layer_order(config):
        layer, lp = config["layers"][li], f"l{li}."
        m = layer["mixer"]
        mixer = latent_attention_mixer if layer["type"] == "latent_attention" else general_delta_mixer
        streams = sublayer(streams, t, lp, 1, lambda h: mixer(h, t, lp + "mix.", m, eps))
        if layer.get("mlp") is not None:
            streams = sublayer(streams, t, lp, 2, lambda h: mixture_of_experts(h, t, lp + "mlp.", layer["mlp"]))
        if taps is not None:
            taps.append(streams.sum(dim=0))
    x = streams.sum(dim=0)
    return dynamic_tanh(x, t, "final.norm") @ t["head"].T


def greedy(config, t, prompt, n_new, dtype=torch.float64):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(config, t, tokens, dtype)[-1].argmax()))
    return tokens[len(prompt):]
