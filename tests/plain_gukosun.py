"""A plain, slow implementation of the Gukosun design, one function per mechanism, in float64 torch on
the CPU.  It shares no code with the engine: tests compare the engine's parts and whole models with it.

Notation: W the model width, ``unit(y) = y / sqrt(mean(y^2) + eps)`` over the last axis, positions
count from 0 in every sequence, matrices are stored [out][in] and applied as ``y = x @ M.T``.

``rnd`` (optional, in some functions): a function applied where the serving precision rounds (inputs
of matrix products, cached keys and values); the identity by default.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def bf16(value):
    """To bfloat16 and back: what the serving precision loses where it keeps 16 bits."""
    return value.to(torch.bfloat16).to(value.dtype)


def load_model_dir(path):
    """(config dict, name -> tensor in float64, integer tensors as they are) of a model folder: the file
    is a little-endian header length, a JSON header (dtype, shape, byte range per name) and the data."""
    path = Path(path)
    config = json.loads((path / "config.json").read_text())
    blob = (path / "model.safetensors").read_bytes()
    (header_len,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + header_len].decode("utf-8"))
    data = memoryview(blob)[8 + header_len:]
    dtypes = {"F64": torch.float64, "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64}
    weights = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        lo, hi = entry["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=dtypes[entry["dtype"]]).reshape(entry["shape"])
        weights[name] = t.to(F64) if t.is_floating_point() else t
    return config, weights


def unit(y, eps):
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.relu(z) ** 2


# ------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2, then the wavelength-dependent scaling: short waves stay, long
    waves are divided by ``factor``, the band between is blended."""
    dims = int(rot["dims"])
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    scaling = rot.get("scaling")
    if scaling:
        factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
        original = float(scaling["original"])
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < original / high:
                out.append(fi)
            elif wave > original / low:
                out.append(fi / factor)
            else:
                s = (original / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate_pairs(x, positions, rot):
    """x: [T][heads][dim].  Channels 2i and 2i+1 (i < dims/2) of every head turn by positions * f_i; the
    channels from ``dims`` on pass unchanged."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    f = rotary_frequencies(rot)
    angle = positions.to(F64)[:, None] * f[None, :]                      # [T][dims/2]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------ softmax attention with a sink
def sink_attention(q, k, v, q_pos, k_pos, scale, sink, window=0, softcap=0.0):
    """q: [Tq][H][d], k: [Tk][G][d], v: [Tk][G][e]; query head j reads key/value head j // (H/G).
    Query at position i sees the key at position j when j <= i and (no window or i - j < window).
    score = scale q.k, optionally cap * tanh(score / cap); the softmax's denominator also holds
    exp(sink_j): one more term without a value.  Returns [Tq][H][e]."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((Tq, H, v.shape[2]), dtype=F64)
    diff = q_pos[:, None] - k_pos[None, :]
    seen = diff >= 0
    if window:
        seen = seen & (diff < window)
    for j in range(H):
        g = j // (H // G)
        s = (q[:, j] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(dim=1).values, sink[j].to(F64))
        p = torch.exp(s - top[:, None])
        denom = p.sum(dim=1) + torch.exp(sink[j].to(F64) - top)
        out[:, j] = (p / denom[:, None]) @ v[:, g]
    return out


# ------------------------------------------------------------------ the windowed attention mixer
def window_attention_mixer(h, w, prefix, m, eps, positions, v_first=None, rnd=lambda t: t):
    """The mixer of an 'attention' layer over one whole sequence.  Per-head RMS norm of q and k with
    one weight of size dim shared by the heads; no rotation; window ``mask.size``; sink; values mixed with
    the first such layer's (``v_first`` given: v <- (1 - lam) v + lam v_first); an elementwise
    sigmoid gate on the concatenated heads; output projection.  Returns (out [T][W], v [T][G][e])."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    hr = rnd(h)
    q = rnd(hr @ w[prefix + "q"].T).view(T, H, d)
    k = rnd(hr @ w[prefix + "k"].T).view(T, G, d)
    v = rnd(hr @ w[prefix + "v"].T).view(T, G, e)
    q = unit(q, eps) * w[prefix + "q.norm"]
    k = unit(k, eps) * w[prefix + "k.norm"]
    if v_first is not None:
        lam = w[prefix + "vmix"].reshape(())
        v = (1.0 - lam) * v + lam * v_first
    q, k, v = rnd(q), rnd(k), rnd(v)
    window = int((m.get("mask") or {}).get("size") or 0)
    o = sink_attention(q, k, v, positions, positions, float(m["scale"]), w[prefix + "sink"], window=window)
    gate = torch.sigmoid(rnd(hr @ w[prefix + "g"].T))
    z = rnd(o.reshape(T, H * e) * gate)
    return z @ w[prefix + "o"].T, v


# ------------------------------------------------------------------ the two halves of the parallel mixer
def left_attention_mixer(h, w, prefix, m, eps, positions, rnd=lambda t: t):
    """Softmax attention over every earlier key: RMS norm over the whole q projection (and the whole k
    projection) with a weight of that size; rotation of interleaved pairs on the first rot.dims channels
    of each head; capped scores; sink; one sigmoid gate per head; output projection."""
    T = h.shape[0]
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    hr = rnd(h)
    q = unit(rnd(hr @ w[prefix + "q"].T), eps) * w[prefix + "q.norm"]
    k = unit(rnd(hr @ w[prefix + "k"].T), eps) * w[prefix + "k.norm"]
    v = rnd(hr @ w[prefix + "v"].T).view(T, G, e)
    rot = m.get("rot") or {"dims": 0}
    q = rnd(rotate_pairs(q.view(T, H, d), positions, rot))
    k = rnd(rotate_pairs(k.view(T, G, d), positions, rot))
    o = sink_attention(q, k, v, positions, positions, float(m["scale"]), w[prefix + "sink"],
                       softcap=float(m.get("softcap") or 0.0))
    gate = torch.sigmoid(rnd(hr @ w[prefix + "g"].T))                    # [T][H]
    z = rnd((o * gate[:, :, None]).reshape(T, H * e))
    return z @ w[prefix + "o"].T


def decayed_outer_state(q, k, v, decay, state=None):
    """The linear recurrence of one sequence, token by token.  q, k: [T][H][d], v: [T][H][e], decay [H].
    S_t = decay S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t.  Returns (o [T][H][e], S [H][d][e])."""
    T, H, d = q.shape
    e = v.shape[2]
    S = torch.zeros((H, d, e), dtype=F64) if state is None else state.clone()
    o = torch.zeros((T, H, e), dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o, S


def right_linear_mixer(h, w, prefix, m, eps, rnd=lambda t: t):
    """Linear attention with a fixed decay per head: silu on q, k and v; the recurrence; RMS norm over all
    heads together with a weight; sigmoid gate; output projection."""
    T = h.shape[0]
    H, d, e = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    hr = rnd(h)
    q = rnd(silu(rnd(hr @ w[prefix + "q"].T))).view(T, H, d)
    k = rnd(silu(rnd(hr @ w[prefix + "k"].T))).view(T, H, d)
    v = rnd(silu(rnd(hr @ w[prefix + "v"].T))).view(T, H, e)
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=F64)
    o, _ = decayed_outer_state(q, k, v, decay)
    z = unit(o.reshape(T, H * e), eps) * w[prefix + "norm"]
    z = rnd(z * torch.sigmoid(rnd(hr @ w[prefix + "g"].T)))
    return z @ w[prefix + "o"].T


def parallel_mixer(h, w, prefix, m, eps, positions, rnd=lambda t: t):
    """Half the sum of the two halves' outputs, each RMS-normed over the width with its own weight."""
    left = left_attention_mixer(h, w, prefix + "left.", m["left"], eps, positions, rnd)
    right = right_linear_mixer(h, w, prefix + "right.", m["right"], eps, rnd)
    return 0.5 * (unit(left, eps) * w[prefix + "left.out"] + unit(right, eps) * w[prefix + "right.out"])


# ------------------------------------------------------------------ feed-forward, side input
def dense_feed_forward(h, w, prefix, rnd=lambda t: t):
    return rnd(relu_squared(rnd(rnd(h) @ w[prefix + "up"].T))) @ w[prefix + "down"].T


def token_side_input(x, tokens, w, prefix, index, dim, eps, rnd=lambda t: t):
    """What a layer adds from its own slice of the side table: e = side.embed[token][index*dim:(index+1)*dim];
    y = proj(gelu(gate x) * e); returns norm_weight * unit(y)."""
    e = w["side.embed"][tokens][:, index * dim:(index + 1) * dim]
    g = gelu_tanh(rnd(rnd(x) @ w[prefix + "gate"].T)) * e
    y = rnd(g) @ w[prefix + "proj"].T
    return unit(y, eps) * w[prefix + "norm"]


# ------------------------------------------------------------------ the whole model
def forward(config, weights, tokens, rnd=lambda t: t, layers_out=None):
    """Logits [T][vocab] of one whole sequence.  ``weights``: name -> tensor (any float dtype); with
    ``layers_out`` (a list) the stream after every layer is appended to it."""
    w = {name: (t.to(F64) if t.is_floating_point() else t) for name, t in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    eps = float(config["norm"]["eps"])
    x = w["embed"][tokens]
    side_dim = int((config.get("token_side") or {}).get("dim") or 0)
    v_first = None
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = unit(x, eps) * w[p + "norm1"]
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, v = window_attention_mixer(h, w, p + "mix.", m, eps, positions,
                                          v_first if mixes else None, rnd)
            if mixes and v_first is None:
                v_first = v
        else:
            y = parallel_mixer(h, w, p + "mix.", m, eps, positions, rnd)
        delta = y * w[p + "ls1"]
        if layer.get("mlp") is not None:
            delta = delta + dense_feed_forward(h, w, p + "mlp.", rnd) * w[p + "ls2"]
        x = x + delta
        if side_dim:
            x = x + token_side_input(x, tokens, w, p + "side.", index, side_dim, eps, rnd)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = unit(x, eps) * w["final.norm"]
    return (rnd(x) @ w["head"].T) * float(config.get("logit_scale", 1.0))


def greedy_generate(config, weights, prompt, n_new):
    """``n_new`` tokens, each the place of the largest logit behind everything so far; the whole sequence
    is run again for every token."""
    tokens = [int(t) for t in prompt]
    for _ in range(n_new):
        tokens.append(int(forward(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
