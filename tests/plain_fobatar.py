"""A plain, slow implementation of the Fobatar design, one function per mechanism, in float64 torch on
the CPU.  It shares no code with the engine: tests compare the engine's parts and whole models with it.

Notation: W the model width, ``unit(y) = y / sqrt(mean(y^2) + eps)`` over the last axis, positions
count from 0 in every sequence, matrices are stored [out][in] and applied as ``y = x @ M.T``.

``rnd`` (optional, in some functions): a function applied where the serving precision rounds (inputs
of matrix products, cached rows); the identity by default.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

F64 = torch.float64


def same(value):
    return value


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


# ------------------------------------------------------------------ rotation
def banded_frequencies(rot):
    """f_i = base^(-2i/n), i < n/2.  With ``scaling`` (factor, original, fast, slow): the pair index at
    which a wave turns t times over ``original`` positions is c(t) = n ln(original / (2 pi t)) / (2 ln base);
    between lo = max(floor(c(fast)), 0) and hi = min(ceil(c(slow)), n - 1) a ramp r_i goes from 0 to 1, and
    the frequency becomes r_i f_i / factor + (1 - r_i) f_i.  Returns (frequencies, amplitude): cos and
    sin are both multiplied by amplitude = 0.1 ln(factor) + 1 (1 without scaling)."""
    n = int(rot["dims"])
    base = float(rot["base"])
    f = [base ** (-2.0 * i / n) for i in range(n // 2)]
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_index(turns):
        return n * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_index(float(scaling["slow"]))), n - 1)
    out = []
    for i, fi in enumerate(f):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * r + fi * (1.0 - r))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, rot):
    """x: [T][heads][d].  Channels (2i, 2i+1), i < dims/2, of every head turn by positions * f_i, scaled by
    the amplitude; the other channels pass."""
    n = int(rot["dims"])
    if n == 0:
        return x
    f, amplitude = banded_frequencies(rot)
    angle = positions.to(F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]          # [T][n/2]
    cos, sin = (torch.cos(angle) * amplitude)[:, None, :], (torch.sin(angle) * amplitude)[:, None, :]
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = a * cos - b * sin
    out[..., 1:n:2] = b * cos + a * sin
    return out


# ------------------------------------------------------------------ attention
def softmax_attention(q, k, v, q_pos, k_pos, scale, chunk=0, sink_zero=False):
    """q: [Tq][H][d], k: [Tk][G][d], v: [Tk][G][e]; query head h reads key/value head h // (H/G).  A key at
    position j is visible from position i when j <= i and, with ``chunk`` > 0, i // chunk == j // chunk.
    ``sink_zero``: the denominator of the softmax holds one more term, exp(0), without a value."""
    H, G = q.shape[1], k.shape[1]
    rep = H // G
    out = torch.zeros((q.shape[0], H, v.shape[2]), dtype=q.dtype)
    visible = k_pos[None, :] <= q_pos[:, None]
    if chunk > 0:
        visible &= (k_pos[None, :] // chunk) == (q_pos[:, None] // chunk)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, -math.inf)
        m = s.max(dim=1, keepdim=True).values
        if sink_zero:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        denom = e.sum(dim=1, keepdim=True)
        if sink_zero:
            denom = denom + torch.exp(-m)
        out[:, h] = (e / denom) @ v[:, g]
    return out


def causal_taps(u, taps, history=None):
    """u: [T][C], taps: [C][n].  y_t = sum_j taps[:, j] * u_(t - n + 1 + j); what lies before the sequence
    is zero, or ``history`` ([n - 1][C], the rows just before u)."""
    n = taps.shape[1]
    before = torch.zeros((n - 1, u.shape[1]), dtype=u.dtype) if history is None else history
    padded = torch.cat([before, u], dim=0)
    y = torch.zeros_like(u)
    for j in range(n):
        y = y + padded[j:j + u.shape[0]] * taps[:, j][None, :]
    return y


def chunked_attention_mixer(h, w, prefix, m, eps, positions, rnd=same):
    """The mixer 'attention': projections, a short causal convolution on each of q, k, v, RMS norm over the
    whole of q and of k, rotation, attention inside chunks with a zero sink, a gate per head, output."""
    H, G, d, e = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    hr = rnd(h)
    q, k, v = hr @ w[prefix + "q"].T, hr @ w[prefix + "k"].T, hr @ w[prefix + "v"].T
    if m.get("conv"):
        q, k, v = (causal_taps(t, w[prefix + name + ".conv"]) for t, name in ((q, "q"), (k, "k"), (v, "v")))
    q = unit(q, eps) * w[prefix + "q.norm"]
    k = unit(k, eps) * w[prefix + "k.norm"]
    T = h.shape[0]
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, e)
    if m.get("rot"):
        q, k = rotate_neighbours(q, positions, m["rot"]), rotate_neighbours(k, positions, m["rot"])
    chunk = int((m.get("mask") or {}).get("size") or 0)
    o = softmax_attention(rnd(q), rnd(k), rnd(v), positions, positions, float(m["scale"]), chunk, sink_zero=True)
    gate = torch.sigmoid(hr @ w[prefix + "g"].T)                   # [T][H]
    o = o * gate[:, :, None]
    return rnd(o.reshape(T, H * e)) @ w[prefix + "o"].T


def latent_attention_mixer(h, w, prefix, m, eps, positions, rnd=same):
    """The mixer 'latent_attention': per token a normed latent c and one turned key part shared by the heads;
    head keys U_h c and values V_h c; plain softmax over every earlier key; a gate per head; output."""
    H, d, r, e, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    T = h.shape[0]
    hr = rnd(h)
    q = (hr @ w[prefix + "q"].T).view(T, H, d + r)
    low = hr @ w[prefix + "dkv"].T
    c = rnd(unit(low[:, :rank], eps) * w[prefix + "dkv.norm"])
    rot = dict(m["rot"])
    rot["dims"] = r
    k_turned = rnd(rotate_neighbours(low[:, None, rank:], positions, rot))          # [T][1][r]
    q_turned = rotate_neighbours(q[:, :, d:], positions, rot)
    k_plain = (c @ w[prefix + "uk"].T).view(T, H, d)
    value = (c @ w[prefix + "uv"].T).view(T, H, e)
    keys = torch.cat([k_plain, k_turned.expand(T, H, r)], dim=-1)
    queries = torch.cat([q[:, :, :d], q_turned], dim=-1)
    o = softmax_attention(rnd(queries), keys, value, positions, positions, float(m["scale"]))
    gate = torch.sigmoid(hr @ w[prefix + "g"].T)
    o = o * gate[:, :, None]
    return rnd(o.reshape(T, H * e)) @ w[prefix + "o"].T


# ------------------------------------------------------------------ feed-forward
def clamped_gated_expert(h, gate, up, down, limit, rnd=same):
    """g = min(gate h, limit), u = clamp(up h, -limit, limit); down(g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return rnd(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def table_experts(h, tokens, w, prefix, mlp, rnd=same):
    """Every token id names its experts in a table; each counts 1/top; a shared expert is added."""
    top = int(mlp["router"]["top"])
    limit = float(mlp["expert"]["limit"])
    table = w[prefix + "table"]
    hr = rnd(h)
    out = torch.zeros_like(h)
    for t, token in enumerate(tokens):
        for slot in range(top):
            j = int(table[int(token), slot])
            out[t] += clamped_gated_expert(hr[t:t + 1], w[f"{prefix}e{j}.gate"], w[f"{prefix}e{j}.up"],
                                           w[f"{prefix}e{j}.down"], limit, rnd)[0] / top
    shared = mlp.get("shared")
    if shared:
        out = out + clamped_gated_expert(hr, w[prefix + "shared.gate"], w[prefix + "shared.up"],
                                         w[prefix + "shared.down"], float(shared["limit"]), rnd)
    return out


# ------------------------------------------------------------------ the model
def layer_runs(config):
    """(layer index, first of a repeated pass) in the order the layers run: layers start .. stop-1 run
    ``times`` times in a row, every pass but the first marked."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or int(loop["stop"]) <= int(loop["start"]):
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(start)]
    for p in range(times):
        runs += [(i, p > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def forward(config, weights, tokens, rnd=same, layers_out=None):
    """Logits [T][vocab] of one sequence from position 0.  ``layers_out``: a list that receives the stream
    behind every layer run."""
    w = weights
    eps = float(config["norm"]["eps"])
    mult = float(config["residual_mult"])
    tokens = [int(t) for t in tokens]
    positions = torch.arange(len(tokens))
    first = w["embed"][tokens] * float(config["embedding"]["scale"])
    x = first.clone()
    for index, again in layer_runs(config):
        layer = config["layers"][index]
        p = f"l{index}."
        if again:
            x = x + first
        mixer = {"attention": chunked_attention_mixer, "latent_attention": latent_attention_mixer}[layer["type"]]
        y = mixer(unit(x, eps) * w[p + "norm1"], w, p + "mix.", layer["mixer"], eps, positions, rnd)
        x = x + mult * (unit(y, eps) * w[p + "norm1b"])
        if layer.get("mlp") is not None:
            y = table_experts(unit(x, eps) * w[p + "norm2"], tokens, w, p + "mlp.", layer["mlp"], rnd)
            x = x + mult * (unit(y, eps) * w[p + "norm2b"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return rnd(unit(x, eps) * w["final.norm"]) @ rnd(w["embed"]).T


def greedy_generate(config, weights, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(config, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]
