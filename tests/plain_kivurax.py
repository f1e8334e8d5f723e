"""A plain, slow statement of the Kivurax decoder in float64: one function per mechanism, whole sequences, every
recurrence walked token by token.  It shares no code with the package; the tests compare the engine with it.

Notation: ``h [T, width]`` is a sublayer's input (the residual stream itself: this design norms a sublayer's OUTPUT
only), ``w`` the dictionary of tensors, ``p`` the prefix of the part's tensor names, ``m`` the part's section of
``config.json``, ``rms(v) = sqrt(mean(v^2) + eps)``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F64 = torch.float64


def load_folder(folder):
    from safetensors.torch import load_file

    config = json.loads((Path(folder) / "config.json").read_text())
    weights = {k: v.to(F64) for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}
    return config, weights


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(u, weight, bias=None):
    """``out[t, c] = bias[c] + sum_k weight[c, k] u[t - (taps - 1 - k), c]`` with zeros before the start."""
    T, taps = u.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=F64), u], dim=0)
    out = torch.zeros_like(u)
    for k in range(taps):
        out = out + padded[k:k + T] * weight[:, k]
    return out if bias is None else out + bias


# --------------------------------------------------------------------------- mixer: matrix memory with exponential gates


def mlstm(h, w, p, m, eps):
    heads, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, heads, dim) * dim ** -0.5
    k = (h @ w[p + "k"].T).view(T, heads, dim)
    v = (h @ w[p + "v"].T).view(T, heads, vdim)
    log_i = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    log_f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    S = torch.zeros(heads, dim, vdim, dtype=F64)
    n = torch.zeros(heads, dim, dtype=F64)
    peak = torch.zeros(heads, dtype=F64)             # the running maximum starts at 0
    out = torch.zeros(T, heads, vdim, dtype=F64)
    for t in range(T):
        new_peak = torch.maximum(log_f[t] + peak, log_i[t])
        keep = torch.exp(log_f[t] + peak - new_peak)
        write = torch.exp(log_i[t] - new_peak)
        S = keep[:, None, None] * S + write[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[t]
        peak = new_peak
        top = torch.einsum("hdv,hd->hv", S, q[t])
        bottom = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-peak)) + 1e-6
        out[t] = top / bottom[:, None]
    out = unit_rms(out, eps).reshape(T, heads * vdim) * w[p + "norm"]
    out = out * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# --------------------------------------------------------------------------- mixer: windowed attention beside a gated linear recurrence


def rotation_frequencies(rot):
    dims, base = rot["dims"], float(rot["base"])
    freqs = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    magnitude = 1.0
    scaling = rot.get("scaling")
    if scaling:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def where(turns):
            return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(where(float(scaling["fast"]))), 0)
        hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
        for i in range(dims // 2):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            freqs[i] = freqs[i] / factor * ramp + freqs[i] * (1.0 - ramp)
        magnitude = 0.1 * math.log(factor) + 1.0
    return torch.tensor(freqs, dtype=F64), magnitude


def rotate_pairs(x, rot, first_position=0):
    """Neighbouring entries (2i, 2i + 1) of the first ``dims`` entries of every head of ``x [T, heads, d]`` turn by
    ``position * f_i``."""
    dims = rot["dims"]
    if not dims:
        return x
    freqs, magnitude = rotation_frequencies(rot)
    positions = torch.arange(first_position, first_position + x.shape[0], dtype=F64)
    angle = positions[:, None] * freqs[None, :]
    cos, sin = (magnitude * angle.cos())[:, None, :], (magnitude * angle.sin())[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def window_attention(h, w, p, m, eps):
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, heads, dim)
    k = (h @ w[p + "k"].T).view(T, groups, dim)
    v = k.clone()                                    # the values are the keys as projected
    assert vdim == dim
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    q, k = rotate_pairs(q, m["rot"]), rotate_pairs(k, m["rot"])
    size = m["mask"]["size"]
    out = torch.zeros(T, heads, vdim, dtype=F64)
    for head in range(heads):
        g = head // (heads // groups)
        for i in range(T):
            lo = max(0, i - size + 1)
            s = (k[lo:i + 1, g] @ q[i, head]) * float(m["scale"])
            peak = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - peak)
            weights = e / (torch.exp(-peak) + e.sum())      # one more term in the denominator: a key of score 0 without a value
            out[i, head] = weights @ v[lo:i + 1, g]
    return out.reshape(T, heads * vdim) @ w[p + "o"].T


def gated_linear_recurrence(h, w, p, m):
    width, blocks = m["width"], m["blocks"]
    T = h.shape[0]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    part = width // blocks
    ub = u.view(T, blocks, part)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ra"], ub) + w[p + "ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ri"], ub) + w[p + "ri.b"]).reshape(T, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    S = torch.zeros(width, dtype=F64)
    out = torch.zeros(T, width, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ w[p + "o"].T


def side_by_side(h, w, p, m, eps):
    left = window_attention(h, w, p + "left.", m["left"], eps)
    right = gated_linear_recurrence(h, w, p + "right.", m["right"])
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# --------------------------------------------------------------------------- mixer: gated delta rule


def delta_rule(h, w, p, m, eps):
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, groups, dim)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, groups, dim)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, heads, vdim)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    per = heads // groups
    S = torch.zeros(heads, dim, vdim, dtype=F64)
    out = torch.zeros(T, heads, vdim, dtype=F64)
    for t in range(T):
        kt = k[t].repeat_interleave(per, dim=0)      # head j reads q/k head j // per
        qt = q[t].repeat_interleave(per, dim=0)
        S = decay[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, qt)
    out = unit_rms(out, eps) * w[p + "norm"]
    out = out.reshape(T, heads * vdim) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forwards


def dense(h, w, p):
    gate = h @ w[p + "gate"].T + w[p + "gate.b"]
    up = h @ w[p + "up"].T + w[p + "up.b"]
    return (silu(gate) * up) @ w[p + "down"].T + w[p + "down.b"]


def route(h, w, p, mlp):
    """(ids [T, top], weights [T, top], the smallest gap between a chosen and a not-chosen score)."""
    top = mlp["router"]["top"]
    scores = torch.sigmoid(h @ w[p + "router"].T)
    ordered = torch.sort(scores, dim=-1, descending=True, stable=True)
    ids, weights = ordered.indices[:, :top], ordered.values[:, :top]
    gap = float("inf")
    if top < scores.shape[1]:
        gap = float((ordered.values[:, top - 1] - ordered.values[:, top]).min())
    return ids, weights, gap


def mixture(h, w, p, mlp):
    ids, weights, _ = route(h, w, p, mlp)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, weight in zip(ids[t].tolist(), weights[t]):
            x = weight * h[t]                        # the weight multiplies the expert's input
            e_p = f"{p}e{e}."
            out[t] += (silu(w[e_p + "gate"] @ x) * (w[e_p + "up"] @ x)) @ w[e_p + "down"].T
    return out


def feed_forward(h, w, p, mlp):
    return dense(h, w, p) if mlp["kind"] == "dense" else mixture(h, w, p, mlp)


# --------------------------------------------------------------------------- the model


def mixer(h, w, p, layer, eps):
    kind, m = layer["type"], layer["mixer"]
    if kind == "mlstm":
        return mlstm(h, w, p, m, eps)
    if kind == "parallel":
        return side_by_side(h, w, p, m, eps)
    if kind == "delta":
        return delta_rule(h, w, p, m, eps)
    raise ValueError(kind)


def forward(tokens, w, config, streams=None):
    """float64 logits ``[T, vocab]``; ``streams``: a list that receives the residual stream after every layer."""
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        x = x + mult * unit_rms(mixer(x, w, p + "mix.", layer, eps), eps) * w[p + "norm1"]
        if layer.get("mlp") is not None:
            x = x + mult * unit_rms(feed_forward(x, w, p + "mlp.", layer["mlp"]), eps) * w[p + "norm2"]
        if streams is not None:
            streams.append(x.clone())
    x = unit_rms(x, eps) * w["final.norm"]
    return x @ w["embed"].T
