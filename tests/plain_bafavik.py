"""A plain, slow restatement of the Bafavik decoder in float64 torch on the CPU: one function per mechanism, whole
sequences, token-by-token loops for everything that carries state.  It shares no code with the package; the tests compare
the engine with it.

Notation: ``x`` is the residual stream ``[T, width]``, ``h`` a mixer's input, ``rms(v) = sqrt(mean(v^2) + eps)``.
``weights`` maps tensor names to float64 tensors, ``config`` is the ``config.json`` mapping.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_divide(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps)


def stream_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm of the stream: the stored weight lies around zero."""
    return rms_divide(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) + torch.log1p(torch.exp(-z.abs()))


# --------------------------------------------------------------------------- frame


def embed(tokens: list, weights: dict, config: dict) -> torch.Tensor:
    """Token rows times the scale, plus a row of the bigram table chosen by the token before and the token."""
    e = config["embedding"]
    x = weights["embed"][tokens] * e["scale"]
    bigram = e.get("bigram")
    if bigram:
        rows = []
        for t, token in enumerate(tokens):
            if t == 0:
                rows.append(bigram["buckets"])
            else:
                rows.append((tokens[t - 1] * bigram["mul_prev"] + token * bigram["mul_cur"]) % bigram["buckets"])
        x = x + weights["bigram"][rows]
    return x


def token_shift(h: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    """Every token's input moves towards the input of the token before it (zeros before the first)."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (before - h) * shift


def short_convolution(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y_t = sum_j w[:, j] u_(t - taps + 1 + j)`` per channel; ``u [T, C]``, ``w [C, taps]``; zeros before the start."""
    taps = w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, u.shape[1]), dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(taps):
            out[t] += w[:, j] * padded[t + j]
    return out


def rotate(v: torch.Tensor, dims: int, base: float, interleaved: bool) -> torch.Tensor:
    """``v [T, heads, dim]``: the first ``dims`` entries of each head are rotated by ``position * base^(-2i/dims)``; entry i
    is paired with entry ``i + dims/2``, or (``interleaved``) entry 2i with entry 2i + 1."""
    if dims == 0:
        return v
    out = v.clone()
    half = dims // 2
    for t in range(v.shape[0]):
        for i in range(half):
            angle = t * base ** (-2.0 * i / dims)
            a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
            c, s = math.cos(angle), math.sin(angle)
            out[t, :, a] = v[t, :, a] * c - v[t, :, b] * s
            out[t, :, b] = v[t, :, b] * c + v[t, :, a] * s
    return out


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, chunk=None) -> torch.Tensor:
    """``q [T, H, d]``, ``k [T, G, d]``, ``v [T, G, dv]``; query head j reads key/value head ``j // (H / G)``.  Position i sees
    j <= i, and with ``chunk`` only those of its own chunk (chunks counted from position 0)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            first = 0 if chunk is None else (i // chunk) * chunk
            scores = (k[first:i + 1, g] @ q[i, head]) * scale
            out[i, head] = torch.softmax(scores, dim=0) @ v[first:i + 1, g]
    return out


# --------------------------------------------------------------------------- mixers


def linear(h, weights, name, bias=False):
    y = h @ weights[name].T
    return y + weights[name + ".b"] if bias else y


def rotary_attention_with_norm(h, weights, p, m, eps):
    """Biased projections, half-split rotation, queries and keys divided by their root mean square, softmax attention."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, weights, p + "q", True).view(T, H, d)
    k = linear(h, weights, p + "k", True).view(T, G, d)
    v = linear(h, weights, p + "v", True).view(T, G, dv)
    q = rms_divide(rotate(q, m["rot"]["dims"], m["rot"]["base"], False), eps)
    k = rms_divide(rotate(k, m["rot"]["dims"], m["rot"]["base"], False), eps)
    return linear(softmax_attention(q, k, v, m["scale"]).reshape(T, H * dv), weights, p + "o", True)


def lightning_attention(h, weights, p, m, eps):
    """A matrix per head that decays by a constant of the head and receives ``k v^T``; read out with q."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(linear(h, weights, p + "q")).view(T, H, d)
    k = silu(linear(h, weights, p + "k")).view(T, H, d)
    v = silu(linear(h, weights, p + "v")).view(T, H, dv)
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    for head in range(H):
        S = torch.zeros((d, dv), dtype=h.dtype)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    y = rms_divide(out.reshape(T, H * dv), eps) * weights[p + "norm"]
    return linear(y * torch.sigmoid(linear(h, weights, p + "g")), weights, p + "o")


def differential_attention(h, weights, p, m, eps):
    """Two score maps per head over the same values; the second, times lambda, is taken off the first."""
    T = h.shape[0]
    H, G, d, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    q = linear(h, weights, p + "q", True).view(T, H, 2, d)
    k = linear(h, weights, p + "k", True).view(T, G, 2, d)
    v = linear(h, weights, p + "v", True).view(T, G, dv)
    chunk = m["mask"]["size"]
    first = softmax_attention(q[:, :, 0], k[:, :, 0], v, m["scale"], chunk)
    second = softmax_attention(q[:, :, 1], k[:, :, 1], v, m["scale"], chunk)
    lam = (torch.exp((weights[p + "lq1"] * weights[p + "lk1"]).sum()) - torch.exp((weights[p + "lq2"] * weights[p + "lk2"]).sum())
           + diff)
    o = rms_divide(first - lam * second, eps) * (1.0 - diff)
    gated = o.reshape(T, H * dv) * torch.sigmoid(linear(h, weights, p + "g"))
    return linear(gated, weights, p + "o")


def convolved_rotary_attention(h, weights, p, m):
    """Projections without biases, a short convolution on each, interleaved rotation, softmax attention, a gate per entry."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_convolution(linear(h, weights, p + "q"), weights[p + "q.conv"]).view(T, H, d)
    k = short_convolution(linear(h, weights, p + "k"), weights[p + "k.conv"]).view(T, G, d)
    v = short_convolution(linear(h, weights, p + "v"), weights[p + "v.conv"]).view(T, G, dv)
    q = rotate(q, m["rot"]["dims"], m["rot"]["base"], True)
    k = rotate(k, m["rot"]["dims"], m["rot"]["base"], True)
    attended = softmax_attention(q, k, v, m["scale"]).reshape(T, H * dv)
    return linear(attended * torch.sigmoid(linear(h, weights, p + "g")), weights, p + "o")


def gated_delta_rule(h, weights, p, m, eps):
    """The delta rule with a decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(linear(h, weights, p + "q"), weights[p + "q.conv"])).view(T, G, d)
    k = silu(short_convolution(linear(h, weights, p + "k"), weights[p + "k.conv"])).view(T, G, d)
    v = silu(short_convolution(linear(h, weights, p + "v"), weights[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(linear(h, weights, p + "b"))                                   # [T, H]
    step = softplus((h @ weights[p + "a1"].T) @ weights[p + "a2"].T + weights[p + "dt_bias"]).view(T, H, d)
    decay = torch.exp(-torch.exp(weights[p + "A_log"]).view(1, H, 1) * step)            # [T, H, d]
    out = torch.zeros((T, H, dv), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros((d, dv), dtype=h.dtype)
        for t in range(T):
            S = decay[t, head].unsqueeze(1) * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    gate = torch.sigmoid((h @ weights[p + "g1"].T) @ weights[p + "g2"].T).view(T, H, dv)
    y = rms_divide(out, eps) * weights[p + "norm"] * gate
    return linear(y.reshape(T, H * dv), weights, p + "o")


def mixer(kind: str, h, weights, p, m, eps):
    if kind == "attention":
        return differential_attention(h, weights, p, m, eps)
    if kind == "parallel":
        left = rotary_attention_with_norm(h, weights, p + "left.", m["left"], eps)
        right = lightning_attention(h, weights, p + "right.", m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    if kind == "parallel_2":
        left = convolved_rotary_attention(h, weights, p + "left.", m["left"])
        right = gated_delta_rule(h, weights, p + "right.", m["right"], eps)
        return 0.5 * (rms_divide(left, eps) * weights[p + "left.out"] + rms_divide(right, eps) * weights[p + "right.out"])
    raise ValueError(kind)


def feed_forward(h, weights, p):
    return torch.relu(h @ weights[p + "up"].T) ** 2 @ weights[p + "down"].T


# --------------------------------------------------------------------------- the model


def layer_order(config: dict) -> list:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def run_layer(x, index: int, weights, config):
    layer, eps, mult = config["layers"][index], config["norm"]["eps"], config["residual_mult"]
    p = f"l{index}."
    h = token_shift(stream_norm(x, weights[p + "norm1"], eps), weights[p + "shift"])
    x = x + mult * weights[p + "ls1"] * mixer(layer["type"], h, weights, p + "mix.", layer["mixer"], eps)
    if layer.get("mlp") is not None:
        x = x + mult * weights[p + "ls2"] * feed_forward(stream_norm(x, weights[p + "norm2"], eps), weights, p + "mlp.")
    return x


def forward(tokens: list, weights: dict, config: dict, streams: list = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence.  ``streams``: a list that receives the stream after every layer run."""
    x = embed(tokens, weights, config)
    for index in layer_order(config):
        x = run_layer(x, index, weights, config)
        if streams is not None:
            streams.append(x.clone())
    x = stream_norm(x, weights["final.norm"], config["norm"]["eps"])
    return (x @ weights["head"].T) * config["logit_scale"]
