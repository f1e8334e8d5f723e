"""Plain PyTorch statements of what each kernel entry point computes.

Two uses: the GPU tests compare every kernel alone with the function of the same name here
(computed in float64 from the same inputs), and the CPU tests put these functions in the
kernels' place (``install``) so that the host-side logic of the engine (batching, cache
manager, step function) can be exercised on a machine without a GPU.  Nothing here is used by
the package itself.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

import plain_qwen3 as plain


def scale_softcap(x, scale=1.0, cap=None):
    x.mul_(scale)
    if cap:
        x.copy_(cap * torch.tanh(x / cap))


def embedding(tokens, table, out, scale=1.0):
    out.copy_((scale * table[tokens.long()].double()).to(out.dtype))


def add_rmsnorm(residual, delta, weight, eps, out, rows=None, delta2=None):
    if delta2 is not None:
        delta = delta2 if delta is None else (delta.double() + delta2.double())
    if rows is None:
        if delta is not None:
            residual += delta.to(residual.dtype)
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].to(residual.dtype)
    x = x.double()
    y = weight.double() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))
    out.copy_(y.to(out.dtype))


def rmsnorm(x, weight, eps, out):
    xd = x.double()
    y = weight.double() * (xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps))
    out.copy_(y.to(out.dtype))


def rope_table(positions, inv_freq, cos_sin, magnitude=1.0):
    angles = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).double()
    cos_sin[..., 0] = (magnitude * angles.cos()).to(cos_sin.dtype)
    cos_sin[..., 1] = (magnitude * angles.sin()).to(cos_sin.dtype)


def rotate(x, cos_sin, rotary_dim, interleaved):
    """x [N, heads, d] float64; cos_sin [N, rotary_dim/2, 2]."""
    cos, sin = cos_sin[..., 0].double()[:, None, :], cos_sin[..., 1].double()[:, None, :]
    out = x.clone()
    half = rotary_dim // 2
    if interleaved:
        a, b = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2] = a * cos - b * sin
        out[..., 1:rotary_dim:2] = b * cos + a * sin
    else:
        a, b = x[..., :half], x[..., half:rotary_dim]
        out[..., :half] = a * cos - b * sin
        out[..., half:rotary_dim] = b * cos + a * sin
    return out


def qk_norm_rope_append(qkv, slots, q_weight, k_weight, eps, cos_sin, rotary_dim, interleaved, k_pool, v_pool,
                        n_q, n_kv, head_dim, q_out):
    n = qkv.shape[0]
    heads = qkv.view(n, n_q + 2 * n_kv, head_dim).double()
    q, k, v = heads[:, :n_q], heads[:, n_q:n_q + n_kv], heads[:, n_q + n_kv:]

    def norm(x, w):
        if w is None:
            return x
        return w.double() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))

    q, k = norm(q, q_weight), norm(k, k_weight)
    if cos_sin is not None:
        q, k = rotate(q, cos_sin, rotary_dim, interleaved), rotate(k, cos_sin, rotary_dim, interleaved)
    q_out.copy_(q.to(q_out.dtype))
    page_size = k_pool.shape[2]
    for token in range(n):
        slot = int(slots[token])
        if slot < 0:
            continue
        page, offset = divmod(slot, page_size)
        k_pool[page, :, offset, :] = k[token].to(k_pool.dtype)
        v_pool[page, :, offset, :] = v[token].to(v_pool.dtype)


def silu_mul(gate_up, out, paired=False, bias=None):
    n, inter = out.shape
    if bias is not None:
        gate_up = gate_up.double() + bias.double()
    if paired:      # blocks of sixteen columns: eight of the gate, then the same eight of the up projection
        blocks = gate_up.reshape(n, inter // 8, 2, 8)
        g, u = blocks[:, :, 0].reshape(n, inter).double(), blocks[:, :, 1].reshape(n, inter).double()
    else:
        g, u = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


def _row_factor(row_stats, size):
    """1 / rms of every row from the partial sums of squares that a folded norm left (kernels.RowStats)."""
    total = row_stats.partials[:row_stats.count].double().sum(dim=0)
    return 1.0 / torch.sqrt(total / size + row_stats.eps)


def gated_up(x, weight, out, row_stats=None):
    gate_up = x.double() @ weight.double().T
    if row_stats is not None:
        gate_up = gate_up * _row_factor(row_stats, x.shape[1])[:x.shape[0], None]
    silu_mul(gate_up.to(x.dtype), out, paired=True)


FOLD_BLOCKS = 3     # the plain stand-in leaves its sums of squares in this many rows, as a kernel of three blocks would


def linear_residual(x, weight, residual, norm_weight, eps, x_next, partials):
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels

    residual += (x.double() @ weight.double().T).to(residual.dtype)
    x_next.copy_((residual.double() * norm_weight.double()).to(x_next.dtype))
    partials.zero_()
    for block, columns in enumerate(torch.arange(residual.shape[1]).chunk(FOLD_BLOCKS)):
        partials[block, :residual.shape[0]] = residual[:, columns].double().pow(2).sum(dim=1).to(partials.dtype)
    return kernels.RowStats(partials, FOLD_BLOCKS, eps, per_row=partials.shape[1] != 8)


def linear_add(x, weight, residual):
    residual += (x.double() @ weight.double().T).to(residual.dtype)


def paged_attention(q, k_pool, v_pool, block_tables, request_of_token, positions, query_start, context_lens,
                    max_query_len, max_context_len, scale, window, out, host_query_start=None, softcap=None,
                    bias_slopes=None, sink=False, gate=None, gate_col=0, chunk=None):
    n, n_q, d = q.shape
    n_kv, page_size = k_pool.shape[1], k_pool.shape[2]
    group = n_q // n_kv
    for token in range(n):
        pos = int(positions[token])
        table = block_tables[int(request_of_token[token])]
        first = max(0, pos - window + 1) if window else 0
        if chunk:
            first = max(first, pos - pos % chunk)
        keys = torch.arange(first, pos + 1)
        pages = table[(keys // page_size).long()].long()
        offsets = (keys % page_size).long()
        k = k_pool[pages, :, offsets, :].double()      # [keys, n_kv, d]
        v = v_pool[pages, :, offsets, :].double()      # [keys, value heads, dv]
        n_v = v.shape[1]
        for head in range(n_q):
            scores = (k[:, head // group, :] @ q[token, head].double()) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if bias_slopes is not None:
                scores = scores + float(bias_slopes[head]) * (keys - pos).double()
            if sink:        # one more term exp(0) in the denominator: a key of score 0 without a value
                top = torch.clamp(scores.max(), min=0.0)
                e = torch.exp(scores - top)
                p = e / (e.sum() + torch.exp(-top))
            else:
                p = torch.softmax(scores, dim=0)
            result = p @ v[:, (head // group) % n_v, :]
            if gate is not None:
                result = result * torch.sigmoid(gate[token, gate_col + head].double())
            out[token, head] = result.to(out.dtype)


def linear(x, weight, out, row_stats=None):
    product = x.double() @ weight.double().T
    if row_stats is not None:
        product = product * _row_factor(row_stats, x.shape[1])[:x.shape[0], None]
    out.copy_(product.to(out.dtype))


def gated_linear(gate_up, weight, out):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].double(), gate_up[:, inter:].double()
    hidden = (g * torch.sigmoid(g) * u).to(gate_up.dtype)
    out.copy_((hidden.double() @ weight.double().T).to(out.dtype))


def sample(logits, records, slot_of_row, draw_index, out):
    import struct

    for row in range(logits.shape[0]):
        if records is None:
            out[row] = int(torch.argmax(logits[row]))
            continue
        words = records[int(slot_of_row[row])].tolist()
        temperature, top_p, top_k, seed_lo, seed_hi, *_ = struct.unpack("<ffiIIiii", struct.pack("<8i", *words))
        out[row] = plain.plain_sample(logits[row].cpu(), temperature, top_k, top_p, seed_lo | (seed_hi << 32),
                                      int(draw_index[row]))


# --------------------------------------------------------------------------- latent attention


def latent_prepare(proj, q_col, dkv_col, heads, dim, rot, rank, slots, norm_weight, eps, cos_sin, rot_dims, cache, q_full):
    n = proj.shape[0]
    p = proj.double()

    def turn(x):                       # x [n, ..., rot]: the first rot_dims entries rotated, entry i with i + rot_dims / 2
        if cos_sin is None or not rot_dims:
            return x
        half = rot_dims // 2
        shape = [n] + [1] * (x.dim() - 2) + [half]
        cos, sin = cos_sin[..., 0].double().view(shape), cos_sin[..., 1].double().view(shape)
        out = x.clone()
        u, v = x[..., :half], x[..., half:rot_dims]
        out[..., :half], out[..., half:rot_dims] = u * cos - v * sin, v * cos + u * sin
        return out

    q = p[:, q_col:q_col + heads * (dim + rot)].view(n, heads, dim + rot)
    q_full[:, :, rank:] = turn(q[..., dim:]).to(q_full.dtype)
    latent = p[:, dkv_col:dkv_col + rank]
    latent = norm_weight.double() * (latent * torch.rsqrt(latent.pow(2).mean(-1, keepdim=True) + eps))
    rows = torch.cat([latent, turn(p[:, dkv_col + rank:dkv_col + rank + rot])], dim=1).to(cache.dtype)
    flat = cache.view(-1, rank + rot)
    for token in range(n):
        if int(slots[token]) >= 0:
            flat[int(slots[token])] = rows[token]


def latent_attention(q_full, cache, block_tables, request_of_token, positions, query_start, context_lens, max_query_len,
                     max_context_len, rank, scale, window, out):
    n, heads, dk = q_full.shape
    page_size = cache.shape[1]
    for token in range(n):
        pos = int(positions[token])
        table = block_tables[int(request_of_token[token])]
        first = max(0, pos - window + 1) if window else 0
        keys = torch.arange(first, pos + 1)
        rows = cache[table[(keys // page_size).long()].long(), (keys % page_size).long()].double()     # [keys, dk]
        for head in range(heads):
            p = torch.softmax((rows @ q_full[token, head].double()) * scale, dim=0)
            out[token, head] = (p @ rows[:, :rank]).to(out.dtype)


def head_gate(x, gate, gate_col):
    heads = x.shape[1]
    x.copy_((x.double() * torch.sigmoid(gate[:, gate_col:gate_col + heads].double())[:, :, None]).to(x.dtype))


def linear_batched(x, weight, out):
    out.copy_(torch.einsum("bmk,bnk->bmn", x.double(), weight.double()).to(out.dtype))


# --------------------------------------------------------------------------- routed experts


def router_topk(x, weight, bias, top, ids, weights, scratch=None, *, choose_from=None, scoring="chosen_softmax",
                correction=None, groups=(1, 1)):
    logits = x.double() @ weight.double().T
    if bias is not None:
        logits = logits + bias.double()
    if scratch is not None:
        scratch.copy_(logits.to(scratch.dtype))
    if scoring in ("all_softmax", "sigmoid"):
        total = logits.shape[1] if choose_from is None else choose_from
        n = logits.shape[0]
        scores = torch.softmax(logits[:, :total], dim=1) if scoring == "all_softmax" else torch.sigmoid(logits[:, :total])
        choice = scores if correction is None else scores + correction.double()
        count, keep = groups
        if keep < count:
            best = choice.view(n, count, total // count).max(dim=2).values
            kept = torch.zeros(n, count, dtype=torch.bool)
            kept.scatter_(1, best.sort(dim=1, descending=True, stable=True).indices[:, :keep], True)
            choice = choice.masked_fill(~kept[:, :, None].expand(n, count, total // count).reshape(n, total), -math.inf)
        chosen = choice.sort(dim=1, descending=True, stable=True).indices[:, :top]
        ids.copy_(chosen.to(ids.dtype))
        weights.copy_(torch.gather(scores, 1, chosen).to(weights.dtype))
        return
    ranked = logits.sort(dim=1, descending=True, stable=True)
    ids.copy_(ranked.indices[:, :top].to(ids.dtype))
    weights.copy_(torch.softmax(ranked.values[:, :top], dim=1).to(weights.dtype))


def expert_route(ids, experts, offsets, order, place):
    flat = ids.reshape(-1).long()
    sorted_pairs = torch.sort(flat, stable=True).indices
    order.copy_(sorted_pairs.to(order.dtype))
    place[sorted_pairs] = torch.arange(flat.numel(), dtype=place.dtype)
    counts = torch.bincount(flat, minlength=experts)
    offsets[0] = 0
    offsets[1:] = counts.cumsum(0).to(offsets.dtype)


def clamped_glu_values(gate, up, limit):
    g, u = gate.clamp(max=limit), up.clamp(min=-limit, max=limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def clamped_glu(both, limit, out):
    both = both.double()
    out.copy_(clamped_glu_values(both[:, 0::2], both[:, 1::2], limit).to(out.dtype))


def expert_linear(x, order, top, weight, out, offsets, relu_square=False, activation="none", limit=0.0, pair_scale=None):
    for e in range(weight.shape[0]):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi == lo:
            continue
        rows = x[(order[lo:hi] // top).long()] if order is not None else x[lo:hi]
        y = rows.double() @ weight[e].double().T
        if relu_square or activation == "relu_square":
            y = y.clamp(min=0).pow(2)
        elif activation == "clamped_glu":
            y = clamped_glu_values(y[:, 0::2], y[:, 1::2], limit)
        elif activation == "silu_glu":
            if pair_scale is not None:
                y = y * pair_scale.double().reshape(-1)[order[lo:hi].long()][:, None]
            y = y[:, 0::2] * torch.sigmoid(y[:, 0::2]) * y[:, 1::2]
        out[lo:hi] = y.to(out.dtype)


def expert_combine(y, place, weights, shared, out, ids=None, first_identity=0, x=None, shared_gate=None, shared_gate_col=0):
    n = out.shape[0]
    top = place.numel() // max(n, 1) if weights is None else weights.shape[1]
    if weights is None:
        weights = torch.ones(n, top, dtype=torch.float64)
    picked = y.double()[place.long()].view(n, top, -1)
    if ids is not None:
        identity = (ids.long() >= first_identity)[:, :, None]
        picked = torch.where(identity, x.double()[:, None, :].expand_as(picked), picked)
    total = (weights.double()[:, :, None] * picked).sum(dim=1)
    if shared is not None:
        share = shared.double()
        if shared_gate is not None:
            share = share * torch.sigmoid(shared_gate[:, shared_gate_col].double())[:, None]
        total = total + share
    out.copy_(total.to(out.dtype))


def relu_square(x):
    x.copy_(x.double().clamp(min=0).pow(2).to(x.dtype))


# --------------------------------------------------------------------------- norms on both sides, free projection layouts


def postnorm_add_rmsnorm(residual, delta, post_weight, post_eps, weight, eps, out, rows=None, post_scale=1.0, post_norm=True):
    add = 0.0
    if delta is not None:
        d = delta.double()
        if post_norm:
            d = d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + post_eps)
        add = post_scale * post_weight.double() * d
    if rows is None:
        if delta is not None:
            residual += add.to(residual.dtype)
        x = residual.double()
    else:
        x = (residual.double() + add)[rows.long()]
    if weight is not None:
        x = weight.double() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))
    out.copy_(x.to(out.dtype))


def qkv_prepare(proj, q_col, k_col, v_col, n_q, n_kv, head_dim, value_dim, slots, q_weight, k_weight, eps, cos_sin,
                rotary_dim, k_pool, v_pool, q_out, interleaved=False, bias=None, value_heads=None):
    n = proj.shape[0]
    if bias is not None:
        proj = proj.double() + bias.double()

    def heads(col, count, size, weight):
        x = proj[:, col:col + count * size].double().view(n, count, size)
        if weight is not None:
            x = weight.double() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))
        if cos_sin is not None:
            x = rotate(x, cos_sin, rotary_dim, interleaved)
        return x

    q_out.copy_(heads(q_col, n_q, head_dim, q_weight).to(q_out.dtype))
    if k_col < 0:
        return
    k = heads(k_col, n_kv, head_dim, k_weight)
    value_heads = n_kv if value_heads is None else value_heads
    v = proj[:, v_col:v_col + value_heads * value_dim].view(n, value_heads, value_dim)
    page_size = k_pool.shape[2]
    for token in range(n):
        slot = int(slots[token])
        if slot < 0:
            continue
        k_pool[slot // page_size, :, slot % page_size, :] = k[token].to(k_pool.dtype)
        v_pool[slot // page_size, :, slot % page_size, :] = v[token].to(v_pool.dtype)


# --------------------------------------------------------------------------- state-space mixer


def causal_conv_silu(proj, col, weight, bias, states, state_offset, state_slots, query_start, max_query_len, out):
    causal_conv(proj, col, weight, bias, states, state_offset, state_slots, query_start, max_query_len, out)


def causal_conv(proj, col, weight, bias, states, state_offset, state_slots, query_start, max_query_len, out, activation="silu",
                in_bias=None):
    channels, taps = weight.shape
    keep = taps - 1
    for r in range(state_slots.numel()):
        lo, hi = int(query_start[r]), int(query_start[r + 1])
        if hi == lo:
            continue
        state = states[int(state_slots[r]), state_offset:state_offset + keep * channels].view(keep, channels)
        fresh = proj[lo:hi, col:col + channels].double()
        if in_bias is not None:
            fresh = fresh + in_bias.double()
        u = torch.cat([state.double(), fresh], dim=0)      # inputs -keep .. hi - lo - 1
        total = torch.zeros(hi - lo, channels, dtype=torch.float64) if bias is None else bias.double().expand(hi - lo, -1).clone()
        for k in range(taps):
            total = total + u[k:k + hi - lo] * weight[:, k].double()
        out[lo:hi] = (total * torch.sigmoid(total) if activation == "silu" else total).to(out.dtype)
        state.copy_(u[u.shape[0] - keep:].to(state.dtype))


def selective_scan(conv, proj, dt_col, dt_bias, a_log, d, states, state_offset, state_slots, query_start, heads, head_dim,
                   state, groups, y, max_query_len=None):
    inner = heads * head_dim
    for r in range(state_slots.numel()):
        lo, hi = int(query_start[r]), int(query_start[r + 1])
        kept = states[int(state_slots[r]), state_offset:state_offset + inner * state].view(heads, head_dim, state)
        S = kept.double()
        for t in range(lo, hi):
            x = conv[t, :inner].double().view(heads, head_dim)
            B = conv[t, inner:inner + groups * state].double().view(groups, state).repeat_interleave(heads // groups, dim=0)
            C = conv[t, inner + groups * state:].double().view(groups, state).repeat_interleave(heads // groups, dim=0)
            step = torch.nn.functional.softplus(proj[t, dt_col:dt_col + heads].double() + dt_bias.double(), threshold=30.0)
            decay = torch.exp(-torch.exp(a_log.double()) * step)
            S = decay[:, None, None] * S + (step[:, None] * x)[:, :, None] * B[:, None, :]
            y[t] = ((S * C[:, None, :]).sum(-1) + d.double()[:, None] * x).reshape(inner).to(y.dtype)
        kept.copy_(S.to(kept.dtype))


def gated_group_norm(y, proj, z_col, weight, groups, eps, out):
    n, inner = y.shape
    z = proj[:, z_col:z_col + inner].double()
    v = (y.double() * z * torch.sigmoid(z)).view(n, groups, inner // groups)
    v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, inner)
    out.copy_((v * weight.double()).to(out.dtype))


# --------------------------------------------------------------------------- recurrences that carry a matrix or a vector


def add_bias(x, bias):
    x.copy_((x.double() + bias.double()).to(x.dtype))


def scaled_sum(a, a_scale, b, b_scale, out):
    out.copy_((a_scale * a.double() + b_scale * b.double()).to(out.dtype))


def small_linear_f32(x, weight, bias, out):
    y = x.double() @ weight.double().T
    out.copy_((y if bias is None else y + bias.double()).to(out.dtype))


def unit_norm_heads(x, col, heads, dim, eps, scale):
    v = x[:, col:col + heads * dim].double().view(-1, heads, dim)
    v = scale * v / torch.sqrt(v.pow(2).sum(-1, keepdim=True) + eps)
    x[:, col:col + heads * dim] = v.reshape(-1, heads * dim).to(x.dtype)


def exponential_gates(logits, cap, states, state_offset, state_slots, query_start, max_query_len, gates):
    heads = gates.shape[1]
    squashed = cap * torch.tanh(logits.double() / cap)
    log_i, log_f = squashed[:, :heads], torch.nn.functional.logsigmoid(squashed[:, heads:])
    for r in range(state_slots.numel()):
        lo, hi = int(query_start[r]), int(query_start[r + 1])
        kept = states[int(state_slots[r]), state_offset:state_offset + heads]
        peak = kept.double()
        for t in range(lo, hi):
            new_peak = torch.maximum(log_f[t] + peak, log_i[t])
            gates[t, :, 0] = torch.exp(log_f[t] + peak - new_peak).to(gates.dtype)
            gates[t, :, 1] = torch.exp(log_i[t] - new_peak).to(gates.dtype)
            gates[t, :, 2] = torch.exp(-new_peak).to(gates.dtype)
            peak = new_peak
        if hi > lo:
            kept.copy_(peak.to(kept.dtype))


def decay_gates(logits, a_log, dt_bias, gates):
    heads = gates.shape[1]
    step = torch.nn.functional.softplus(logits[:, heads:].double() + dt_bias.double(), threshold=50.0)
    gates[:, :, 0] = torch.exp(-torch.exp(a_log.double()) * step).to(gates.dtype)
    gates[:, :, 1] = torch.sigmoid(logits[:, :heads].double()).to(gates.dtype)


def matrix_scan(mode, q, q_col, k, k_col, v, v_col, gates, states, state_offset, state_slots, query_start, max_query_len, heads,
                kv_heads, dim, vdim, y, q_scale=1.0, bottom=None, gate_col=0, channel_decay=None, input_activation="none"):
    per = heads // kv_heads

    def act(x):
        return x * torch.sigmoid(x) if input_activation == "silu" else x

    columns = vdim + 1 if mode == "memory" else vdim
    for r in range(state_slots.numel()):
        lo, hi = int(query_start[r]), int(query_start[r + 1])
        if hi == lo:
            continue
        kept = states[int(state_slots[r]), state_offset:state_offset + heads * columns * dim].view(heads, columns, dim)
        S = kept.double().clone()                # [head, column, dim]: column c of the matrix, the last one n
        for t in range(lo, hi):
            qt = (q_scale * act(q[t, q_col:q_col + kv_heads * dim].double())).view(kv_heads, dim).repeat_interleave(per, dim=0)
            kt = act(k[t, k_col:k_col + kv_heads * dim].double()).view(kv_heads, dim).repeat_interleave(per, dim=0)
            vt = act(v[t, v_col:v_col + heads * vdim].double()).view(heads, vdim)
            if mode == "decay":
                S = gates.double()[:, None, None] * S + vt[:, :, None] * kt[:, None, :]
                y[t] = torch.einsum("hcd,hd->hc", S, qt).to(y.dtype)
                continue
            if mode == "channel_delta":
                beta = torch.sigmoid(gates[t, gate_col:gate_col + heads].double())
                S = channel_decay[t].double().view(heads, 1, dim) * S
                u = beta[:, None] * (vt - torch.einsum("hcd,hd->hc", S, kt))
                S = S + u[:, :, None] * kt[:, None, :]
                y[t] = torch.einsum("hcd,hd->hc", S, qt).to(y.dtype)
                continue
            g = gates[t].double()
            if mode == "memory":
                vt = torch.cat([vt, torch.ones(heads, 1, dtype=torch.float64)], dim=1)
                S = g[:, 0, None, None] * S + g[:, 1, None, None] * vt[:, :, None] * kt[:, None, :]
                read = torch.einsum("hcd,hd->hc", S, qt)
                y[t] = read[:, :vdim].to(y.dtype)
                bottom[t] = (torch.maximum(read[:, vdim].abs(), g[:, 2]) + 1e-6).to(bottom.dtype)
            else:
                S = g[:, 0, None, None] * S
                u = g[:, 1, None] * (vt - torch.einsum("hcd,hd->hc", S, kt))
                S = S + u[:, :, None] * kt[:, None, :]
                y[t] = torch.einsum("hcd,hd->hc", S, qt).to(y.dtype)
        kept.copy_(S.to(kept.dtype))


def head_norm_gate(y, bottom, weight, gate, gate_col, activation, eps, out):
    n, heads, vdim = y.shape
    v = y.double()
    if bottom is not None:
        v = v / bottom.double()[:, :, None]
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.double().view(heads, vdim) if weight.numel() == heads * vdim else weight.double().view(1, vdim)
    z = gate[:, gate_col:gate_col + heads * vdim].double().view(n, heads, vdim)
    act = torch.sigmoid(z) if activation == "sigmoid" else z * torch.sigmoid(z)
    out.copy_((v * w * act).reshape(n, heads * vdim).to(out.dtype))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_recurrence_scan(u, pre, gate_bias, rate, proj, y_col, y_bias, states, state_offset, state_slots, query_start,
                          max_query_len, out):
    width = u.shape[1]
    r = torch.sigmoid(pre[0].double() + gate_bias[0].double())
    i = torch.sigmoid(pre[1].double() + gate_bias[1].double())
    log_a = rate.double() * r
    a, b = torch.exp(log_a), torch.sqrt(-torch.expm1(2.0 * log_a))
    z = proj[:, y_col:y_col + width].double()
    if y_bias is not None:
        z = z + y_bias.double()
    for req in range(state_slots.numel()):
        lo, hi = int(query_start[req]), int(query_start[req + 1])
        if hi == lo:
            continue
        kept = states[int(state_slots[req]), state_offset:state_offset + width]
        S = kept.double()
        for t in range(lo, hi):
            S = a[t] * S + b[t] * i[t] * u[t].double()
            out[t] = (S * gelu_tanh(z[t])).to(out.dtype)
        kept.copy_(S.to(kept.dtype))


# --------------------------------------------------------------------------- one token back, pairs of outputs, two score maps


def softplus(x):
    return torch.clamp(x, min=0.0) + torch.log1p(torch.exp(-x.abs()))


def low_rank_expand(mid, col, weight_t, out, a_log=None, bias=None, per_head=0):
    rank = weight_t.shape[0]
    value = mid[:, col:col + rank].double() @ weight_t.double()
    if a_log is not None:
        value = torch.exp(-torch.exp(a_log.double()).repeat_interleave(per_head) * softplus(value + bias.double()))
    out.copy_(value.to(out.dtype))


def channel_decays(logits, col, a_log, dt_bias, per_head, out):
    rows = out.shape[1]
    value = logits[:, col:col + rows].double()
    out.copy_(torch.exp(-torch.exp(a_log.double()).repeat_interleave(per_head) * softplus(value + dt_bias.double())).to(out.dtype))


def normed_sum(a, a_weight, a_scale, b, b_weight, b_scale, eps, out):
    def normed(x, w):
        x = x.double()
        return w.double() * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))
    out.copy_((a_scale * normed(a, a_weight) + b_scale * normed(b, b_weight)).to(out.dtype))


def sigmoid_gate_mul(x, gate, gate_col, out):
    width = x.shape[1]
    out.copy_((x.double() * torch.sigmoid(gate[:, gate_col:gate_col + width].double())).to(out.dtype))


def differential_combine(a, lam, eps, out_scale, gate, gate_col, out):
    n, both, dv = a.shape
    heads = both // 2
    o = a[:, :heads].double() - lam * a[:, heads:].double()
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * out_scale
    if gate is not None:
        o = o * torch.sigmoid(gate[:, gate_col:gate_col + heads * dv].double()).view(n, heads, dv)
    out.copy_(o.to(out.dtype))


def token_shift(x, shift, states, state_offset, state_slots, query_start, request_of_token, out):
    hidden = x.shape[1]
    for r in range(state_slots.numel()):
        lo, hi = int(query_start[r]), int(query_start[r + 1])
        if hi == lo:
            continue
        kept = states[int(state_slots[r]), state_offset:state_offset + hidden]
        before = torch.cat([kept.double()[None, :], x[lo:hi - 1].double()], dim=0)
        now = x[lo:hi].double()
        kept.copy_(x[hi - 1].to(kept.dtype))
        out[lo:hi] = (now + (before - now) * shift.double()).to(out.dtype)


def pair_embedding(tokens, table, buckets, mul_prev, mul_cur, states, state_slots, query_start, request_of_token, residual):
    for r in range(state_slots.numel()):
        lo, hi = int(query_start[r]), int(query_start[r + 1])
        if hi == lo:
            continue
        before = int(states[int(state_slots[r]), 0]) - 1
        for t in range(lo, hi):
            token = int(tokens[t])
            row = buckets if before < 0 else (before * mul_prev + token * mul_cur) % buckets
            residual[t] += table[row].to(residual.dtype)
            before = token
        states[int(state_slots[r]), 0] = before + 1


def install(monkeypatch) -> None:
    """Puts the functions above in place of the kernel bindings (CPU tests of host logic only)."""
    import miniserve_b200  # noqa: F401
    from miniserve_b200 import kernels

    for name in ("embedding", "add_rmsnorm", "rmsnorm", "rope_table", "qk_norm_rope_append", "silu_mul",
                 "paged_attention", "linear", "gated_linear", "gated_up", "sample", "scale_softcap", "latent_prepare",
                 "latent_attention", "head_gate", "linear_batched", "router_topk", "expert_route", "expert_linear",
                 "expert_combine", "relu_square", "clamped_glu", "postnorm_add_rmsnorm", "qkv_prepare", "causal_conv_silu",
                 "selective_scan", "gated_group_norm", "causal_conv", "add_bias", "scaled_sum", "small_linear_f32",
                 "unit_norm_heads", "exponential_gates", "decay_gates", "matrix_scan", "head_norm_gate", "gated_recurrence_scan",
                 "low_rank_expand", "channel_decays", "normed_sum", "sigmoid_gate_mul", "differential_combine", "token_shift",
                 "pair_embedding"):
        monkeypatch.setattr(kernels, name, globals()[name])
    monkeypatch.setattr(kernels, "attention_kernels", lambda *sizes: {"decode": "plain", "prompt": "plain"})
    monkeypatch.setattr(kernels, "latent_attention_kernels", lambda *sizes: {"decode": "plain", "prompt": "plain"})
    # norms folded into the products around them: offered for steps of up to eight rows and for steps of many
    # (here: 24 and more), as on the device, with the two layouts of the sums of squares
    monkeypatch.setattr(kernels, "linear_residual", linear_residual)
    monkeypatch.setattr(kernels, "residual_partials_shape", lambda rows, n, k: (FOLD_BLOCKS, 8 if rows <= 8 else rows))
    monkeypatch.setattr(kernels, "fold_supported", lambda rows, dtype, producer, consumer, gated=False: 0 < rows <= 8 or rows >= 24)
    monkeypatch.setattr(kernels, "qkv_in_product_supported", lambda *sizes: False)
    # products that add into the residual stream themselves: offered for steps of 12 to 23 rows
    monkeypatch.setattr(kernels, "linear_add", linear_add)
    monkeypatch.setattr(kernels, "add_in_product_supported", lambda rows, dtype, weight: 12 <= rows < 24)
