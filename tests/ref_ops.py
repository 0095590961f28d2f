"""Plain PyTorch restatements of the engine's operations, one per kernel, with the
same signatures as ``qwen_engine_b200.ops``.

Two uses: the ``-m gpu`` tests compare each CUDA kernel alone with its function
here; and the CPU tests put these functions in the place of the kernels
(``install``), so that the host side of the engine (cache manager, step function,
scheduler, replay) can be checked against the plain model without a GPU.  They
are test code: the product has no CPU path.

Arithmetic is float32 (inputs are converted up, results rounded to the output's
dtype), as in the kernels.
"""
from __future__ import annotations

import torch

ATTN_TILE_Q = 16


def prepare_matrix(w):
    return w.contiguous()


def embedding(token_ids, table, out, ssq=None, scale=1.0, accumulate=False):
    from qwen_engine_b200.ops import ResidualStream
    if isinstance(out, ResidualStream):
        if not accumulate:
            out.has_delta = False
        out.n_ssq = 0
        out = out.resid
    rows = table[token_ids.long()].to(torch.float32) * scale
    if accumulate:
        out.add_(rows)
    else:
        out.copy_(rows)


def _rms(x, weight, eps):
    x = x.to(torch.float32)
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def add_rmsnorm(resid, delta, weight, eps, out):
    if delta is not None:
        resid.add_(delta.to(torch.float32))
    out.copy_(_rms(resid, weight, eps).to(out.dtype))


def add_rmsnorm_rows(resid, delta, rows, weight, eps, out):
    n = out.shape[0]
    idx = rows[:n].long()
    x = resid[idx]
    if delta is not None:
        x = x + delta[idx].to(torch.float32)
    out.copy_(_rms(x, weight, eps).to(out.dtype))


def linear(x, w, out):
    from qwen_engine_b200.ops import NormedInput, ResidualSink
    if isinstance(x, NormedInput):
        x = x.materialize()
    if isinstance(out, ResidualSink):
        out = out.as_delta()
    out.copy_((x.to(torch.float32) @ w.to(torch.float32).t()).to(out.dtype))


def _rotate(x, positions, inv_freq, rotary_dim, magnitude=1.0):
    """x [T, heads, D] float32 -> rotated copy (half-split pairs over the first rotary_dim dims)."""
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    c, s = torch.cos(ang)[:, None, :] * magnitude, torch.sin(ang)[:, None, :] * magnitude
    half = rotary_dim // 2
    x1, x2 = x[..., :half], x[..., half:rotary_dim]
    return torch.cat([c * x1 - s * x2, s * x1 + c * x2, x[..., rotary_dim:]], dim=-1)


def place_tokens(token_ids, rows, src, src_index):
    token_ids[rows.long()] = src[src_index.long()]


def swiglu_fused_applies(*args, **kwargs):
    return False


def rope_table(positions, inv_freq, out):
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    out[..., 0], out[..., 1] = torch.cos(ang), torch.sin(ang)


def qk_norm_rope_kv_write(qkv, positions, q_norm_w, k_norm_w, eps, inv_freq, rotary_dim, kv_pages,
                          slot_mapping, num_heads, num_kv_heads, head_dim, write_kv=True, cos_sin=None, norm_dim=None,
                          magnitude=1.0, value_mix=None):
    T = qkv.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    q = qkv[:, :Hq * D].reshape(T, Hq, D).to(torch.float32)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D).to(torch.float32)
    v = qkv[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
    n = norm_dim or D          # the mean runs over the head's own channels; the rest is zero padding
    if q_norm_w is not None:
        q = q * torch.rsqrt((q * q).sum(dim=-1, keepdim=True) / n + eps) * q_norm_w
    if k_norm_w is not None:
        k = k * torch.rsqrt((k * k).sum(dim=-1, keepdim=True) / n + eps) * k_norm_w
    if inv_freq is not None:
        q = _rotate(q, positions, inv_freq, rotary_dim, magnitude)
        k = _rotate(k, positions, inv_freq, rotary_dim, magnitude)
    if value_mix is not None:
        dv = value_mix[1].shape[1] // Hkv                  # the heads' own channels (layers pad differently)
        if value_mix[0] == "keep":
            value_mix[1].copy_(v[:, :, :dv].reshape(T, Hkv * dv))
        else:
            lam = float(value_mix[2])
            first = torch.zeros(T, Hkv, D, dtype=torch.float32)
            first[:, :, :dv] = value_mix[1].reshape(T, Hkv, dv).to(torch.float32)
            v = ((1.0 - lam) * v.to(torch.float32) + lam * first).to(qkv.dtype)
    qkv[:, :Hq * D] = q.reshape(T, Hq * D).to(qkv.dtype)
    qkv[:, Hq * D:(Hq + Hkv) * D] = k.reshape(T, Hkv * D).to(qkv.dtype)
    if write_kv:
        P = kv_pages.shape[3]
        slots = slot_mapping.long()
        page, off = slots // P, slots % P
        kv_pages[page, 0, :, off, :] = k.to(kv_pages.dtype)
        kv_pages[page, 1, :, off, :] = v.to(kv_pages.dtype)


def rope_neox(q, k, positions, inv_freq, rotary_dim):
    q.copy_(_rotate(q.to(torch.float32), positions, inv_freq, rotary_dim).to(q.dtype))
    k.copy_(_rotate(k.to(torch.float32), positions, inv_freq, rotary_dim).to(k.dtype))


def plan_attention(q_lens, ctx_lens, page_size, geometries=(), dtype=None, uniform_splits=None):
    tiles = []
    for r, n in enumerate(q_lens):
        for q0 in range(0, n, ATTN_TILE_Q):
            tiles += [r, q0]
    return {"tiles": tiles}


def paged_attention(qkv, kv_pages, block_tables, ctx, out, scale, window, num_heads, num_kv_heads, head_dim, next_pages=None,
                    slopes=None, softcap=0.0, sinks=None, value_shift=0, value_shifts=1):
    """For each request: gather its keys and values from the pages by its block table, then
    softmax(scale q k^T + mask) v with key j allowed for the query at position i iff
    j <= i and (window == 0 or j > i - window)."""
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    if value_shifts > 1:                  # out [S, T, Hq D]: one output per shift of the values' kv head
        for s in range(value_shifts):
            paged_attention(qkv, kv_pages, block_tables, ctx, out[s], scale, window, Hq, Hkv, D, next_pages, slopes, softcap, sinks, s)
        return
    P = kv_pages.shape[3]
    cu = ctx.cu_q.tolist()
    ctx_lens = ctx.ctx_lens.tolist()
    group = Hq // Hkv
    for r in range(len(ctx_lens)):
        a, b = cu[r], cu[r + 1]
        n, c = b - a, ctx_lens[r]
        if n == 0:
            continue
        total = c + n
        q = qkv[a:b, :Hq * D].reshape(n, Hq, D).to(torch.float32)
        kpos = torch.arange(total)
        qpos = c + torch.arange(n)
        allowed = kpos[None, :] <= qpos[:, None]
        if window and window > 0:
            allowed &= kpos[None, :] > qpos[:, None] - window
        needed = allowed.any(dim=0)
        table = block_tables[r].long()
        pages = table[kpos // P]
        assert bool((pages[needed] >= 0).all()), "attention needs a key whose page was given back"
        pages = pages.clamp(min=0)
        k = kv_pages[pages, 0, :, kpos % P, :].to(torch.float32)      # [total, Hkv, D]
        # (a cache of one plane: the values are the keys' channels)
        v = kv_pages[pages, kv_pages.shape[1] - 1, :, kpos % P, :].to(torch.float32)
        k = torch.where(needed[:, None, None], k, torch.zeros_like(k))
        v = torch.where(needed[:, None, None], v, torch.zeros_like(v))
        for h in range(Hq):
            s = (q[:, h, :] @ k[:, h // group, :].t()) * scale
            if slopes is not None:
                s = s - float(slopes[h]) * (qpos[:, None] - kpos[None, :]).to(torch.float32)
            if softcap and softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            s = s.masked_fill(~allowed, float("-inf"))
            if sinks is not None:
                p = torch.softmax(torch.cat([s, sinks[h].reshape(1, 1).expand(n, 1)], dim=-1), dim=-1)[:, :-1]
            else:
                p = torch.softmax(s, dim=-1)
            out[a:b, h * D:(h + 1) * D] = (p @ v[:, (h // group + value_shift) % Hkv, :]).to(out.dtype)


def silu_mul(gate_up, out):
    I = out.shape[1]
    g = gate_up[:, :I].to(torch.float32)
    u = gate_up[:, I:].to(torch.float32)
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def act_mul(gate_up, out, activation="silu"):
    import math
    I = out.shape[1]
    g = gate_up[:, :I].to(torch.float32)
    u = gate_up[:, I:].to(torch.float32)
    if activation == "silu":
        a = g / (1.0 + torch.exp(-g))
    elif activation == "gelu_tanh":
        a = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
    elif isinstance(activation, (tuple, list)) and activation[0] == "swish_limit":
        lim = float(activation[1])
        g = torch.clamp(g, max=lim)
        u = torch.clamp(u, -lim, lim) + 1.0
        a = g * torch.sigmoid(1.702 * g)
    else:
        raise ValueError(activation)
    out.copy_((a * u).to(out.dtype))


def channel_decay(a, w, bias, tau, out, log_rate=None):
    z = a.to(torch.float32) @ w.to(torch.float32).t()
    if bias is not None:
        z = z + bias
    if log_rate is not None:
        rate = torch.exp(log_rate).repeat_interleave(z.shape[1] // log_rate.numel())
        out.copy_(torch.exp(-rate * torch.nn.functional.softplus(z)))
    else:
        out.copy_(torch.exp(torch.nn.functional.logsigmoid(z) / tau))


def linear_attention_scan(q, k, v, alpha, state, ctx, out, q_scale, num_heads, key_dim, value_dim, write_state=True, decay=None,
                          head_decay=None):
    """state [slots, H, dv, dk]; per request and head, token by token."""
    H, dk, dv = num_heads, key_dim, value_dim
    if head_decay is not None:
        alpha = head_decay.to(torch.float32).repeat_interleave(dk)[None, :].expand(q.shape[0], H * dk)
    elif alpha is None:
        a, w, bias, tau = decay
        alpha = torch.empty(q.shape[0], H * dk, dtype=torch.float32)
        channel_decay(a, w, bias, tau, alpha)
    cu, ctx_lens, slots = ctx.cu_q.tolist(), ctx.ctx_lens.tolist(), ctx.slot_ids.tolist()
    for r in range(len(ctx_lens)):
        a, b = cu[r], cu[r + 1]
        if b <= a:
            continue
        S = state[slots[r]].clone() if ctx_lens[r] > 0 else torch.zeros_like(state[slots[r]])     # [H, dv, dk]
        for t in range(a, b):
            qt = q[t].to(torch.float32).reshape(H, dk) * q_scale
            kt = k[t].to(torch.float32).reshape(H, dk)
            vt = v[t].to(torch.float32).reshape(H, dv)
            at = alpha[t].reshape(H, dk)
            S = S * at[:, None, :] + vt[:, :, None] * kt[:, None, :]
            out[t] = (S * qt[:, None, :]).sum(dim=-1).reshape(H * dv)
        if write_state:
            state[slots[r]] = S


def head_norm_gate(x, gate, weight, eps, out, num_heads, head_dim, gate_kind="silu", scale=1.0):
    T = x.shape[0]
    y = x.to(torch.float32).reshape(T, num_heads, head_dim)
    if weight is not None:
        y = y * torch.rsqrt((y * y).mean(dim=-1, keepdim=True) + eps) * weight
    if gate is not None:
        g = gate.to(torch.float32).reshape(T, num_heads, head_dim)
        y = y * (g / (1.0 + torch.exp(-g)) if gate_kind == "silu" else torch.sigmoid(g))
    out.copy_((y * scale).reshape(T, num_heads * head_dim).to(out.dtype))


def latent_prepare(down, q, norm_w, eps, positions, inv_freq, rot_dims, cache, slot_mapping, qlat, num_heads, plain_dim,
                   latent_dim, rot_dim, write_kv=True):
    T, H, dn, R, Dr = q.shape[0], num_heads, plain_dim, latent_dim, rot_dim
    D, P = R + Dr, cache.shape[3]
    half = rot_dims // 2
    ang = positions.to(torch.float32)[:, None] * inv_freq[:half][None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)

    def turn(x):                       # [T, ..., Dr]
        x = x.to(torch.float32).clone()
        shape = [T] + [1] * (x.dim() - 2) + [half]
        u, v = x[..., :half].clone(), x[..., half:rot_dims].clone()
        x[..., :half] = u * cos.reshape(shape) - v * sin.reshape(shape)
        x[..., half:rot_dims] = v * cos.reshape(shape) + u * sin.reshape(shape)
        return x
    if write_kv:
        row = torch.cat([_rms(down[:, :R], norm_w, eps), turn(down[:, R:])], dim=1).to(cache.dtype)
        slots = slot_mapping.long()
        cache[slots // P, 0, 0, slots % P] = row
    out = qlat.view(T, H, D)
    out[:, :, R:] = turn(q.reshape(T, H, dn + Dr)[:, :, dn:]).to(qlat.dtype)


def head_linear(x, w, out, x_head_stride, out_head_stride):
    H, N, K = w.shape
    for h in range(H):
        xs = x[:, h * x_head_stride:h * x_head_stride + K].to(torch.float32)
        out[:, h * out_head_stride:h * out_head_stride + N] = (xs @ w[h].to(torch.float32).t()).to(out.dtype)


def short_conv(x, w, state, ctx, out, write_state=True, silu=True):
    taps = w.shape[1]
    hist = taps - 1
    cu, ctx_lens, slots = ctx.cu_q.tolist(), ctx.ctx_lens.tolist(), ctx.slot_ids.tolist()
    for r in range(len(ctx_lens)):
        a, b = cu[r], cu[r + 1]
        if b <= a:
            continue
        old = state[slots[r]].clone() if ctx_lens[r] > 0 else torch.zeros_like(state[slots[r]])     # [hist, C]
        seq = torch.cat([old, x[a:b].to(torch.float32)], dim=0)
        y = torch.zeros(b - a, x.shape[1], dtype=torch.float32)
        for j in range(taps):
            y = y + seq[j:j + b - a] * w[:, j][None, :]
        out[a:b] = y * torch.sigmoid(y) if silu else y
        if write_state and hist > 0:
            state[slots[r]] = seq[-hist:]


def unit_norm(x, num_heads, head_dim, eps, scale=1.0):
    T = x.shape[0]
    y = x.reshape(T, num_heads, head_dim)
    y = y * torch.rsqrt((y * y).sum(dim=-1, keepdim=True) + eps) * scale
    x.copy_(y.reshape(T, num_heads * head_dim))


def delta_rule_scan(q, k, v, g, beta, state, ctx, out, num_heads, num_key_heads, key_dim, value_dim, write_state=True,
                    head_decay=None):
    H, G, dk, dv = num_heads, num_key_heads, key_dim, value_dim
    rep = H // G
    cu, ctx_lens, slots = ctx.cu_q.tolist(), ctx.ctx_lens.tolist(), ctx.slot_ids.tolist()
    gh = None
    if head_decay is not None:
        a, rate, bias = head_decay
        gh = torch.exp(-torch.exp(rate) * torch.nn.functional.softplus(a.to(torch.float32) + bias))      # [T, H]
    for r in range(len(ctx_lens)):
        a, b = cu[r], cu[r + 1]
        if b <= a:
            continue
        S = state[slots[r]].clone() if ctx_lens[r] > 0 else torch.zeros_like(state[slots[r]])     # [H, dv, dk]
        for t in range(a, b):
            qt = q[t].reshape(G, dk).repeat_interleave(rep, dim=0)
            kt = k[t].reshape(G, dk).repeat_interleave(rep, dim=0)
            vt = v[t].reshape(H, dv)
            if g is not None:
                S = S * g[t].reshape(H, dk)[:, None, :]
            if gh is not None:
                S = S * gh[t][:, None, None]
            bt = torch.sigmoid(beta[t].to(torch.float32))
            u = bt[:, None] * (vt - (S * kt[:, None, :]).sum(dim=-1))
            S = S + u[:, :, None] * kt[:, None, :]
            out[t] = (S * qt[:, None, :]).sum(dim=-1).reshape(H * dv)
        if write_state:
            state[slots[r]] = S


def moe_route(x, w, bias, top_idx, top_w, scoring="softmax_chosen", correction=None):
    z = x.to(torch.float32) @ w.t()
    if bias is not None:
        z = z + bias
    if scoring == "softmax_all":
        s = torch.softmax(z, dim=-1)
        idx = torch.topk(s if correction is None else s + correction, top_idx.shape[1], dim=-1).indices
        top_idx.copy_(idx.to(torch.int32))
        top_w.copy_(torch.gather(s, 1, idx))
        return
    val, idx = torch.topk(z, top_idx.shape[1], dim=-1)
    top_idx.copy_(idx.to(torch.int32))
    top_w.copy_(torch.sigmoid(val) if scoring == "sigmoid" else torch.softmax(val, dim=-1))


def moe_experts(x, top_idx, top_w, w_gate_up, w_down, out, activation, alloc, num_identity=0, weight_inputs=False):
    T = x.shape[0]
    E = w_gate_up.shape[0]
    I = w_gate_up.shape[1] // 2
    acc = torch.zeros(T, w_down.shape[1], dtype=torch.float32)
    for t in range(T):
        for j in range(top_idx.shape[1]):
            e = int(top_idx[t, j])
            if e >= E:                       # an expert that hands its input on
                assert e < E + num_identity
                acc[t] += float(top_w[t, j]) * x[t].to(torch.float32)
                continue
            gu = x[t:t + 1].to(torch.float32) @ w_gate_up[e].to(torch.float32).t()
            if weight_inputs:                # the weight meets the first products' sums ahead of the activation
                gu = gu * float(top_w[t, j])
            gu = gu.to(x.dtype)
            act = torch.empty(1, I, dtype=x.dtype)
            act_mul(gu, act, activation)
            acc[t] += (1.0 if weight_inputs else float(top_w[t, j])) * (act.to(torch.float32) @ w_down[e].to(torch.float32).t())[0]
    out.copy_(acc.to(out.dtype))


def qk_bias_norm_kv_write(proj, positions, q_bias, k_bias, eps, q_temp, kv_pages, slot_mapping, num_heads, num_kv_heads,
                          head_dim, write_kv=True):
    T = proj.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    q = proj[:, :Hq * D].to(torch.float32)
    k = proj[:, Hq * D:(Hq + Hkv) * D].to(torch.float32)
    if q_bias is not None:
        q = (q + q_bias).to(proj.dtype).to(torch.float32)
    if k_bias is not None:
        k = (k + k_bias).to(proj.dtype).to(torch.float32)
    v = k.reshape(T, Hkv, D)
    q, k = q.reshape(T, Hq, D), k.reshape(T, Hkv, D)
    q = q * torch.rsqrt((q * q).mean(dim=-1, keepdim=True) + eps)
    k = k * torch.rsqrt((k * k).mean(dim=-1, keepdim=True) + eps)
    if q_temp is not None:
        coef, every = q_temp
        steps = torch.div(positions.long() + 1, every, rounding_mode="floor").to(torch.float32)
        q = q * (1.0 + coef * torch.log(steps + 1.0))[:, None, None]
    proj[:, :Hq * D] = q.reshape(T, Hq * D).to(proj.dtype)
    proj[:, Hq * D:(Hq + Hkv) * D] = k.reshape(T, Hkv * D).to(proj.dtype)
    if write_kv:
        P = kv_pages.shape[3]
        slots = slot_mapping.long()
        page, off = slots // P, slots % P
        kv_pages[page, 0, :, off, :] = k.to(kv_pages.dtype)
        kv_pages[page, 1, :, off, :] = v.to(kv_pages.dtype)


def stream_conv(resid, w, state, ctx, out_plain, out_conv, write_state=True):
    taps = w.shape[1]
    hist = taps - 1
    cu, ctx_lens, slots = ctx.cu_q.tolist(), ctx.ctx_lens.tolist(), ctx.slot_ids.tolist()
    if out_plain is not None:
        out_plain.copy_(resid.to(out_plain.dtype))
    for r in range(len(ctx_lens)):
        a, b = cu[r], cu[r + 1]
        if b <= a:
            continue
        if hist > 0:
            old = state[slots[r]].clone() if ctx_lens[r] > 0 else torch.zeros_like(state[slots[r]])     # [hist, W]
        else:
            old = resid.new_zeros((0, resid.shape[1]))
        seq = torch.cat([old, resid[a:b]], dim=0)
        y = torch.zeros(b - a, resid.shape[1], dtype=torch.float32)
        for j in range(taps):
            y = y + seq[j:j + b - a] * w[:, j][None, :]
        out_conv[a:b] = (resid[a:b] + y).to(out_conv.dtype)
        if write_state and hist > 0:
            state[slots[r]] = seq[-hist:]


def gated_norm_add(src, branch, gate, gate_bias, weight, eps, dst, dst_cast=None, depth_mix=None):
    v = branch.to(torch.float32)
    if gate is not None:
        z = gate.to(torch.float32)
        if gate_bias is not None:
            z = z + gate_bias
        v = v * torch.sigmoid(z)
    res = src + _rms(v, weight, eps)
    dst.copy_(res)
    if dst_cast is not None:
        dst_cast.copy_(res.to(dst_cast.dtype))
    if depth_mix is not None:
        history, weights, count, mixed = depth_mix
        assert dst.data_ptr() == history[count - 1].data_ptr()
        globals()["depth_mix"](history, weights, count, mixed)


def _group_rms(x, weight, eps, groups):
    x = x.to(torch.float32)
    n, W = x.shape
    parts = x.reshape(n, groups, W // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(n, W) * weight


def group_rmsnorm(x, rows, weight, eps, groups, out):
    src = x if rows is None else x[rows[:out.shape[0]].long()]
    out.copy_(_group_rms(src, weight, eps, groups).to(out.dtype))


def group_norm_add(src, branch, weight, eps, groups, dst, next_weight=None, next_out=None):
    res = src + _group_rms(branch, weight, eps, groups)
    dst.copy_(res)
    if next_out is not None:
        next_out.copy_(_group_rms(res, next_weight, eps, groups).to(next_out.dtype))


def head_mix_gate(partial, mix, gate, out, num_heads, num_kv_heads, head_dim):
    S, T = partial.shape[0], partial.shape[1]
    H, Hkv, D = num_heads, num_kv_heads, head_dim
    G = H // Hkv
    p = partial.to(torch.float32).reshape(S, T, H, D)
    if mix is None:
        res = p[0].clone()
    else:
        res = torch.zeros(T, H, D, dtype=torch.float32)
        for h in range(H):
            for g in range(H):
                res[:, h] += mix[h, g] * p[(h // G - g // G) % Hkv, :, g]
    if gate is not None:
        res = res * torch.sigmoid(gate.to(torch.float32))[:, :, None]
    out.copy_(res.reshape(T, H * D).to(out.dtype))


def token_side_gate(gate, table, token_ids, out):
    g = gate.to(torch.float32)
    a = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    out.copy_((a * table[token_ids.long()].to(torch.float32)).to(out.dtype))


def depth_mix(history, weights, count, out):
    acc = torch.zeros_like(out)
    for j in range(count):
        acc = acc + weights[j] * history[j]
    out.copy_(acc)


def scaled_add(acc, x, scale, first=False):
    base = torch.zeros_like(acc, dtype=torch.float32) if first else acc.to(torch.float32)
    acc.copy_((base + scale * x.to(torch.float32)).to(acc.dtype))


def linear_silu_mul(gate_up, w, out, scratch):
    from qwen_engine_b200.ops import ResidualSink
    if isinstance(out, ResidualSink):
        out = out.as_delta()
    act = scratch((gate_up.shape[0], gate_up.shape[1] // 2), gate_up.dtype)
    silu_mul(gate_up, act)
    linear(act, w, out)


def argmax(logits, out):
    out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))


def sample_row(row, temperature, top_k, u):
    """One row of the sampling rule: temperature 0 -> argmax (lowest index on a tie); else keep the
    logits >= the top_k-th largest (all when top_k is 0 or >= V), p = exp((logit - max) / temperature)
    in float32, and take the first index whose running sum (float64, index order) exceeds u * total."""
    row = row.to(torch.float32)
    best = int(torch.argmax(row))
    if not temperature > 0:
        return best
    V = row.numel()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.topk(row, top_k).values[-1]
        keep = row >= kth
    p = torch.exp((row - row.max()) / torch.tensor(temperature, dtype=torch.float32))
    p = torch.where(keep, p, torch.zeros_like(p)).to(torch.float64)
    cum = torch.cumsum(p, dim=0)
    target = float(torch.tensor(u, dtype=torch.float32)) * float(cum[-1])
    hit = torch.nonzero(cum > target)
    return int(hit[0]) if hit.numel() else best


def sample(logits, temperature, top_k, uniform, out):
    for n in range(logits.shape[0]):
        out[n] = sample_row(logits[n].cpu(), float(temperature[n]), int(top_k[n]), float(uniform[n]))


def swiglu_small_applies(M, I, K, dtype):
    return False                 # the host-side tests take the route of separate operations


def qkv_rope_small_applies(M, N, K, dtype, head_dim, rotary_dim):
    return False                 # the host-side tests take the route of separate operations


def copy_pages(cache, pairs):
    """cache [slots, pages, ...]: page pairs[2 i] of every slot is copied to page pairs[2 i + 1]."""
    flat = pairs.tolist()
    for src, dst in zip(flat[0::2], flat[1::2]):
        cache[:, dst] = cache[:, src].clone()


_NAMES = ["group_rmsnorm", "group_norm_add", "head_mix_gate", "qk_bias_norm_kv_write", "stream_conv", "gated_norm_add", "token_side_gate", "depth_mix", "latent_prepare", "head_linear", "short_conv", "unit_norm", "delta_rule_scan", "moe_route", "moe_experts",
          "act_mul", "channel_decay", "linear_attention_scan", "head_norm_gate", "scaled_add", "copy_pages", "swiglu_small_applies", "qkv_rope_small_applies", "prepare_matrix", "embedding", "add_rmsnorm", "add_rmsnorm_rows", "linear",
          "qk_norm_rope_kv_write", "rope_neox", "rope_table", "place_tokens", "swiglu_fused_applies", "plan_attention", "paged_attention", "silu_mul", "linear_silu_mul",
          "argmax", "sample"]


def install(monkeypatch) -> None:
    """Put these functions in the place of the CUDA fronts for the length of a test."""
    import qwen_engine_b200.ops as ops
    g = globals()
    for name in _NAMES:
        monkeypatch.setattr(ops, name, g[name])
