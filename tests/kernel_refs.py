"""Plain references of the package's kernels, one per function of
``litinfer_b200.kernels``, with the same signatures, in float32 torch on
whatever device the tensors are on.

Two uses: the GPU tests compare each kernel alone with its reference here;
the CPU tests patch these in place of the kernels, so that the cache manager,
the step function and the scheduler can be checked against the plain model
without a GPU.  They are test code: nothing in the package imports them.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def _store(out, value):
    out.copy_(value.to(out.dtype))


def embedding(table, ids, out32):
    _store(out32, table[ids.long()].float())


def _rms(x, weight, eps):
    x = x.float()
    r = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (weight * x) * r


def rmsnorm(x32, weight, eps, out):
    _store(out, _rms(x32, weight, eps))


def add_rmsnorm(x32, delta, weight, eps, out):
    x32.add_(delta.float())
    _store(out, _rms(x32, weight, eps))


def gather_rmsnorm(x32, rows, weight, eps, out):
    _store(out, _rms(x32[rows.long()], weight, eps))


def residual_add(x32, delta):
    x32.add_(delta.float())


def linear(a, weight, bias, out, epilogue=None, row_scale=None, epilogue_params=None):
    y = a.float() @ weight.float().t()
    if row_scale is not None:
        y = y * _factor(row_scale)
    if bias is not None:
        y = y + bias
    if epilogue == "swiglu":
        # columns come as 8 gate, 8 up, 8 gate, 8 up, ...
        M, N = y.shape
        y = y.view(M, N // 16, 2, 8)
        g, u = y[:, :, 0, :], y[:, :, 1, :]
        y = (u * (g / (1.0 + torch.exp(-g)))).reshape(M, N // 2)
    elif epilogue == "glu_clamped":
        M, N = y.shape
        limit, alpha = (float(v) for v in epilogue_params.tolist())
        y = y.view(M, N // 16, 2, 8)
        g, u = torch.clamp(y[:, :, 0, :], max=limit), torch.clamp(y[:, :, 1, :], min=-limit, max=limit)
        y = (g * torch.sigmoid(alpha * g) * (u + 1.0)).reshape(M, N // 2)
    _store(out, y)


def _factor(row_scale):
    ssq, width, eps = row_scale
    return (1.0 / torch.sqrt(ssq.sum(1) / width + eps)).unsqueeze(1)


def linear_scaled_accepts(a, weight, out):
    return True


def linear_add_scaled_parts(a, weight, x32, hprime):
    return 3


def linear_add_scaled(a, weight, bias, x32, norm_weight, hprime, ssq):
    y = a.float() @ weight.float().t()
    if bias is not None:
        y = y + bias
    x32.add_(y)
    _store(hprime, norm_weight * x32)
    # any split of the columns into parts gives the same sums; here: everything in part 0
    ssq.zero_()
    ssq[:, 0] = (x32 * x32).sum(-1)


def apply_row_scale(hprime, ssq, width, eps, out):
    _store(out, hprime.float() * _factor((ssq, width, eps)))


def interleave_gate_up(gate, up):
    I, Kd = gate.shape
    return torch.stack((gate.view(I // 8, 8, Kd), up.view(I // 8, 8, Kd)), dim=1).reshape(2 * I, Kd).contiguous()


def rope_kv_write(qkv, positions, denominators, rotary_dim, slot_mapping, k_cache, v_cache,
                  num_heads, num_kv_heads, head_dim, write=True):
    T = qkv.shape[0]
    q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
    half = rotary_dim // 2
    if rotary_dim:
        phi = positions.float()[:, None] / denominators[None, :]
        cos, sin = torch.cos(phi)[:, None, :], torch.sin(phi)[:, None, :]

    def rot(x):
        x = x.float().clone()
        if not rotary_dim:
            return x
        a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
        x[..., :half] = a * cos - b * sin
        x[..., half:rotary_dim] = b * cos + a * sin
        return x

    q = rot(qkv[:, :q_dim].reshape(T, num_heads, head_dim))
    qkv[:, :q_dim] = q.reshape(T, q_dim).to(qkv.dtype)
    if not write:
        return
    k = rot(qkv[:, q_dim:q_dim + kv_dim].reshape(T, num_kv_heads, head_dim)).to(qkv.dtype)
    v = qkv[:, q_dim + kv_dim:].reshape(T, num_kv_heads, head_dim)
    page_size = k_cache.shape[2]
    page = (slot_mapping // page_size).long()
    off = (slot_mapping % page_size).long()
    k_cache[page, :, off] = k
    v_cache[page, :, :, off] = v         # values are cached transposed: [page, kv_head, head_dim, slot]


def linear_rope_kv(a, weight, bias, qkv, positions, denominators, rotary_dim, slot_mapping, k_cache, v_cache,
                   num_heads, num_kv_heads, head_dim, write=True, fused=True, row_scale=None, cos_sin=None):
    linear(a, weight, bias, qkv, row_scale=row_scale)
    rope_kv_write(qkv, positions, denominators, rotary_dim, slot_mapping, k_cache, v_cache, num_heads, num_kv_heads, head_dim, write)


def rope_table(positions, denominators, out):
    phi = positions.float().unsqueeze(1) / denominators.unsqueeze(0)
    out[..., 0] = torch.cos(phi)
    out[..., 1] = torch.sin(phi)


def paged_attention(qkv, out, k_cache, v_cache, block_table, q_start, ctx_lens, seq_of_token, positions,
                    num_heads, num_kv_heads, head_dim, scale, window, max_q_len, max_ctx_len, implementation=None, old_lens=None, singles=0,
                    units=None, unit_slots=(0, 0), softcap=0.0, slopes=None, gate=None, keep_first=0, sinks=None):
    # old_lens only tells a kernel which keys it may read early, singles which kernel takes which sequence, units how a
    # kernel shares its work out; the result does not depend on them
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    q = qkv[:, :num_heads * head_dim].reshape(T, num_heads, head_dim).float()
    res = torch.zeros(T, num_heads, head_dim, dtype=torch.float32, device=qkv.device)
    seqs = seq_of_token.tolist()
    poss = positions.tolist()
    for t in range(T):
        s, p = seqs[t], poss[t]
        lo = 0 if not window else max(0, p - window + 1)
        keys = torch.arange(lo, p + 1, device=qkv.device)
        if keep_first and lo > 0:
            keys = torch.cat([torch.arange(0, min(keep_first, lo), device=qkv.device), keys])
        pages = block_table[s].long()[keys // page_size]
        offs = keys % page_size
        k = k_cache[pages, :, offs].float()          # [n, kv_heads, dh]
        v = v_cache[pages, :, :, offs].float()
        for h in range(num_heads):
            sc = (k[:, h // group] @ q[t, h]) * scale
            if softcap:
                sc = softcap * torch.tanh(sc / softcap)
            if slopes is not None:
                sc = sc - slopes[h] * (p - keys).float()
            if sinks is not None:
                pr = torch.softmax(torch.cat([sc, sinks[h:h + 1].float()]), dim=0)[:-1]
            else:
                pr = torch.softmax(sc, dim=0)
            res[t, h] = pr @ v[:, h // group]
            if gate is not None:
                res[t, h] *= torch.sigmoid(gate[t, h].float())
    _store(out, res.reshape(T, num_heads * head_dim))


def paged_attention_dense(qkv, out, k_cache, v_cache, block_table, q_start, ctx_lens, seq_of_token, positions,
                          num_heads, num_kv_heads, head_dim, scale, window, max_q_len, max_ctx_len, implementation=None, old_lens=None,
                          singles=0, units=None, unit_slots=(0, 0), softcap=0.0, slopes=None, gate=None, keep_first=0, sinks=None):
    """The same formula as :func:`paged_attention`, a sequence at a time instead of a token and a head at a time (for
    contexts of thousands of keys): scores of all the sequence's tokens against all its keys in float32, keys outside
    [p - window + 1, p] masked, softmax, weighted sum."""
    T = qkv.shape[0]
    page_size = k_cache.shape[2]
    group = num_heads // num_kv_heads
    q = qkv[:, :num_heads * head_dim].reshape(T, num_heads, head_dim).float()
    res = torch.zeros(T, num_heads, head_dim, dtype=torch.float32, device=qkv.device)
    starts, lens = q_start.tolist(), ctx_lens.tolist()
    for s, c in enumerate(lens):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        keys = torch.arange(c, device=qkv.device)
        pages = block_table[s].long()[keys // page_size]
        offs = keys % page_size
        k = k_cache[pages, :, offs].float().repeat_interleave(group, dim=1)          # [c, heads, dh]
        v = v_cache[pages, :, :, offs].float().repeat_interleave(group, dim=1)
        pos = positions[lo:hi].long()
        sc = torch.einsum("thd,chd->htc", q[lo:hi], k) * scale
        if softcap:
            sc = softcap * torch.tanh(sc / softcap)
        if slopes is not None:
            sc = sc - slopes[:, None, None] * (pos[:, None] - keys[None, :]).float()[None]
        seen = keys[None, :] <= pos[:, None]
        if window:
            inside = keys[None, :] > pos[:, None] - window
            if keep_first:
                inside |= keys[None, :] < keep_first
            seen &= inside
        sc = sc.masked_fill(~seen[None], float("-inf"))
        if sinks is not None:
            sk = sinks.float()[:, None, None].expand(num_heads, hi - lo, 1)
            pr = torch.softmax(torch.cat([sc, sk], dim=-1), dim=-1)[..., :-1]
        else:
            pr = torch.softmax(sc, dim=-1)
        res[lo:hi] = torch.einsum("htc,chd->thd", pr, v)
        if gate is not None:
            res[lo:hi] *= torch.sigmoid(gate[lo:hi].float())[:, :, None]
    _store(out, res.reshape(T, num_heads * head_dim))


def _norm_of(v, spec):
    weight, centered, eps = spec
    v = v.float()
    if weight is None:                                    # no norm: the row as it is
        return v
    if int(centered) == 2:                                # a factor per channel and no statistic
        return v * weight
    if centered:
        v = v - v.mean(-1, keepdim=True)
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight


def norm_add_norm(x32, y, post, nxt, out, rows=None):
    if hasattr(y, "place_of"):                           # a sum of rows (kernels.RowSum), taken in float32
        T, H = x32.shape
        r = y.rows[y.place_of.long()].float().view(T, y.top, H)
        y = (r * y.weights[:, :, None] if y.weights is not None else r).sum(1)
    if y is not None:
        x32.add_(_norm_of(y, post) if post is not None else y.float())
    if nxt is not None:
        _store(out, _norm_of(x32 if rows is None else x32[rows.long()], nxt))


def add_row(x32, row):
    x32.add_(row)


def rmsnorm_cols(x, col, n, width, weight, eps, out, col_a, col_b=-1):
    v = x[:, col:col + n].float()
    r = (v / torch.sqrt((v * v).sum(-1, keepdim=True) / width + eps) * weight).to(out.dtype)
    out[:, col_a:col_a + n] = r
    if col_b >= 0:
        out[:, col_b:col_b + n] = r


def conv_norm_rope_kv(proj, out, conv_w, state, state_off, q_start, seq_of_token, slots, q_norm, k_norm, eps, norm_width, positions,
                      denominators, rotary_dim, slot_mapping, k_cache, v_cache, num_heads, num_kv_heads, head_dim, write=True, shift=False, to_cache=True,
                      row_rinv=None):
    if shift and write and conv_w is not None and conv_w.shape[1] > 1:
        # (the state moves on after the convolution has read it: taken care of at the end)
        conv_norm_rope_kv(proj, out, conv_w, state, state_off, q_start, seq_of_token, slots, q_norm, k_norm, eps, norm_width, positions,
                          denominators, rotary_dim, slot_mapping, k_cache, v_cache, num_heads, num_kv_heads, head_dim, write, False, to_cache, row_rinv)
        conv_state_shift(proj, 0, proj.shape[1], conv_w.shape[1], state, state_off, q_start, slots)
        return
    T, N = proj.shape
    u = proj.float()
    if conv_w is not None:
        taps = conv_w.shape[1]
        starts, sl = q_start.tolist(), slots.tolist()
        res = torch.zeros_like(u)
        for s in range(len(starts) - 1):
            lo, hi = starts[s], starts[s + 1]
            if hi == lo:
                continue
            old = state[sl[s], state_off:state_off + (taps - 1) * N].view(taps - 1, N) if taps > 1 else u[:0]
            padded = torch.cat([old, u[lo:hi]], dim=0)
            for j in range(taps):
                res[lo:hi] += padded[j:j + hi - lo] * conv_w[:, j]
        u = res
    q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
    half = rotary_dim // 2
    if rotary_dim:
        phi = positions.float()[:, None] / denominators[None, :]
        cos, sin = torch.cos(phi)[:, None, :], torch.sin(phi)[:, None, :]

    def shape(x, weight, which=0):
        x = x.clone()
        if weight is not None and row_rinv is not None:
            # the norm over the whole projection: its factor is given, the weight is per channel
            x = x * row_rinv[:, which, None, None] * weight.view(1, x.shape[1], x.shape[2])
        elif weight is not None:
            x = x / torch.sqrt((x * x).sum(-1, keepdim=True) / norm_width + eps) * weight
        if rotary_dim:
            a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
            x[..., :half] = a * cos - b * sin
            x[..., half:rotary_dim] = b * cos + a * sin
        return x

    out[:, :q_dim] = shape(u[:, :q_dim].reshape(T, num_heads, head_dim), q_norm).reshape(T, q_dim).to(out.dtype)
    if not write or num_kv_heads == 0:
        return
    k = shape(u[:, q_dim:q_dim + kv_dim].reshape(T, num_kv_heads, head_dim), k_norm, 1).to(out.dtype)
    v = u[:, q_dim + kv_dim:].reshape(T, num_kv_heads, head_dim).to(out.dtype)
    if not to_cache:
        out[:, q_dim:q_dim + kv_dim] = k.reshape(T, kv_dim)
        out[:, q_dim + kv_dim:] = v.reshape(T, kv_dim)
        return
    page_size = k_cache.shape[2]
    page = (slot_mapping // page_size).long()
    off = (slot_mapping % page_size).long()
    k_cache[page, :, off] = k
    v_cache[page, :, :, off] = v


def row_rinv(x, ranges, eps, out):
    out.zero_()
    for j, (col, n, width) in enumerate(ranges):
        v = x[:, col:col + n].float()
        out[:, j] = 1.0 / torch.sqrt((v * v).sum(-1) / width + eps)


def add_pair_rows(x32, pairs, ids, positions, q_start, seq_of_token, slots, state, mul_prev, mul_cur):
    buckets = pairs.shape[0] - 1
    starts, sl = q_start.tolist(), slots.tolist()
    tok, pos = ids.tolist(), positions.tolist()
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        prev = int(state[sl[s], 0])
        for t in range(lo, hi):
            row = buckets if pos[t] == 0 else (prev * int(mul_prev) + tok[t] * int(mul_cur)) % buckets
            x32[t] += pairs[row].float()
            prev = tok[t]
        state[sl[s], 0] = prev


def grouped_linear(a, weight, out, row_offsets=None, a_group_cols=0, out_group_cols=0, tile_group=None, epilogue=None, epilogue_params=None):
    G, N, Kd = weight.shape
    if row_offsets is not None:
        offs = row_offsets.tolist()
        for g in range(G):
            lo, hi = offs[g], offs[g + 1]
            if hi > lo:
                y = a[lo:hi].float() @ weight[g].float().t()
                if epilogue == "swiglu":
                    y = y.view(hi - lo, N // 16, 2, 8)                 # columns come as 8 gate, 8 up, 8 gate, 8 up, ...
                    gate, up = y[:, :, 0, :], y[:, :, 1, :]
                    y = (up * (gate / (1.0 + torch.exp(-gate)))).reshape(hi - lo, N // 2)
                elif epilogue == "glu_clamped":
                    limit, alpha = (float(x) for x in epilogue_params.tolist())
                    y = y.view(hi - lo, N // 16, 2, 8)
                    gate, up = torch.clamp(y[:, :, 0, :], max=limit), torch.clamp(y[:, :, 1, :], min=-limit, max=limit)
                    y = (gate / (1.0 + torch.exp(-alpha * gate)) * (up + 1.0)).reshape(hi - lo, N // 2)
                out[lo:hi] = y.to(out.dtype)
        return
    for g in range(G):
        out[:, g * out_group_cols:g * out_group_cols + N] = (a[:, g * a_group_cols:g * a_group_cols + Kd].float() @ weight[g].float().t()).to(out.dtype)


def moe_route(logits, top, ids, weights, scoring="sigmoid"):
    if scoring == "softmax_chosen":
        order = torch.sort(logits.float(), dim=-1, descending=True, stable=True)
        ids.copy_(order.indices[:, :top].to(torch.int32))
        weights.copy_(torch.softmax(order.values[:, :top], dim=-1))
        return
    s = torch.sigmoid(logits.float())
    E = s.shape[1]
    # the largest scores, the lower index first among equals
    order = torch.sort(s - torch.arange(E, device=s.device) * 0.0, dim=-1, descending=True, stable=True)
    ids.copy_(order.indices[:, :top].to(torch.int32))
    weights.copy_(order.values[:, :top])


def sorted_rows(pairs, experts, pad=1):
    return pairs if pad <= 1 else -(-(pairs + experts * (pad - 1)) // pad) * pad


def moe_sort(ids, experts, offsets, pair_at, place_of, pad=1, tile_group=None, matrices=None):
    flat = ids.reshape(-1).long()
    counts = torch.bincount(flat, minlength=experts).tolist()
    pair_at.fill_(-1)
    if tile_group is not None:
        tile_group.fill_(-1)
    start = 0
    for e in range(experts):
        mine = torch.nonzero(flat == e).reshape(-1)                  # ascending: the order of the pairs
        offsets[e] = start
        pair_at[start:start + counts[e]] = mine.to(torch.int32)
        place_of[mine] = torch.arange(start, start + counts[e], dtype=torch.int32, device=ids.device)
        run = -(-counts[e] // pad) * pad
        if tile_group is not None:
            tile_group[start // pad:(start + run) // pad] = e if matrices is None or e < matrices else -1
        start += run
    offsets[experts] = start


def moe_gather(h, pair_at, weights, top, out):
    at = pair_at.long().clamp_min(0)
    src = h[at // top].float()
    if weights is not None:
        src = src * weights.reshape(-1)[at][:, None]
    _store(out, src * (pair_at >= 0).float()[:, None])


def moe_combine(rows, place_of, weights, top, y):
    T, H = y.shape
    r = rows[place_of.long()].float().view(T, top, H)
    if weights is not None:
        r = r * weights[:, :, None]
    _store(y, r.sum(1))


def gather_rows(src, rows, out):
    out.copy_(src[rows.long()])


def scale_inplace(x32, factor):
    x32.mul_(factor)


def logit_cap(logits, cap):
    logits.copy_(cap * torch.tanh(logits / cap))


def swiglu(gate_up, out):
    I = gate_up.shape[1] // 2
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    _store(out, u * (g / (1.0 + torch.exp(-g))))


def glu_clamped(gate_up, out, limit, alpha):
    I = gate_up.shape[1] // 2
    g = torch.clamp(gate_up[:, :I].float(), max=limit)
    u = torch.clamp(gate_up[:, I:].float(), min=-limit, max=limit)
    _store(out, g * torch.sigmoid(alpha * g) * (u + 1.0))


def weighted_sum2(a, b, sa, sb, out):
    _store(out, sa * a.float() + sb * b.float())


def add_position_rows(x32, table, positions):
    x32.add_(table[positions.long()].float())


def hc_expand(x32, xs):
    xs.copy_(x32[:, None, :].expand_as(xs))


def hc_read_norm(xs, in_w, rows, weight, eps, out):
    src = xs if rows is None else xs[rows.long()]
    u = src.sum(dim=1) if in_w is None else torch.einsum("s,tsw->tw", in_w, src)
    _store(out, _rms(u, weight, eps))


def hc_update(xs, y, mix, out_w, next_in=None, next_weight=None, eps=0.0, next_out=None):
    if hasattr(y, "sa"):                                   # a pair that stands for sa * a + sb * b
        y = y.sa * y.a.float() + y.sb * y.b.float()
    new = torch.einsum("sr,tsw->trw", mix, xs) + out_w[None, :, None] * y.float()[:, None, :]
    xs.copy_(new)
    if next_out is not None:
        _store(next_out, _rms(torch.einsum("s,tsw->tw", next_in, xs), next_weight, eps))


def _silu(x):
    return x * torch.sigmoid(x)


def causal_conv_silu(x, col, weight, bias, state, state_off, q_start, seq_of_token, slots, out, shift=False):
    C, taps = weight.shape
    starts, sl = q_start.tolist(), slots.tolist()
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        before = state[sl[s], state_off:state_off + (taps - 1) * C].view(taps - 1, C)
        seq = torch.cat([before, x[lo:hi, col:col + C].float()], dim=0)
        acc = bias[None, :].expand(hi - lo, C).clone()
        for k in range(taps):
            acc += weight[:, k][None, :] * seq[k:k + hi - lo]
        _store(out[lo:hi], _silu(acc))
    if shift:
        conv_state_shift(x, col, C, taps, state, state_off, q_start, slots)


def conv_state_shift(x, col, channels, taps, state, state_off, q_start, slots):
    starts, sl = q_start.tolist(), slots.tolist()
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo or taps == 1:
            continue
        view = state[sl[s], state_off:state_off + (taps - 1) * channels].view(taps - 1, channels)
        seq = torch.cat([view, x[lo:hi, col:col + channels].float()], dim=0)
        view.copy_(seq[-(taps - 1):])


def ssm_scan(xbc, proj, dt_col, dt_bias, A_log, D, state, q_start, slots, y32, heads, head_dim, state_size, groups, chunks=None):
    # (chunks only says how a kernel shares the work out)
    starts, sl = q_start.tolist(), slots.tolist()
    inner, P, N = heads * head_dim, head_dim, state_size
    rate = torch.exp(A_log)
    per = heads // groups
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        S = state[sl[s], :heads * N * P].view(heads, P, N).transpose(1, 2)          # kept column by column: [heads][P][N]
        for t in range(lo, hi):
            row = xbc[t].float()
            x = row[:inner].view(heads, P)
            B = row[inner:inner + groups * N].view(groups, N).repeat_interleave(per, dim=0)
            Cm = row[inner + groups * N:].view(groups, N).repeat_interleave(per, dim=0)
            dt = torch.nn.functional.softplus(proj[t, dt_col:dt_col + heads].float() + dt_bias, threshold=1e9)
            S.mul_(torch.exp(-rate * dt)[:, None, None]).add_((dt[:, None] * B)[:, :, None] * x[:, None, :])
            y32[t] = (torch.einsum("hnp,hn->hp", S, Cm) + D[:, None] * x).reshape(inner)


def decay_scan(qkv, q_col, k_col, v_col, decay, state, q_start, slots, out32, heads, dim, vdim, chunks=None):
    starts, sl = q_start.tolist(), slots.tolist()
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        S = state[sl[s], :heads * dim * vdim].view(heads, vdim, dim).transpose(1, 2)      # kept column by column: [heads][vdim][dim]
        for t in range(lo, hi):
            row = qkv[t].float()
            q = _silu(row[q_col:q_col + heads * dim]).view(heads, dim)
            k = _silu(row[k_col:k_col + heads * dim]).view(heads, dim)
            v = _silu(row[v_col:v_col + heads * vdim]).view(heads, vdim)
            S.mul_(decay[:, None, None]).add_(k[:, :, None] * v[:, None, :])
            out32[t] = torch.einsum("hdv,hd->hv", S, q).reshape(heads * vdim)


def gla_scan(qkv, q_col, k_col, v_col, za, za_col, tau, state, q_start, slots, out32, heads, dim, vdim, chunks=None):
    starts, sl = q_start.tolist(), slots.tolist()
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        S = state[sl[s], :heads * dim * vdim].view(heads, vdim, dim).transpose(1, 2)      # kept column by column: [heads][vdim][dim]
        for t in range(lo, hi):
            row = qkv[t].float()
            q = row[q_col:q_col + heads * dim].view(heads, dim) * float(dim) ** -0.5
            k = row[k_col:k_col + heads * dim].view(heads, dim)
            v = row[v_col:v_col + heads * vdim].view(heads, vdim)
            a = torch.exp(torch.nn.functional.logsigmoid(za[t, za_col:za_col + heads * dim].float()) / float(tau)).view(heads, dim)
            S.mul_(a[:, :, None]).add_(k[:, :, None] * v[:, None, :])
            out32[t] = torch.einsum("hdv,hd->hv", S, q).reshape(heads * vdim)


def channel_scan(x, x_col, bc, b_col, c_col, dt32, z, z_col, A_log, D, state, q_start, slots, y, chunks=None):
    starts, sl = q_start.tolist(), slots.tolist()
    inner, N = A_log.shape
    A = -torch.exp(A_log)
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        S = state[sl[s], :inner * N].view(inner, N)
        for t in range(lo, hi):
            xt = x[t, x_col:x_col + inner].float()
            B, Cm = bc[t, b_col:b_col + N].float(), bc[t, c_col:c_col + N].float()
            dt = torch.nn.functional.softplus(dt32[t], threshold=1e9)
            S.mul_(torch.exp(dt[:, None] * A)).add_((dt * xt)[:, None] * B[None, :])
            r = S @ Cm + D * xt
            y[t] = (r * _silu(z[t, z_col:z_col + inner].float())).to(y.dtype)


def gated_rmsnorm(y32, gate, gate_col, weight, eps, groups, gate_first, out, gate_act="sigmoid"):
    T, n = y32.shape
    z = gate[:, gate_col:gate_col + n].float()
    v = y32 * _silu(z) if gate_first else y32
    v = v.view(T, groups, n // groups)
    v = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)).reshape(T, n) * weight
    _store(out, v if gate_first else v * (_silu(z) if gate_act == "silu" else torch.sigmoid(z)))



def moe_route_grouped(logits, correction, top, groups, keep, scale, ids, weights):
    s = torch.softmax(logits.float(), dim=-1)
    T, E = s.shape
    choice = s + correction if correction is not None else s.clone()
    if keep < groups:
        best = choice.view(T, groups, E // groups).max(dim=-1).values
        order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
        kept = torch.zeros((T, groups), dtype=torch.bool, device=s.device)
        kept.scatter_(1, order, True)
        choice = choice.masked_fill(~kept[:, :, None].expand(T, groups, E // groups).reshape(T, E), float("-inf"))
    chosen = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    sc = torch.gather(s, 1, chosen)
    ids.copy_(chosen.to(torch.int32))
    weights.copy_(sc / (sc.sum(-1, keepdim=True) + 1e-20) * scale)


def polynorm(z, coef, eps, out):
    a, b, c, e = (float(x) for x in coef.tolist())
    v = z.float()

    def n(u):
        return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)

    _store(out, a * n(v) + b * n(v * v) + c * n(v * v * v) + e)


def mul_sigmoid(x, gate, gate_col=0, group=1):
    T, n = x.shape
    g = gate[:, gate_col:gate_col + n // group].float().repeat_interleave(group, dim=1)
    _store(x, x.float() * torch.sigmoid(g))


def latent_rope_post(low, col_c, col_r, q, dim, weight, eps, positions, denominators, magnitude, interleaved, out, num_heads, rank, rot_dim, head):
    T = low.shape[0]
    c = low[:, col_c:col_c + rank].float()
    c = (c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * weight).to(out.dtype)
    rows = out.view(T, num_heads + 2, head)
    rows[:, num_heads, :rank] = c
    rows[:, num_heads + 1, :rank] = c
    rows[:, num_heads + 1, rank:] = 0
    rows[:, :num_heads + 1, rank + rot_dim:] = 0
    if not rot_dim:
        return
    half = rot_dim // 2
    ang = positions.float()[:, None] / denominators[None, :]
    cs, sn = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    src = torch.cat([q[:, :num_heads * (dim + rot_dim)].reshape(T, num_heads, dim + rot_dim)[:, :, dim:], low[:, None, col_r:col_r + rot_dim]], dim=1).float()
    ia = torch.arange(0, rot_dim, 2) if interleaved else torch.arange(0, half)
    ib = ia + 1 if interleaved else ia + half
    a, b = src[..., ia], src[..., ib]
    res = torch.empty_like(src)
    res[..., ia] = a * cs - b * sn
    res[..., ib] = b * cs + a * sn
    rows[:, :num_heads + 1, rank:rank + rot_dim] = res.to(out.dtype)


def delta_row_elements(dim):
    return 32 if dim <= 32 else 64 if dim <= 64 else 128 if dim <= 128 else 256


def delta_prepare(proj, col, b_col, conv_w, state, state_off, q_start, seq_of_token, slots, za, za_col, A_log, prep_qk, prep_g, v32, heads, kv_heads,
                  dim, vdim, unit_eps=1e-6, shift=False):
    T = proj.shape[0]
    C, taps = conv_w.shape
    DP = delta_row_elements(dim)
    starts, sl = q_start.tolist(), slots.tolist()
    u = torch.zeros((T, C), dtype=torch.float32, device=proj.device)
    x = proj[:, col:col + C].float()
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        old = state[sl[s], state_off:state_off + (taps - 1) * C].view(taps - 1, C)
        hist = torch.cat([old, x[lo:hi]], dim=0)
        for k in range(taps):
            u[lo:hi] += hist[k:k + hi - lo] * conv_w[:, k][None, :]
        if shift and taps > 1:
            old.copy_(hist[hi - lo:])
    u = u * torch.sigmoid(u)
    G = kv_heads
    q, k, v = u[:, :G * dim].view(T, G, dim), u[:, G * dim:2 * G * dim].view(T, G, dim), u[:, 2 * G * dim:]
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * float(dim) ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    prep_qk.zero_()
    prep_qk[:, :, :dim] = q
    prep_qk[:, :, DP:DP + dim] = k
    prep_qk[:, :, 2 * DP] = (q * k).sum(-1)
    prep_g.zero_()
    sp = torch.nn.functional.softplus(za[:, za_col:za_col + heads * dim].float(), threshold=1e9).view(T, heads, dim)
    prep_g[:, :, :dim] = torch.exp(-torch.exp(A_log)[None, :, None] * sp)
    prep_g[:, :, DP] = torch.sigmoid(proj[:, b_col:b_col + heads].float())
    v32.copy_(v)


def delta_scan(prep_qk, prep_g, v32, state, q_start, slots, out32, heads, kv_heads, dim, vdim):
    starts, sl = q_start.tolist(), slots.tolist()
    rep = heads // kv_heads
    DP = delta_row_elements(dim)
    for s in range(len(starts) - 1):
        lo, hi = starts[s], starts[s + 1]
        if hi == lo:
            continue
        S = state[sl[s], :heads * dim * vdim].view(heads, vdim, dim).transpose(1, 2)      # kept column by column: [heads][vdim][dim]
        for t in range(lo, hi):
            q = prep_qk[t, :, :dim].repeat_interleave(rep, dim=0)
            k = prep_qk[t, :, DP:DP + dim].repeat_interleave(rep, dim=0)
            g, beta = prep_g[t, :, :dim], prep_g[t, :, DP]
            v = v32[t].view(heads, vdim)
            S.mul_(g[:, :, None])
            u = beta[:, None] * (v - torch.einsum("hdv,hd->hv", S, k))
            S.add_(k[:, :, None] * u[:, None, :])
            out32[t] = torch.einsum("hdv,hd->hv", S, q).reshape(heads * vdim)


def argmax(logits, out):
    # first maximum
    m = logits.max(dim=1, keepdim=True).values
    idx = torch.where(logits == m, torch.arange(logits.shape[1], device=logits.device)[None, :], logits.shape[1]).min(dim=1).values
    out.copy_(idx.to(torch.int32))


# ---- sampling ---------------------------------------------------------------

_M64 = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def uniform_for(seed: int, output_index: int, token: int) -> float:
    """The generator of the sample kernel: 23 bits of a hash of (seed, index, token), in (0, 1)."""
    key = _splitmix64((seed & _M64) ^ _splitmix64(output_index & _M64))
    bits = _splitmix64(key ^ ((token * 0xD1342543DE82EF95) & _M64)) >> 41
    return (bits + 0.5) / 8388608.0


def sample_row(logits_row, temperature, top_k, top_p, seed, output_index):
    """(token, kept ids) as the sample kernel computes them."""
    z = logits_row.float().cpu()
    V = z.numel()
    if temperature <= 0.0 or top_k == 1:
        m = z.max()
        return int(torch.nonzero(z == m)[0]), None
    z = z / np.float32(temperature)
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.topk(z, top_k).values[-1]
        keep &= z >= kth
    if 0.0 < top_p < 1.0:
        m = z[keep].max()
        e = torch.where(keep, torch.exp(z - m), torch.zeros(()))
        p = e / e.sum()
        # kept iff the probability mass of strictly larger candidates is below top_p
        order = torch.argsort(z, descending=True, stable=True)
        ps = p[order]
        zs = z[order]
        before = torch.cumsum(ps, 0) - ps
        # equal values share the mass before the first of them
        first_of_value = torch.ones(V, dtype=torch.bool)
        first_of_value[1:] = zs[1:] != zs[:-1]
        idx = torch.where(first_of_value, torch.arange(V), torch.zeros((), dtype=torch.long))
        idx = torch.cummax(idx, 0).values
        before = before[idx]
        ok = torch.zeros(V, dtype=torch.bool)
        ok[order] = before < top_p
        keep &= ok
    u = torch.tensor([uniform_for(seed, output_index, i) for i in range(V)], dtype=torch.float32)
    g = -torch.log(-torch.log(u))
    score = torch.where(keep, z + g, torch.full((), float("-inf")))
    m = score.max()
    return int(torch.nonzero(score == m)[0]), torch.nonzero(keep).flatten().tolist()


def sample(logits, params, out):
    host = params.cpu()
    f = host.view(torch.float32)
    res = []
    for r in range(logits.shape[0]):
        seed = (int(host[r, 3]) & 0xFFFFFFFF) | ((int(host[r, 4]) & 0xFFFFFFFF) << 32)
        tok, _ = sample_row(logits[r], float(f[r, 0]), int(host[r, 1]), float(f[r, 2]), seed, int(host[r, 5]))
        res.append(tok)
    out.copy_(torch.tensor(res, dtype=torch.int32))


def table_gather(resident, updates, slots, out, trash_page):
    """The resident block tables brought up to date and a row per sequence copied out: plain loops."""
    rows, cols = resident.shape
    n = int(updates[0])
    wanted = set(int(x) for x in slots.tolist())
    for i in range(n):
        slot, block, page = (int(x) for x in updates[1 + 3 * i:4 + 3 * i].tolist())
        if slot in wanted and slot != rows - 1 and 0 <= block < cols:
            resident[slot, block] = page
    for s, slot in enumerate(slots.tolist()):
        slot = slot if 0 <= slot < rows else rows - 1
        for b in range(out.shape[1]):
            out[s, b] = resident[slot, b] if b < cols else trash_page


ALL = ["moe_route_grouped", "polynorm", "mul_sigmoid", "latent_rope_post", "delta_prepare", "delta_scan", "delta_row_elements", "row_rinv", "add_pair_rows", "gla_scan", "channel_scan", "sorted_rows", "norm_add_norm", "add_row", "rmsnorm_cols", "conv_norm_rope_kv", "grouped_linear", "moe_route", "moe_sort", "moe_gather", "moe_combine",
       "glu_clamped", "weighted_sum2", "add_position_rows", "hc_expand", "hc_read_norm", "hc_update", "causal_conv_silu", "conv_state_shift", "ssm_scan",
       "decay_scan", "gated_rmsnorm", "table_gather", "gather_rows", "scale_inplace", "logit_cap", "rope_table", "linear_scaled_accepts", "linear_add_scaled_parts", "linear_add_scaled", "apply_row_scale", "linear_rope_kv", "interleave_gate_up", "embedding", "rmsnorm", "add_rmsnorm", "gather_rmsnorm", "residual_add", "linear", "rope_kv_write",
       "paged_attention", "swiglu", "argmax", "sample"]
