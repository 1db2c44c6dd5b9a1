"""Test doubles of the CUDA kernels in plain torch, for tests of host-side logic on the CPU.

``install(monkeypatch)`` replaces the functions of ``pico_vllm_b200.ops`` so that the step
function, the cache and the scheduler can be driven without a GPU.  These doubles also serve
as the plain reference of each kernel in the GPU tests (same signatures, float32 arithmetic).
They are not part of the product: the package itself has no CPU path.
"""
import math

import torch

import plain_qwen2 as plain


def embedding(ids, table, out, feedback=None):
    ids = ids.long()
    if feedback is not None:
        ids = torch.where(ids < 0, feedback.long()[(-ids - 1).clamp(min=0)], ids)
    out.copy_(table[ids].float())
    return out


def add_rmsnorm(x, delta, weight, eps, out, rows=None):
    if rows is None:
        if delta is not None:
            x.add_(delta.float())
        src = x
    else:
        src = x[rows.long()]
        if delta is not None:
            src = src + delta[rows.long()].float()
    out.copy_(plain.rms_norm(src, weight, eps).to(out.dtype))
    return out


def swiglu(gate_up, out):
    I = out.shape[1]
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))
    return out


def rope_store(qkv, bias, positions, inv_freq, slots, k_pages, v_pages, n_heads, n_kv_heads, head_dim,
               page_size, pairing="half"):
    T = qkv.shape[0]
    x = qkv.float()
    if bias is not None:
        x = x + bias
    nq, nk = n_heads * head_dim, n_kv_heads * head_dim
    q = x[:, :nq].view(T, n_heads, head_dim)
    k = x[:, nq:nq + nk].view(T, n_kv_heads, head_dim)
    v = x[:, nq + nk:].view(T, n_kv_heads, head_dim)
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = ang.cos(), ang.sin()
    r = inv_freq.shape[0]
    half = head_dim // 2

    def rot(t):
        t = t.clone()
        x1, x2 = t[..., :r].clone(), t[..., half:half + r].clone()
        t[..., :r] = x1 * cos[:, None, :] - x2 * sin[:, None, :]
        t[..., half:half + r] = x2 * cos[:, None, :] + x1 * sin[:, None, :]
        return t
    qkv[:, :nq] = rot(q).reshape(T, nq).to(qkv.dtype)
    if slots is not None:
        kr = rot(k)
        keep = slots >= 0
        s = slots[keep].long()
        page, off = s // page_size, s % page_size
        k_pages[page, :, off, :] = kr[keep].to(k_pages.dtype)
        v_pages[page, :, off, :] = v[keep].to(v_pages.dtype)


def attention_scratch_floats(T, n_heads, head_dim, n_splits):
    return 0 if n_splits <= 1 else T * n_heads * n_splits * (head_dim + 2)


def paged_attention(q, k_pages, v_pages, out, tok_seg, positions, block_table, n_heads, n_kv_heads,
                    head_dim, page_size, window, scale, n_splits=1, scratch=None, softcap=None, slopes=None, chunk=None,
                    sinks=None):
    T = q.shape[0]
    g = n_heads // n_kv_heads
    for t in range(T):
        p = int(positions[t])
        if p < 0:
            out[t] = 0
            continue
        lo = max(0, p + 1 - window) if window else 0
        if chunk:
            lo = max(lo, p // chunk * chunk)
        n = torch.arange(lo, p + 1)
        pages = block_table[int(tok_seg[t])].long()[n // page_size]
        k = k_pages[pages, :, n % page_size, :].float()    # [keys, kv_heads, hd]
        v = v_pages[pages, :, n % page_size, :].float()
        qt = q[t, :n_heads * head_dim].float().view(n_heads, head_dim)
        for h in range(n_heads):
            s = (k[:, h // g, :] @ qt[h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if slopes is not None:
                s = s - float(slopes[h]) * (p - n).float()
            if sinks is not None:
                e = torch.exp(s - float(sinks[h]))
                pr = e / (1.0 + e.sum())
            else:
                pr = torch.softmax(s, dim=0)
            out[t, h * head_dim:(h + 1) * head_dim] = (pr @ v[:, h // g, :]).to(out.dtype)
    return out


def mma_attention_takes(dtype, n_heads, n_kv_heads, head_dim):
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 16)


def paged_attention_mma(q, k_pages, v_pages, out, tok_seg, positions, block_table, cu_q, prefill_segs,
                        n_prefill_segs, max_prefill_q, decode_tokens, n_decode_tokens, n_heads, n_kv_heads, head_dim,
                        page_size, window, scale, n_splits=1, scratch=None, k_map=None, v_map=None, k_map2d=None,
                        v_map2d=None, pair_min_keys=0, softcap=None, slopes=None, chunk=None, sinks=None):
    return paged_attention(q, k_pages, v_pages, out, tok_seg, positions, block_table, n_heads, n_kv_heads, head_dim,
                           page_size, window, scale, softcap=softcap, slopes=slopes, chunk=chunk, sinks=sinks)


SKINNY_MAX_TOKENS = 16


def skinny_takes(x, weight, n_multiple=16):
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and 1 <= x.shape[0] <= 16
            and x.shape[1] % 16 == 0 and weight.shape[0] % n_multiple == 0 and weight.shape[0] >= 16)


def skinny_norm_takes(x, weight, n_rows=None):
    M = x.shape[0] if n_rows is None else n_rows
    return x.dtype == torch.float32 and weight.dtype == torch.bfloat16 and 1 <= M <= 16 and x.shape[1] % 16 == 0 \
        and weight.shape[0] % 16 == 0 and x.shape[1] <= 2000


def _normed(x, norm_weight, eps, rows=None):
    if norm_weight is None:
        return x
    if rows is not None:
        x = x[rows.long()]
    return plain.rms_norm(x.float(), norm_weight, eps).to(torch.bfloat16)


def skinny_linear(x, weight, bias=None, out_dtype=torch.bfloat16, norm_weight=None, eps=0.0, rows=None):
    x = _normed(x, norm_weight, eps, rows)
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias
    return y.to(out_dtype)


def skinny_argmax(x, weight, out, norm_weight=None, eps=0.0, rows=None):
    logits = skinny_linear(x, weight, None, torch.float32, norm_weight, eps, rows)
    out[:logits.shape[0]] = logits.argmax(-1).to(out.dtype)
    return out


def skinny_linear_residual(x, weight, residual):
    residual.add_(x.float() @ weight.float().t())


def skinny_gate_up_swiglu(x, gate_up_weight, norm_weight=None, eps=0.0):
    x = _normed(x, norm_weight, eps)
    gu = x.float() @ gate_up_weight.float().t()
    I = gu.shape[1] // 2
    g, u = gu[:, :I], gu[:, I:]
    return (g * torch.sigmoid(g) * u).to(torch.bfloat16)


def skinny_qkv_rope_store(x, qkv_weight, bias, positions, inv_freq, slots, k_pages, v_pages, n_heads, n_kv_heads,
                          head_dim, page_size, norm_weight=None, eps=0.0, pairing="half"):
    x = _normed(x, norm_weight, eps)
    qkv = x.float() @ qkv_weight.float().t()          # float32 until after the rotation, like the kernel
    rope_store(qkv, bias, positions, inv_freq, slots, k_pages, v_pages, n_heads, n_kv_heads, head_dim, page_size)
    return qkv[:, :n_heads * head_dim].to(torch.bfloat16)


def make_kv_tensor_map(pages):
    return None


def make_kv_tensor_map_2d(pages, values=False):
    return None


def tc_takes(x, weight):
    return False


def linear(x, weight, out=None):
    y = (x.float() @ weight.float().t()).to(x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def logits_linear(x, weight):
    return x.float() @ weight.float().t()


def sample(logits, temperature, top_p, uniform, out):
    R, V = logits.shape
    for r in range(R):
        t = 0.0 if temperature is None else float(temperature[r])
        if t <= 0:
            out[r] = int(torch.argmax(logits[r]))
            continue
        probs = plain.softmax_temperature(logits[r].double(), t)
        tp = 1.0 if top_p is None else float(top_p[r])
        if tp < 1.0:
            probs = plain.top_p_filter(probs[None], tp)[0]
        cum = torch.cumsum(probs, 0)
        idx = int(torch.searchsorted(cum, torch.tensor(float(uniform[r]) * float(cum[-1]), dtype=cum.dtype),
                                     right=True))
        out[r] = min(idx, V - 1)
    return out


# ------------------------------------------------------------------ norm -> add -> norm, latent attention, routed experts
def _norm(u, kind, w, eps):
    if kind in (0, 3):          # none; 3: no norm on the way out, the row is only written in the activation type
        return u
    if kind == 2:
        u = u - u.mean(-1, keepdim=True)
    y = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def post_add_norm(x, delta, post_weight, post_kind, post_eps, weight, kind, eps, out, rows=None):
    d = None if delta is None else _norm(delta.float(), post_kind, post_weight, post_eps)
    if rows is None:
        if d is not None:
            x.add_(d)
        src = x
    else:
        src = x[rows.long()]
        if d is not None:
            src = src + d[rows.long()]
    if out is not None:
        out.copy_(_norm(src, kind, weight, eps).to(out.dtype))
    return out


def scale_softcap(logits, scale, cap):
    logits.mul_(scale)
    if cap:
        logits.copy_(cap * torch.tanh(logits / cap))
    return logits


def latent_norm_store(proj, q_off, q_rank, q_weight, kv_off, kv_rank, kv_weight, slots, cache, g_off, heads, eps):
    p = proj.float()
    cq = _norm(p[:, q_off:q_off + q_rank], 1, q_weight, eps).to(proj.dtype) if q_rank > 0 else None
    if kv_rank > 0:
        c = _norm(p[:, kv_off:kv_off + kv_rank], 1, kv_weight, eps).to(cache.dtype)
        flat = cache.view(-1, cache.shape[-1])
        for t, s in enumerate(slots.tolist()):
            if s >= 0:
                flat[s].zero_()
                flat[s, :kv_rank] = c[t]
    return cq, (torch.sigmoid(p[:, g_off:g_off + heads]) if heads > 0 else None)


def head_linear(x, weight, out, gate=None):
    T = x.shape[0]
    H, K, N = weight.shape
    y = torch.einsum("tak,akn->tan", x.float().view(T, H, K), weight.float())
    if gate is not None:
        y = y * gate[:, :, None]
    out.copy_(y.reshape(T, H * N).to(out.dtype))
    return out


def head_scale(o, gate, heads):
    T = o.shape[0]
    o.copy_((o.float().view(T, heads, -1) * gate[:, :, None]).view(T, -1).to(o.dtype))
    return o


def moe_route(h, router_weight, router_bias, top, scoring=0, choice_bias=None, weight_scale=1.0, groups=1, groups_keep=1,
              renorm=False):
    z = h.float() @ router_weight.t()
    if router_bias is not None:
        z = z + router_bias
    if scoring == 2:
        score = torch.softmax(z, dim=-1)
        choice = score + (choice_bias if choice_bias is not None else 0.0)
        if groups > 1 and groups_keep < groups:
            T, E = choice.shape
            best = choice.view(T, groups, E // groups).max(-1).values
            kept = torch.zeros(T, groups, dtype=torch.bool)
            kept[torch.arange(T)[:, None], torch.topk(best, groups_keep, dim=-1).indices] = True
            choice = torch.where(kept[:, :, None].expand(T, groups, E // groups).reshape(T, E), choice,
                                 torch.full_like(choice, -math.inf))
        idx = torch.topk(choice, top, dim=-1).indices
        w = torch.gather(score, 1, idx)
        if renorm:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return idx.to(torch.int32), w * weight_scale
    val, idx = torch.topk(z, top, dim=-1)
    return idx.to(torch.int32), (torch.sigmoid(val) if scoring == 1 else torch.softmax(val, dim=-1))


def _act(u, act):
    return torch.relu(u) ** 2 if act == 1 else u * torch.sigmoid(u)


def _capped(g, u, limit, alpha=1.702):
    g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
    return g * torch.sigmoid(alpha * g) * (u + 1.0)


def capped_glu(gu, ff, limit, row_gate_col=None, alpha=1.702):
    x = gu.float()
    y = _capped(x[:, :ff], x[:, ff:2 * ff], limit, alpha)
    if row_gate_col is not None:
        y = y * torch.sigmoid(x[:, row_gate_col:row_gate_col + 1])
    return y.to(gu.dtype)


def moe_experts(h, idx, wgt, gate_up_weight, down_weight, gated=True, act=0, weight_on_input=False, base=None, identity=0,
                limit=0.0):
    ff = gate_up_weight.shape[1] // 2 if gated else gate_up_weight.shape[1]
    y = torch.zeros(h.shape, dtype=torch.float32) if base is None else base.float().clone()
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            if e >= gate_up_weight.shape[0]:
                assert e < gate_up_weight.shape[0] + identity
                y[t] += wgt[t, j] * h[t].float()
            elif gated:
                gu = gate_up_weight[e].float() @ h[t].float()
                g, u = gu[:ff], gu[ff:]
                y[t] += wgt[t, j] * (down_weight[e].float() @ (_capped(g, u, limit) if act == 2 else g * torch.sigmoid(g) * u))
            elif weight_on_input:
                y[t] += down_weight[e].float() @ _act(gate_up_weight[e].float() @ (wgt[t, j] * h[t].float()), act)
            else:
                y[t] += wgt[t, j] * (down_weight[e].float() @ _act(gate_up_weight[e].float() @ h[t].float(), act))
    return y.to(h.dtype)


def activation(u, act):
    u.copy_(_act(u.float(), act).to(u.dtype))
    return u


def qk_norm_rope_store(qkv, bias, positions, inv_freq, mult, q_norm, k_norm, eps, slots, k_pages, v_pages, n_heads,
                       n_kv_heads, head_dim, page_size, values_from_keys, norm_dim=None):
    T = qkv.shape[0]
    nq, nk = n_heads * head_dim, n_kv_heads * head_dim
    cols = nq + nk * (1 if values_from_keys else 2)
    x = qkv[:, :cols].float()
    if bias is not None:
        x = x + bias[:cols]
    q = x[:, :nq].view(T, n_heads, head_dim)
    k = x[:, nq:nq + nk].view(T, n_kv_heads, head_dim)
    v = k if values_from_keys else x[:, nq + nk:].view(T, n_kv_heads, head_dim)
    r = inv_freq.shape[0]
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = (ang.cos() * mult)[:, None, :], (ang.sin() * mult)[:, None, :]

    def treat(u, w):
        if w is not None:
            u = u / torch.sqrt((u * u).sum(-1, keepdim=True) / (norm_dim or head_dim) + eps) * w
        a, b = u[..., :r], u[..., r:2 * r]
        return torch.cat([a * cos - b * sin, b * cos + a * sin, u[..., 2 * r:]], dim=-1)
    live = positions >= 0
    qn = torch.where(live[:, None, None], treat(q, q_norm), q)
    qkv[:, :nq] = qn.reshape(T, nq).to(qkv.dtype)
    if slots is None:
        return
    kn = treat(k, k_norm)
    for t, s in enumerate(slots.tolist()):
        if s >= 0 and bool(live[t]):
            k_pages[s // page_size, :, s % page_size, :] = kn[t].to(k_pages.dtype)
            v_pages[s // page_size, :, s % page_size, :] = v[t].to(v_pages.dtype)


def sigmoid_gate(o, gate_logits):
    o.copy_((o.float() * torch.sigmoid(gate_logits.float())).to(o.dtype))
    return o


def decay_linear_attention(proj, q_off, k_off, v_off, decay, state, seg_slots, cu_q, positions, heads, dim, vdim, act=1,
                           max_q_len=1, chunk=None):
    T = proj.shape[0]
    p = proj.float()
    f = (lambda u: u * torch.sigmoid(u)) if act == 1 else (lambda u: u)
    q = f(p[:, q_off:q_off + heads * dim]).view(T, heads, dim)
    k = f(p[:, k_off:k_off + heads * dim]).view(T, heads, dim)
    v = f(p[:, v_off:v_off + heads * vdim]).view(T, heads, vdim)
    out = torch.zeros((T, heads * vdim), dtype=torch.float32)
    for s in range(seg_slots.shape[0]):
        b, e = int(cu_q[s]), int(cu_q[s + 1])
        if e <= b or int(positions[b]) < 0:
            continue
        S = state[int(seg_slots[s])]                            # [heads, vdim, dim]: transposed
        for t in range(b, e):
            S.mul_(decay[:, None, None]).add_(v[t][:, :, None] * k[t][:, None, :])
            out[t] = torch.einsum("hvd,hd->hv", S, q[t]).reshape(-1)
    return out


def gated_rms_norm(x, weight, gate_logits, eps, out_dtype):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight
    if gate_logits is not None:
        y = y * torch.sigmoid(gate_logits.float())
    return y.to(out_dtype)


# ------------------------------------------------------------------ several streams, recurrences with gates per token
def hyper_expand(x, streams):
    return x[:, None, :].repeat(1, streams, 1)


def _rms_unit(u, eps):
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def hyper_step(x, y, mix, out_w, in_w, norm_w, eps, out_dtype, rows=None):
    new = x if y is None else torch.einsum("sr,tsd->trd", mix, x) + out_w[None, :, None] * y.float()[:, None, :]
    if rows is None:
        x.copy_(new)
    else:
        new = new[rows.long()]
    u = new.sum(1) if in_w is None else torch.einsum("s,tsd->td", in_w, new)
    return (_rms_unit(u, eps) * norm_w).to(out_dtype)


def scale_add_rows(x, scale, table, positions):
    x.mul_(scale)
    if table is not None:
        live = positions >= 0
        x[live] += table[positions[live].long()].float()
    return x


def scaled_sum(a, sa, b, sb):
    return (sa * a.float() + sb * b.float()).to(a.dtype)


def gated_linear_attention(q, k, v, gate, per_row, state, seg_slots, cu_q, positions, heads, qk_rep, dim, vdim, max_q_len=1,
                           chunk=None):
    T = q.shape[0]
    out = torch.zeros(T, heads * vdim)
    for s in range(seg_slots.shape[0]):
        a0, a1 = int(cu_q[s]), int(cu_q[s + 1])
        if a1 <= a0 or int(positions[a0]) < 0:
            continue
        for h in range(heads):
            S = state[int(seg_slots[s]), h].T.clone()                       # [dim, vdim]
            g0 = (h // qk_rep) * dim
            for t in range(a0, a1):
                a = gate[t, h * dim:(h + 1) * dim][:, None] if per_row else gate[t, h]
                S = a * S + torch.outer(k[t, g0:g0 + dim], v[t, h * vdim:(h + 1) * vdim])
                out[t, h * vdim:(h + 1) * vdim] = S.T @ q[t, g0:g0 + dim]
            state[int(seg_slots[s]), h] = S.T
    return out


def mlstm_prepare(proj, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, q_scale, m_state, seg_slots, cu_q, positions,
                  heads, dim, vdim):
    T, H = proj.shape[0], heads
    p = proj.float()
    gi = cap * torch.tanh((p[:, i_off:i_off + H] + (i_bias if i_bias is not None else 0.0)) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((p[:, f_off:f_off + H] + (f_bias if f_bias is not None else 0.0)) / cap))
    keep, put, floor = torch.ones(T, H), torch.zeros(T, H), torch.ones(T, H)
    for s in range(seg_slots.shape[0]):
        a0, a1 = int(cu_q[s]), int(cu_q[s + 1])
        if a1 <= a0 or int(positions[a0]) < 0:
            continue
        m = m_state[int(seg_slots[s])].clone()
        for t in range(a0, a1):
            new = torch.maximum(gf[t] + m, gi[t])
            keep[t], put[t], floor[t] = torch.exp(gf[t] + m - new), torch.exp(gi[t] - new), torch.exp(-new)
            m = new
        m_state[int(seg_slots[s])] = m
    q = p[:, q_off:q_off + H * dim] * q_scale
    k = (p[:, k_off:k_off + H * dim].view(T, H, dim) * put[:, :, None]).reshape(T, H * dim)
    v = torch.cat([p[:, v_off:v_off + H * vdim].view(T, H, vdim), torch.ones(T, H, 1)], 2).reshape(T, H * (vdim + 1))
    return keep, floor, torch.cat([q, k, v], 1)


def hgrn2_prepare(proj, q_off, f_off, v_off, f_bias, lower, nqk, nv):
    p = proj.float()
    q = p[:, q_off:q_off + nqk]
    lo = lower if lower is not None else 0.0
    f = lo + (1.0 - lo) * torch.sigmoid(p[:, f_off:f_off + nqk] + (f_bias if f_bias is not None else 0.0))
    return torch.cat([q * torch.sigmoid(q), 1.0 - f, f, p[:, v_off:v_off + nv]], 1)


def causal_conv_silu(proj, c_off, weight, bias, conv_state, tok_seg, seg_slots, cu_q, positions, act=True):
    C, taps = weight.shape
    T = proj.shape[0]
    out = torch.zeros(T, C)
    for s in range(seg_slots.shape[0]):
        a0, a1 = int(cu_q[s]), int(cu_q[s + 1])
        if a1 <= a0 or int(positions[a0]) < 0:
            continue
        slot = int(seg_slots[s])
        x = torch.cat([conv_state[slot], proj[a0:a1, c_off:c_off + C].float()])        # [taps - 1 + n, C]
        for t in range(a1 - a0):
            acc = (x[t:t + taps] * weight.t()).sum(0) + (bias if bias is not None else 0.0)
            out[a0 + t] = acc * torch.sigmoid(acc) if act else acc
        conv_state[slot] = x[x.shape[0] - (taps - 1):]
    return out


def mamba2_prepare(proj, dt_off, dt_bias, a_log, x, heads, vdim):
    T = proj.shape[0]
    dt = torch.nn.functional.softplus(proj[:, dt_off:dt_off + heads].float() + (dt_bias if dt_bias is not None else 0.0),
                                      threshold=30.0)
    keep = torch.exp(-torch.exp(a_log) * dt)
    return keep, (x[:, :heads * vdim].reshape(T, heads, vdim) * dt[:, :, None]).reshape(T, heads * vdim)


def group_rms_norm(x, groups, n, group_stride, weight, eps, out_dtype, den_floor=None, skip=None, skip_w=None, skip_head=1,
                   pre_gate=None, post_gate=None):
    T, N = x.shape[0], groups * n
    val = torch.stack([x[:, g * group_stride:g * group_stride + n] for g in range(groups)], 1)          # [T, groups, n]
    if den_floor is not None:
        den = torch.stack([x[:, g * group_stride + n] for g in range(groups)], 1)
        val = val / (torch.maximum(den.abs(), den_floor) + 1e-6)[:, :, None]
    val = val.reshape(T, N)
    if skip is not None:
        val = val + skip_w.repeat_interleave(skip_head)[:N] * skip[:, :N]
    if pre_gate is not None:
        g = pre_gate[:, :N].float()
        val = val * g * torch.sigmoid(g)
    y = _rms_unit(val.view(T, groups, n), eps).reshape(T, N)
    if weight is not None:
        y = y * weight
    if post_gate is not None:
        y = y * torch.sigmoid(post_gate[:, :N].float())
    return y.to(out_dtype)


def whole_norm_store(proj, q_off, k_off, v_off, q_w, k_w, eps, v_norm, slots, k_pages, v_pages, heads, kv_heads, dim, vdim, row,
                     page_size):
    T = proj.shape[0]
    p = proj.float()
    q, k = p[:, q_off:q_off + heads * dim], p[:, k_off:k_off + kv_heads * dim]
    v = p[:, v_off:v_off + kv_heads * vdim].reshape(T, kv_heads, vdim)
    if q_w is not None:
        q = _rms_unit(q, eps) * q_w
    if k_w is not None:
        k = _rms_unit(k, eps) * k_w
    if v_norm:
        v = _rms_unit(v, eps)
    pad = lambda t, d: torch.cat([t, torch.zeros(t.shape[0], t.shape[1], row - d)], 2)
    q, k, v = pad(q.reshape(T, heads, dim), dim), pad(k.reshape(T, kv_heads, dim), dim), pad(v, vdim)
    if slots is not None:
        for t in range(T):
            sl = int(slots[t])
            if sl >= 0:
                k_pages[sl // page_size, :, sl % page_size, :] = k[t].to(k_pages.dtype)
                v_pages[sl // page_size, :, sl % page_size, :] = v[t].to(v_pages.dtype)
    return q.reshape(T, heads * row).to(proj.dtype)


NAMES = ["hyper_expand", "hyper_step", "scale_add_rows", "scaled_sum", "gated_linear_attention", "mlstm_prepare", "hgrn2_prepare",
         "causal_conv_silu", "mamba2_prepare", "group_rms_norm", "whole_norm_store",
         "activation", "qk_norm_rope_store", "sigmoid_gate", "decay_linear_attention", "gated_rms_norm", "post_add_norm", "scale_softcap", "latent_norm_store", "head_linear", "head_scale", "moe_route", "moe_experts",
         "embedding", "add_rmsnorm", "swiglu", "rope_store", "attention_scratch_floats", "paged_attention",
         "mma_attention_takes", "paged_attention_mma", "make_kv_tensor_map", "make_kv_tensor_map_2d", "tc_takes", "skinny_takes", "skinny_norm_takes", "skinny_linear", "skinny_linear_residual",
         "skinny_gate_up_swiglu", "skinny_qkv_rope_store",
         "linear", "logits_linear", "sample", "delta_prepare", "gated_delta_rule", "pair_rope_norm_store", "sum_add_norm",
         "gelu_gate_rows", "capped_glu"]


def delta_prepare(xc, q_off, k_off, proj, b_off, dt, dt_bias, a_log, heads, kv_heads, dim, unit_eps=1e-6):
    T, H, G, d = xc.shape[0], heads, kv_heads, dim
    q = xc[:, q_off:q_off + G * d].reshape(T, G, d)
    k = xc[:, k_off:k_off + G * d].reshape(T, G, d)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    z = dt.float() + (dt_bias if dt_bias is not None else 0.0)
    keep = torch.exp(-torch.exp(a_log).repeat_interleave(d) * torch.nn.functional.softplus(z, threshold=20.0))
    beta = torch.sigmoid(proj[:, b_off:b_off + H].float())
    return torch.cat([q.reshape(T, -1), k.reshape(T, -1), keep, beta, (q * k).sum(-1)], 1).contiguous()


def gated_delta_rule(prep, v, state, seg_slots, cu_q, positions, heads, kv_heads, dim, vdim):
    T, H, G, d = prep.shape[0], heads, kv_heads, dim
    q, k = prep[:, :G * d].reshape(T, G, d), prep[:, G * d:2 * G * d].reshape(T, G, d)
    keep = prep[:, 2 * G * d:2 * G * d + H * d].reshape(T, H, d)
    beta = prep[:, 2 * G * d + H * d:2 * G * d + H * d + H]
    out = torch.zeros(T, H * vdim)
    for s in range(seg_slots.shape[0]):
        a0, a1 = int(cu_q[s]), int(cu_q[s + 1])
        if a1 <= a0 or int(positions[a0]) < 0:
            continue
        slot = int(seg_slots[s])
        for a in range(H):
            g = a // (H // G)
            S = state[slot, a].t().clone()                       # [d, vdim]
            for t in range(a0, a1):
                S = keep[t, a][:, None] * S
                u = beta[t, a] * (v[t, a * vdim:(a + 1) * vdim] - S.t() @ k[t, g])
                S = S + torch.outer(k[t, g], u)
                out[t, a * vdim:(a + 1) * vdim] = S.t() @ q[t, g]
            state[slot, a] = S.t()
    return out


def pair_rope_norm_store(x, q_off, k_off, v_off, positions, inv_freq, norm, q_w, k_w, eps, slots, k_pages, v_pages, heads,
                         kv_heads, dim, vdim, row, page_size, out_dtype):
    T = x.shape[0]
    pos = positions.float().clamp(min=0)

    def turn(t):                                                 # [T, n, dim]
        t = t.clone()
        if inv_freq is not None and inv_freq.numel():
            r = inv_freq.shape[0]
            ang = pos[:, None] * inv_freq[None, :]
            c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
            a, b = t[..., 0:2 * r:2].clone(), t[..., 1:2 * r:2].clone()
            t[..., 0:2 * r:2] = a * c - b * s
            t[..., 1:2 * r:2] = b * c + a * s
        return t

    def finish(t, w):
        if norm:
            t = t / torch.sqrt((t * t).mean(-1, keepdim=True) + eps)
            if w is not None:
                t = t * w
        return torch.cat([t, t.new_zeros(t.shape[0], t.shape[1], row - dim)], -1)

    q = finish(turn(x[:, q_off:q_off + heads * dim].reshape(T, heads, dim)), q_w)
    k = finish(turn(x[:, k_off:k_off + kv_heads * dim].reshape(T, kv_heads, dim)), k_w)
    v = x[:, v_off:v_off + kv_heads * vdim].reshape(T, kv_heads, vdim)
    v = torch.cat([v, v.new_zeros(T, kv_heads, row - vdim)], -1)
    if slots is not None:
        for t, s in enumerate(slots.tolist()):
            if s >= 0 and int(positions[t]) >= 0:
                k_pages[s // page_size, :, s % page_size, :] = k[t].to(k_pages.dtype)
                v_pages[s // page_size, :, s % page_size, :] = v[t].to(v_pages.dtype)
    q = torch.where((positions >= 0)[:, None, None], q, torch.zeros_like(q))
    return q.reshape(T, heads * row).to(out_dtype)


def sum_add_norm(x, terms, weight, kind, eps, out, rows=None):
    src = x if rows is None else x[rows.long()]
    acc = src.clone()
    for delta, w, k, e, s in terms:
        d = (delta if rows is None else delta[rows.long()]).float()
        if k == 1:
            d = d / torch.sqrt((d * d).mean(-1, keepdim=True) + e)
            if w is not None:
                d = d * w
        acc = acc + s * d
    if rows is None:
        x.copy_(acc)
    if out is None or kind == 0:
        return out
    if kind == 1:
        acc = acc / torch.sqrt((acc * acc).mean(-1, keepdim=True) + eps) * (weight if weight is not None else 1.0)
    out.copy_(acc.to(out.dtype))
    return out


def gelu_gate_rows(z, table, off, tokens, feedback=None):
    ids = tokens.long()
    if feedback is not None:
        ids = torch.where(ids < 0, feedback.long()[(-ids - 1).clamp(min=0)], ids)
    a = z.float()
    g = 0.5 * a * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (a + 0.044715 * a ** 3)))
    return (g * table[ids.clamp(min=0), off:off + z.shape[1]].float()).to(z.dtype)


def install(monkeypatch):
    """Replaces the kernels of pico_vllm_b200.ops with the doubles above."""
    import pico_vllm_b200.ops as ops
    for name in NAMES:
        monkeypatch.setattr(ops, name, globals()[name])
