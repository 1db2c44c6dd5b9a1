"""The Banazen design restated in plain torch, slowly, one function per mechanism: the oracle of the tests.

Everything is float64 and works on ONE whole sequence (tokens 0 .. T-1 from empty memory); the recurrence is a loop over
tokens with the state written out as in the equations, attention a loop over queries with an explicit list of the keys
each one sees.  Nothing here is shared with the package: weights come as a dictionary from tensor name to tensor, the
configuration as the dictionary config.json holds.
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x divided by its root mean square over the last dimension (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def lin(w, x):
    return x @ w.T


def short_conv(u, w):
    """Causal convolution per channel: u [T, C], w [C, taps]; the last tap multiplies the token itself and what lies
    before the sequence is zero."""
    T, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u])
    out = torch.zeros_like(u)
    for t in range(T):
        out[t] = (padded[t:t + taps] * w.T).sum(0)
    return out


def rotate_pairs(x, base, dims):
    """x [T, heads, d]: dimension 2i turns with 2i + 1 by position * base^(-2i / dims) for 2i < dims; the rest stays."""
    T = x.shape[0]
    out = x.clone()
    pos = torch.arange(T, dtype=F64)
    for i in range(dims // 2):
        a = pos * base ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def visible(i, window):
    """The positions query i sees: all up to itself, or with a window the last ``window`` of them."""
    lo = 0 if window is None else max(0, i - window + 1)
    return lo, i + 1


def softmax_attention(q, k, v, group, scale, window=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; head a reads key/value head a // group."""
    T, H = q.shape[:2]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for a in range(H):
        g = a // group
        for i in range(T):
            lo, hi = visible(i, window)
            p = torch.softmax((k[lo:hi, g] @ q[i, a]) * scale, 0)
            out[i, a] = p @ v[lo:hi, g]
    return out


# ----------------------------------------------------------------------------------------- mixers
def latent_attention(h, w, m, eps, latent_of=None):
    """Keys and values of every head are made from one normed vector per token; a window; no positions.  With
    ``latent_of`` the vectors of another layer are used.  Returns (output, latents)."""
    T = h.shape[0]
    H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q = lin(w["q"], h).view(T, H, d)
    c = latent_of if latent_of is not None else rms_unit(lin(w["dkv"], h), eps) * w["dkv.norm"]
    k = lin(w["uk"], c).view(T, H, d)
    v = lin(w["uv"], c).view(T, H, dv)
    window = (m.get("mask") or {}).get("size")
    o = softmax_attention(q, k, v, 1, m["scale"], window)
    return lin(w["o"], o.reshape(T, H * dv)), c


def conv_rope_attention(h, w, m, eps):
    """Grouped-query causal attention: a short convolution over q, k and v, pairs of neighbours turned by the position,
    then q and k divided by their root mean square per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(lin(w["q"], h), w["q.conv"]).view(T, H, d)
    k = short_conv(lin(w["k"], h), w["k.conv"]).view(T, G, d)
    v = short_conv(lin(w["v"], h), w["v.conv"]).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q, k = rotate_pairs(q, rot["base"], rot["dims"]), rotate_pairs(k, rot["base"], rot["dims"])
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    o = softmax_attention(q, k, v, H // G, m["scale"])
    return lin(w["o"], o.reshape(T, H * dv))


def delta_rule(q, k, v, beta, keep):
    """One head: q, k [T, d], v [T, dv], beta [T], keep [T, d].  S [d, dv] from zero: rows decay, the value the memory
    holds under k is taken off what is written, and the read sees the write."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = keep[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def gated_delta_mixer(h, w, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(lin(w["q"], h), w["q.conv"])).view(T, G, d)
    k = silu(short_conv(lin(w["k"], h), w["k.conv"])).view(T, G, d)
    v = silu(short_conv(lin(w["v"], h), w["v.conv"])).view(T, H, dv)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * d ** -0.5, unit(k)
    beta = torch.sigmoid(lin(w["b"], h))                                                   # [T, H]
    dt = softplus(lin(w["a2"], lin(w["a1"], h)) + w["dt_bias"]).view(T, H, d)
    keep = torch.exp(-torch.exp(w["A_log"])[None, :, None] * dt)                           # [T, H, d]
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        out[:, a] = delta_rule(q[:, g], k[:, g], v[:, a], beta[:, a], keep[:, a])
    gate = torch.sigmoid(lin(w["g2"], lin(w["g1"], h))).view(T, H, dv)
    y = rms_unit(out, eps) * w["norm"] * gate
    return lin(w["o"], y.reshape(T, H * dv))


def side_by_side(h, w, m, eps):
    left = conv_rope_attention(h, sub(w, "left."), m["left"], eps)
    right = gated_delta_mixer(h, sub(w, "right."), m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * w["left.out"] + rms_unit(right, eps) * w["right.out"])


# ----------------------------------------------------------------------------------------- feed-forward
def dense_feed_forward(h, w):
    return lin(w["down"], silu(lin(w["gate"], h)) * lin(w["up"], h))


def capped_expert(h, gate, up, down, limit):
    g = torch.clamp(lin(gate, h), max=limit)
    u = torch.clamp(lin(up, h), -limit, limit)
    return lin(down, g * torch.sigmoid(1.702 * g) * (u + 1.0))


def choose_experts(z, correction, top, groups, keep):
    """z [T, E] router outputs.  Returns (chosen [T, top], scores [T, E]): softmax scores; the choice is by score +
    correction, among the experts of the ``keep`` groups (of ``groups`` equal runs of neighbours) whose best such number
    is largest."""
    s = torch.softmax(z, -1)
    c = s + correction
    T, E = c.shape
    if groups and groups > 1 and keep < groups:
        best = c.view(T, groups, E // groups).max(-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        allowed = torch.zeros(T, groups, dtype=torch.bool)
        allowed[torch.arange(T)[:, None], kept] = True
        c = torch.where(allowed[:, :, None].expand(T, groups, E // groups).reshape(T, E), c, torch.full_like(c, -math.inf))
    return torch.topk(c, top, dim=-1).indices, s


def routed_feed_forward(h, w, f, return_choice=False):
    r = f["router"]
    grp = r.get("groups") or {}
    chosen, s = choose_experts(lin(w["router"], h), w["correction"], r["top"], grp.get("count", 1), grp.get("keep", 1))
    limit = f["expert"]["limit"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        es = chosen[t].tolist()
        total = sum(s[t, e] for e in es) + 1e-20
        for e in es:
            out[t] += (s[t, e] / total * r.get("scale", 1.0)) * capped_expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)
    if f.get("shared"):
        y = capped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], f["shared"]["limit"])
        out = out + torch.sigmoid(lin(w["shared.sg"], h)) * y
    return (out, chosen) if return_choice else out


def feed_forward(h, w, f):
    return dense_feed_forward(h, w) if f["kind"] == "dense" else routed_feed_forward(h, w, f)


def token_side(x, tokens, table, part, dim, w, eps):
    """What the layer adds from its own slice of a second embedding row of the token."""
    e = table[tokens][:, part * dim:(part + 1) * dim]
    y = lin(w["proj"], gelu_tanh(lin(w["gate"], x)) * e)
    return rms_unit(y, eps) * w["norm"]


# ----------------------------------------------------------------------------------------- the model
def sub(weights, prefix):
    return {k[len(prefix):]: t.to(F64) for k, t in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also the residual stream after every layer."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = weights["embed"].to(F64)[tokens] * (config.get("embedding") or {}).get("scale", 1.0)
    side = config.get("token_side")
    latents, layers = {}, []
    for i, layer in enumerate(config["layers"]):
        w = sub(weights, f"l{i}.")
        h = rms_unit(x, eps) * w["norm1"]
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, latents[i] = latent_attention(h, sub(w, "mix."), m, eps, None if src is None else latents[src])
        else:
            y = side_by_side(h, sub(w, "mix."), m, eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, sub(w, "mlp."), layer["mlp"])
        x = x + y
        if side:
            x = x + token_side(x, tokens, weights["side.embed"].to(F64), i, side["dim"], sub(w, "side."), eps)
        layers.append(x)
    logits = lin(weights["head"].to(F64), rms_unit(x, eps) * weights["final.norm"].to(F64)) * config.get("logit_scale", 1.0)
    return (logits, torch.stack(layers)) if return_layers else logits
