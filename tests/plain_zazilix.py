"""The Zazilix design restated in plain torch, slowly, one function per mechanism: the oracle of the tests.

Everything is float64 and works on ONE whole sequence (tokens 0 .. T-1 from empty memory); recurrences are loops over
tokens with the state written out as in the equations.  Nothing here is shared with the package: weights come as a
dictionary from tensor name to tensor, the configuration as the dictionary config.json holds.
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


def lin(w, x):
    return x @ w.T


# ----------------------------------------------------------------------------------------- mixers
def mlstm_mixer(h, w, m, eps):
    """Matrix memory with exponential gates kept finite by a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = lin(w["q"], h).view(T, H, d) * d ** -0.5
    k = lin(w["k"], h).view(T, H, d)
    v = lin(w["v"], h).view(T, H, dv)
    gi = cap * torch.tanh((lin(w["i"], h) + w["i.b"]) / cap)                                   # [T, H], a logarithm
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((lin(w["f"], h) + w["f.b"]) / cap))   # [T, H], a logarithm
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        n = torch.zeros(d, dtype=F64)
        mx = 0.0
        for t in range(T):
            new = max(float(gf[t, a]) + mx, float(gi[t, a]))
            keep, put = math.exp(float(gf[t, a]) + mx - new), math.exp(float(gi[t, a]) - new)
            S = keep * S + put * torch.outer(k[t, a], v[t, a])
            n = keep * n + put * k[t, a]
            mx = new
            den = max(abs(float(n @ q[t, a])), math.exp(-mx)) + 1e-6
            out[t, a] = (S.T @ q[t, a]) / den
    y = rms_unit(out, eps).reshape(T, H * dv) * w["norm"] * torch.sigmoid(lin(w["g"], h))
    return lin(w["o"], y)


def chunk_sink_attention(h, w, m, eps):
    """Grouped-query softmax attention without rotation: norms over the whole q and k projections, unit-norm values,
    a distance bias per head, keys of the query's own chunk only, and a sink of score 0 in the denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    chunk = (m.get("mask") or {}).get("size")
    q = (rms_unit(lin(w["q"], h), eps) * w["q.norm"]).view(T, H, d)
    k = (rms_unit(lin(w["k"], h), eps) * w["k.norm"]).view(T, G, d)
    v = rms_unit(lin(w["v"], h).view(T, G, dv), eps)
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        slope = 2.0 ** (-8.0 * (a + 1) / H)
        for i in range(T):
            lo = 0 if chunk is None else (i // chunk) * chunk
            js = torch.arange(lo, i + 1)
            s = (k[lo:i + 1, g] @ q[i, a]) * m["scale"] - slope * (i - js).to(F64)
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            out[i, a] = p @ v[lo:i + 1, g]
    return lin(w["o"], out.reshape(T, H * dv))


def hgrn2_mixer(h, w, m, eps):
    """Linear attention whose forget gate f also writes: the key is 1 - f."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(lin(w["q"], h)).view(T, H, d)
    v = lin(w["v"], h).view(T, H, dv)
    low = w["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(lin(w["f"], h) + w["f.b"])).view(T, H, d)
    out = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = f[t, a][:, None] * S + torch.outer(1.0 - f[t, a], v[t, a])
            out[t, a] = S.T @ q[t, a]
    y = (rms_unit(out, eps) * w["norm"]).reshape(T, H * dv)
    return lin(w["o"], y)


def parallel_mixer(h, w, m, eps):
    left = chunk_sink_attention(h, {k[5:]: t for k, t in w.items() if k.startswith("left.")}, m["left"], eps)
    right = hgrn2_mixer(h, {k[6:]: t for k, t in w.items() if k.startswith("right.")}, m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def mamba2_mixer(h, w, m, eps):
    """State-space layer: a short causal convolution, a decay and step size per head, a gate before a grouped norm."""
    T = h.shape[0]
    H, dv, N, G, taps, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * dv
    zxbcdt = lin(w["in"], h)
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F64), xbc])
    conv = torch.zeros_like(xbc)
    for t in range(T):
        conv[t] = (padded[t:t + taps] * w["conv"].T).sum(0) + w["conv.b"]      # the last tap is the current token's
    conv = silu(conv)
    x = conv[:, :inner].view(T, H, dv)
    B = conv[:, inner:inner + G * N].view(T, G, N)
    C = conv[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w["dt_bias"])                                            # [T, H]
    y = torch.zeros(T, H, dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(N, dv, dtype=F64)
        rate = math.exp(float(w["A_log"][a]))
        for t in range(T):
            S = math.exp(-rate * float(dt[t, a])) * S + float(dt[t, a]) * torch.outer(B[t, g], x[t, a])
            y[t, a] = S.T @ C[t, g] + w["D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return lin(w["o"], y)


MIXERS = {"mlstm": mlstm_mixer, "parallel": parallel_mixer, "mamba2": mamba2_mixer}


# ----------------------------------------------------------------------------------------- feed-forward
def gated_expert(h, gate, up, down):
    return lin(down, silu(lin(gate, h)) * lin(up, h))


def routed_feed_forward(h, w, f, return_choice=False):
    """Softmax over all router outputs; the choice adds a correction, the weights do not; the last outputs are experts
    that hand their input on; a shared expert for every token."""
    E, ident, top = f["router"]["experts"], f["router"].get("identity", 0) or 0, f["router"]["top"]
    s = torch.softmax(lin(w["router"], h), -1)                       # [T, E + ident]
    chosen = torch.topk(s + w["correction"], top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            wt = s[t, e] * f["router"]["scale"]
            if e >= E:
                out[t] += wt * h[t]
            else:
                out[t] += wt * gated_expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])
    if f.get("shared"):
        out = out + gated_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return (out, chosen) if return_choice else out


# ----------------------------------------------------------------------------------------- the model
def sub(weights, prefix):
    return {k[len(prefix):]: t.to(F64) for k, t in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also the residual stream after every layer
    (the sum of the streams when there are several)."""
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    x = weights["embed"].to(F64)[tokens] * (config.get("embedding") or {}).get("scale", 1.0)
    x = x + weights["pos"].to(F64)[:T]
    streams = config.get("streams")
    xs = x[None].repeat(streams, 1, 1) if streams else x             # [streams, T, width] or [T, width]
    layers = []
    for i, layer in enumerate(config["layers"]):
        w = sub(weights, f"l{i}.")
        subs = [(1, lambda u, layer=layer, w=w: MIXERS[layer["type"]](u, sub(w, "mix."), layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda u, layer=layer, w=w: routed_feed_forward(u, sub(w, "mlp."), layer["mlp"])))
        for q, fn in subs:
            g = w[f"norm{q}"]
            if streams:
                u = torch.einsum("s,std->td", w[f"hc{q}.in"], xs)
                y = fn(rms_unit(u, eps) * g)
                xs = torch.einsum("sr,std->rtd", w[f"hc{q}.mix"], xs) + w[f"hc{q}.out"][:, None, None] * y[None]
            else:
                xs = xs + fn(rms_unit(xs, eps) * g)
        layers.append(xs.sum(0) if streams else xs)
    x = xs.sum(0) if streams else xs
    logits = lin(weights["head"].to(F64), rms_unit(x, eps) * weights["final.norm"].to(F64))
    return (logits, torch.stack(layers)) if return_layers else logits
