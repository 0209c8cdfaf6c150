"""A plain, slow implementation of the Sisadra design in float64, one function
per mechanism, written from the design's equations.  It shares no code with the
engine: the tests compare the two.

A model is (config dict, {tensor name: tensor}).  Sequences are handled one at
a time and whole: position t sees what the design lets it see of positions 0..t.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, gain, eps):
    """(x - mean) / sqrt(var + eps) * gain over the last axis; var is the mean squared deviation."""
    c = x - x.mean(-1, keepdim=True)
    return c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * gain


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def embed(tokens, table, scale, bigram=None, buckets=0, mul_prev=0, mul_cur=0):
    """Row of the token times ``scale``; with a pair table plus a row of it chosen by a hash of
    (token before, token); the first token of a sequence takes the table's last row."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = table[ids] * scale
    if bigram is None:
        return x
    rows = torch.empty_like(ids)
    rows[0] = buckets
    rows[1:] = (ids[:-1] * mul_prev + ids[1:] * mul_cur) % buckets
    return x + bigram[rows]


def stretched_frequencies(base, dims, scaling):
    """f_i = base^(-2i/dims); with ``scaling`` (factor, low, high, original) long wavelengths are
    stretched: wavelengths below original/high keep f, those above original/low get f/factor,
    between the two the blend moves linearly in original/wavelength."""
    i = torch.arange(dims // 2, dtype=F64)
    f = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for n in range(f.numel()):
        wl = 2.0 * math.pi / float(f[n])
        if wl < orig / high:
            continue
        if wl > orig / low:
            out[n] = f[n] / factor
        else:
            s = (orig / wl - low) / (high - low)
            out[n] = (1.0 - s) * f[n] / factor + s * f[n]
    return out


def rotate_halves(x, positions, freqs):
    """x [T, ..., dim]: entry i is paired with entry i + n (n = len(freqs)) and the pair is turned by
    position * freqs[i]; entries from 2n on stay."""
    n = freqs.numel()
    if n == 0:
        return x
    ang = positions.to(F64)[:, None] * freqs[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., :n], x[..., n:2 * n]
    out = x.clone()
    out[..., :n] = u * c - v * s
    out[..., n:2 * n] = v * c + u * s
    return out


def softmax_rows(s, seen, sink=None):
    """Softmax over the entries of each row of ``s`` that ``seen`` marks; ``sink`` adds exp(sink)
    to the denominator."""
    s = torch.where(seen, s, torch.full_like(s, -math.inf))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, torch.full_like(m, float(sink)))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + math.exp(float(sink)) / torch.exp(m)
    return e / den


def differential_attention(h, w, m, eps):
    """Two softmax maps per head over the same values, o = a1 - lambda * a2, then an RMS norm per head
    without gain times (1 - diff).  Position i sees j <= i of its own chunk of ``mask.size`` positions."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    diff = float(m["diff"])
    pos = torch.arange(T)
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, 2, dim)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, 2, dim)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, vdim)
    q = rms(q, eps) * w["q.norm"]
    k = rms(k, eps) * w["k.norm"]
    rot = m.get("rot")
    if rot:
        f = stretched_frequencies(rot["base"], int(rot["dims"]), rot.get("scaling"))
        q, k = rotate_halves(q, pos, f), rotate_halves(k, pos, f)
    i, j = pos[:, None], pos[None, :]
    seen = j <= i
    size = (m.get("mask") or {}).get("size")
    if size:
        seen = seen & (i // size == j // size)
    lam = math.exp(float((w["lq1"] * w["lk1"]).sum())) - math.exp(float((w["lq2"] * w["lk2"]).sum())) + diff
    out = torch.zeros(T, H, vdim, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        a = [softmax_rows((q[:, hd, n] @ k[:, g, n].T) * m["scale"], seen) @ v[:, g] for n in (0, 1)]
        out[:, hd] = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    return out.reshape(T, H * vdim) @ w["o"].T + w["o.b"]


def latent_attention(h, w, m, eps):
    """Keys and values of every head derive from one normed latent per position; causal; the softmax
    has a learned sink per head."""
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, dim)
    c = rms(h @ w["dkv"].T, eps) * w["dkv.norm"]
    k = (c @ w["uk"].T).reshape(T, H, dim)
    v = (c @ w["uv"].T).reshape(T, H, vdim)
    pos = torch.arange(T)
    seen = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, vdim, dtype=F64)
    for hd in range(H):
        p = softmax_rows((q[:, hd] @ k[:, hd].T) * m["scale"], seen, sink=w["sink"][hd])
        out[:, hd] = p @ v[:, hd]
    return out.reshape(T, H * vdim) @ w["o"].T


def causal_conv_silu(x, taps):
    """x [T, C], taps [C, K] (the last tap on the current token, zeros before the start), then silu."""
    T, K = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=x.dtype), x], 0)
    y = sum(padded[n:n + T] * taps[:, n] for n in range(K))
    return y * torch.sigmoid(y)


def delta_rule(q, k, v, beta, decay):
    """One head: q, k [T, dim], v [T, vdim], beta [T], decay [T, dim].  S starts at zero;
    S <- decay * S (per key channel); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, dim = q.shape
    S = torch.zeros(dim, v.shape[1], dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = decay[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def channel_delta(h, w, m, eps):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w["q"].T, w["q.conv"]).reshape(T, G, dim)
    k = causal_conv_silu(h @ w["k"].T, w["k.conv"]).reshape(T, G, dim)
    v = causal_conv_silu(h @ w["v"].T, w["v.conv"]).reshape(T, H, vdim)
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q, k = unit(q) * dim ** -0.5, unit(k)
    beta = torch.sigmoid(h @ w["b"].T)
    a = (h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]
    decay = torch.exp(-torch.exp(w["A_log"])[None, :, None] * torch.nn.functional.softplus(a).reshape(T, H, dim))
    gate = torch.sigmoid((h @ w["g1"].T) @ w["g2"].T).reshape(T, H, vdim)
    out = torch.zeros(T, H, vdim, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd] = delta_rule(q[:, g], k[:, g], v[:, hd], beta[:, hd], decay[:, hd])
    out = rms(out, eps) * w["norm"] * gate
    return out.reshape(T, H * vdim) @ w["o"].T


def dense_mlp(h, w):
    z = h @ w["up"].T
    return (0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))) @ w["down"].T


MIXERS = {"attention": differential_attention, "latent_attention": latent_attention, "channel_delta": channel_delta}


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, want=None, layers_out=None):
    """Logits [len(want) or T, vocab] of one sequence; ``layers_out`` (a list) receives the
    stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    e = cfg.get("embedding") or {}
    b = e.get("bigram")
    if b is None:
        x = embed(tokens, tensors["embed"].to(F64), float(e.get("scale", 1.0)))
    else:
        x = embed(tokens, tensors["embed"].to(F64), float(e.get("scale", 1.0)), tensors["bigram"].to(F64),
                  int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"]))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, tensors[p + "norm1"].to(F64), eps)
        x = x + MIXERS[layer["type"]](h, sub(tensors, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            h = layer_norm(x, tensors[p + "norm2"].to(F64), eps)
            x = x + dense_mlp(h, sub(tensors, p + "mlp."))
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, tensors["final.norm"].to(F64), eps)
    if want is not None:
        x = x[torch.as_tensor(want, dtype=torch.long)]
    z = x @ tensors["head"].to(F64).T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap else z
