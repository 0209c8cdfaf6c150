"""A plain, slow implementation of the Selivik design in float64, one function
per mechanism, written from the design's equations.  It shares no code with the
engine: the tests compare the two.

A model is (config dict, {tensor name: tensor}).  Sequences are handled one at
a time and whole: position t sees what the design lets it see of positions 0..t.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """The layers' norm: its stored weight is the gain's distance from one."""
    return rms(x, eps) * (1.0 + w)


def embed(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def frequencies(base, dims, factor=1.0):
    """f_i = base^(-2i/dims) / factor for i < dims/2."""
    i = torch.arange(dims // 2, dtype=F64)
    return torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims) / float(factor)


def _turn(u, v, positions, freqs, lead):
    ang = positions.to(F64)[:, None] * freqs[None, :]
    shape = [u.shape[0]] + [1] * lead + [freqs.numel()]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    return u * c - v * s, v * c + u * s


def rotate_halves(x, positions, freqs):
    """x [T, ..., dim]: entry i pairs with entry i + n (n = len(freqs)); entries from 2n on stay."""
    n = freqs.numel()
    out = x.clone()
    if n:
        out[..., :n], out[..., n:2 * n] = _turn(x[..., :n], x[..., n:2 * n], positions, freqs, x.dim() - 2)
    return out


def rotate_neighbours(x, positions, freqs):
    """x [T, ..., dim]: entry 2i pairs with entry 2i + 1 for i < len(freqs); the rest stays."""
    n = freqs.numel()
    out = x.clone()
    if n:
        out[..., 0:2 * n:2], out[..., 1:2 * n:2] = _turn(x[..., 0:2 * n:2], x[..., 1:2 * n:2], positions, freqs,
                                                        x.dim() - 2)
    return out


def softmax_seen(s, seen, sink=None):
    """Softmax over the entries of each row of s [T, T] that ``seen`` marks; ``sink`` (a number) puts
    exp(sink) into the denominator as well."""
    s = s.masked_fill(~seen, -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.clamp(top, min=float(sink))
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(torch.as_tensor(float(sink), dtype=F64) - top)
    return e / den


def causal(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


def window_with_first(T, size, keep_first):
    """Row i marks j <= i with i - j < size or j < keep_first."""
    i = torch.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & ((d < size) | (i[None, :] < keep_first))


def latent_attention(h, W, p, m, eps):
    """h [T, width]; W the model's tensors, p the mixer's prefix ('l3.mix.'), m its sizes."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, dn + dr)
    both = h @ W[p + "dkv"].T
    c = rms(both[:, :r], eps) * W[p + "dkv.norm"]
    f = frequencies(m["rot"]["base"], m["rot"]["dims"])
    k_turned = rotate_neighbours(both[:, r:], pos, f)                       # [T, dr], one for all heads
    q_turned = rotate_neighbours(q[..., dn:], pos, f)                       # [T, H, dr]
    k_plain = (c @ W[p + "uk"].T).reshape(T, H, dn)
    v = (c @ W[p + "uv"].T).reshape(T, H, dv)
    seen = causal(T)
    out = torch.zeros(T, H, dv, dtype=F64)
    for n in range(H):
        s = (q[:, n, :dn] @ k_plain[:, n].T + q_turned[:, n] @ k_turned.T) * m["scale"]
        out[:, n] = softmax_seen(s, seen) @ v[:, n]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def attention(h, W, p, m, eps):
    T = h.shape[0]
    H, G, dim, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, dim)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, dim)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    rot = m["rot"]
    f = frequencies(rot["base"], rot["dims"], (rot.get("scaling") or {}).get("factor", 1.0))
    q, k = rms(rotate_halves(q, pos, f), eps), rms(rotate_halves(k, pos, f), eps)
    mask = m.get("mask")
    seen = window_with_first(T, mask["size"], mask.get("keep_first", 0)) if mask else causal(T)
    cap = m.get("softcap")
    out = torch.zeros(T, H, dv, dtype=F64)
    for n in range(H):
        g = n // (H // G)
        s = (q[:, n] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        out[:, n] = softmax_seen(s, seen, float(W[p + "sink"][n])) @ v[:, g]
    return out.reshape(T, H * dv) @ W[p + "o"].T


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_unit(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, top):
    """(chosen experts [T, top], their weights [T, top]): the largest logits win, the weights are the
    softmax over the winners' logits alone."""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    best = torch.topk(z, top, dim=-1)
    return best.indices, torch.softmax(best.values, dim=-1)


def experts(h, W, p, f):
    top = f["router"]["top"]
    idx, wts = route(h, W, p, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            q = f"{p}e{e}."
            z = h[t] @ W[q + "gate"].T
            out[t] += wts[t, c] * ((z * torch.sigmoid(z) * (h[t] @ W[q + "up"].T)) @ W[q + "down"].T)
    return out


MIXERS = {"latent_attention": latent_attention, "attention": attention}


def forward(cfg, W, tokens, streams=False):
    """Logits [T, vocab] of one sequence; with ``streams`` also the residual stream behind every layer."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = embed(tokens, W["embed"], float((cfg.get("embedding") or {}).get("scale", 1.0)))
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_around_zero(x, W[p + "norm1"], eps)
        y = MIXERS[layer["type"]](h, W, p + "mix.", layer["mixer"], eps) * W[p + "ls1"]
        f = layer.get("mlp")
        if f is not None:
            ff = dense_unit(h, W, p + "mlp.") if f["kind"] == "dense" else experts(h, W, p + "mlp.", f)
            y = y + ff * W[p + "ls2"]
        x = x + mult * y
        after.append(x)
    logits = norm_around_zero(x, W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(after)) if streams else logits
