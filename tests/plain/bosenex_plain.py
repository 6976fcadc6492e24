"""Bosenex, stated plainly: one function per mechanism, float64, a Python loop per token where the
design has a recurrence. Nothing here is shared with the engine; the tests compare the engine with it.

A model is a dict of tensors by checkpoint name and the config.json dict. Notation: h [T, D] is a
sublayer's input, rows are the positions 0 .. T - 1 of ONE sequence.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


def lin(w, h):
    """Matrices are stored [out, in]."""
    return h @ w.to(F64).T


def soft_cap(x, cap):
    return cap * torch.tanh(x / cap)


# ---- matrix memory with exponential gates ------------------------------------------------------
def mlstm(h, w, p, cfg, eps):
    """w: tensors under '<layer>.mix.' by their last names. cfg: heads, dim, vdim, gate_cap."""
    H, dk, dv, cap = cfg["heads"], cfg["dim"], cfg["vdim"], float(cfg["gate_cap"])
    T = h.shape[0]
    q = lin(w[p + "q"], h).view(T, H, dk) * dk ** -0.5
    k = lin(w[p + "k"], h).view(T, H, dk)
    v = lin(w[p + "v"], h).view(T, H, dv)
    log_i = soft_cap(lin(w[p + "i"], h) + w[p + "i.b"].to(F64), cap)                                   # [T, H]
    log_f = torch.nn.functional.logsigmoid(soft_cap(lin(w[p + "f"], h) + w[p + "f.b"].to(F64), cap))
    S = torch.zeros(H, dk, dv, dtype=F64)
    n = torch.zeros(H, dk, dtype=F64)
    m = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(log_f[t] + m, log_i[t])
        keep = torch.exp(log_f[t] + m - m_new)
        take = torch.exp(log_i[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    out = rms(out, eps).reshape(T, H * dv) * w[p + "norm"].to(F64)
    out = out * torch.sigmoid(lin(w[p + "g"], h))
    return lin(w[p + "o"], out)


# ---- attention: rotation, capped scores, sliding window, sink, per-head gate -------------------
def rotate(x, positions, dims, base):
    """x [T, heads, dim]: the first `dims` of a head are rotated, dimension i with i + dims / 2."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def window_attention(h, w, p, cfg):
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = lin(w[p + "q"], h).view(T, H, dk)
    k = lin(w[p + "k"], h).view(T, G, dk)
    v = lin(w[p + "v"], h).view(T, G, dv)
    rot = cfg.get("rot")
    if rot is not None:
        q, k = rotate(q, pos, rot["dims"], rot["base"]), rotate(k, pos, rot["dims"], rot["base"])
    size = cfg["mask"]["size"] if cfg.get("mask") else None
    sink = w[p + "sink"].to(F64)
    gate = torch.sigmoid(lin(w[p + "g"], h))                                    # [T, H]
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * cfg["scale"]
        if cfg.get("softcap") is not None:
            s = soft_cap(s, float(cfg["softcap"]))
        d = pos[:, None] - pos[None, :]
        seen = d >= 0
        if size is not None:
            seen = seen & (d < size)
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, sink[hd])
        e = torch.exp(s - top)
        weights = e / (e.sum(-1, keepdim=True) + torch.exp(sink[hd] - top))
        out[:, hd] = (weights @ v[:, g]) * gate[:, hd: hd + 1]
    return lin(w[p + "o"], out.reshape(T, H * dv))


# ---- state-space mixer with a short convolution -------------------------------------------------
def ssd(h, w, p, cfg, eps):
    Hn, dv, N, G, taps, parts = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"], cfg["conv"], cfg["norm_groups"]
    inner, T = Hn * dv, h.shape[0]
    u = lin(w[p + "in"], h)
    z, xbc, dt = u[:, :inner], u[:, inner: 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    conv, bias = w[p + "conv"].to(F64), w[p + "conv.b"].to(F64)
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F64), xbc])
    mixed = torch.stack([(padded[t: t + taps].T * conv).sum(-1) for t in range(T)]) + bias
    mixed = mixed * torch.sigmoid(mixed)
    x = mixed[:, :inner].view(T, Hn, dv)
    B = mixed[:, inner: inner + G * N].view(T, G, N)
    Cm = mixed[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"].to(F64))            # [T, heads]
    rate = torch.exp(w[p + "A_log"].to(F64))
    D = w[p + "D"].to(F64)
    S = torch.zeros(Hn, N, dv, dtype=F64)
    y = torch.zeros(T, Hn, dv, dtype=F64)
    group = torch.arange(Hn) // (Hn // G)
    for t in range(T):
        decay = torch.exp(-rate * dt[t])
        S = decay[:, None, None] * S + dt[t][:, None, None] * B[t][group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, Cm[t][group]) + D[:, None] * x[t]
    y = y.reshape(T, inner) * (z * torch.sigmoid(z))
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"].to(F64)
    return lin(w[p + "o"], y)


def side_by_side(h, w, p, cfg, eps):
    left = window_attention(h, w, p + "left.", cfg["left"])
    right = ssd(h, w, p + "right.", cfg["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"].to(F64), eps) + rms_norm(right, w[p + "right.out"].to(F64), eps))


# ---- feed-forwards ----------------------------------------------------------------------------
def dense_ff(h, w, p):
    return lin(w[p + "down"], torch.relu(lin(w[p + "gate"], h)) * lin(w[p + "up"], h))


def clamped_expert(h, w, p, limit):
    g = torch.clamp(lin(w[p + "gate"], h), max=limit)
    u = torch.clamp(lin(w[p + "up"], h), -limit, limit)
    return lin(w[p + "down"], g * torch.sigmoid(1.702 * g) * (u + 1))


def route(h, w, p, top):
    """-> (chosen experts [T, top], their weights [T, top])."""
    z = lin(w[p + "router"], h) + w[p + "router.b"].to(F64)
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h, w, p, cfg):
    idx, weight = route(h, w, p, cfg["router"]["top"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), weight[t]):
            out[t] += a * clamped_expert(h[t: t + 1], w, f"{p}e{e}.", cfg["expert"]["limit"])[0]
    if cfg.get("shared") is not None:
        out = out + clamped_expert(h, w, p + "shared.", cfg["shared"]["limit"])
    return out


# ---- the model ---------------------------------------------------------------------------------
def forward(config: dict, w: dict, tokens, layers_out: list | None = None):
    """Logits [T, vocab] of one sequence from its start; `layers_out` collects the stream after every layer."""
    eps = config["norm"]["eps"]
    scale = config["embedding"]["scale"] if config.get("embedding") else 1.0
    x = w["embed"].to(F64)[torch.tensor(tokens)] * scale
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"].to(F64), eps)
        if layer["type"] == "mlstm":
            x = x + mlstm(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + side_by_side(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"].to(F64), eps)
            x = x + (dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp))
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms_norm(x, w["final.norm"].to(F64), eps)
    return lin(w["head"], x) * config.get("logit_scale", 1.0)
