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


# A test may set this to a function that disturbs every normalised row on its way into a sublayer (and into the
# head): how far the logits of a position move under small disturbances says how well-conditioned the position is
# (a router's close call, a matrix memory whose first q . k is nearly zero).
DISTURB = None
# A test may set this to a list: every router then appends, per position, the margin of its choice.
MARGINS = None


def rms_norm(x, w, eps):
    out = rms(x, eps) * w
    return out if DISTURB is None else DISTURB(out)


def lin(w, h):
    """Matrices are stored [out, in]."""
    return h @ w.to(F64).T


def soft_cap(x, cap):
    return x if not cap else cap * torch.tanh(x / cap)


# ---- matrix memory with exponential gates ------------------------------------------------------
def mlstm_cells(q, k, v, log_i, log_f):
    """The recurrence alone. q (already scaled), k [T, H, dk], v [T, H, dv], log gates [T, H] -> [T, H, dv]."""
    T, H, dk = k.shape
    dv = v.shape[-1]
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
    return out


def mlstm(h, w, p, cfg, eps):
    """w: tensors under '<layer>.mix.' by their last names. cfg: heads, dim, vdim, gate_cap."""
    H, dk, dv, cap = cfg["heads"], cfg["dim"], cfg["vdim"], cfg.get("gate_cap")
    T = h.shape[0]
    q = lin(w[p + "q"], h).view(T, H, dk) * dk ** -0.5
    k = lin(w[p + "k"], h).view(T, H, dk)
    v = lin(w[p + "v"], h).view(T, H, dv)
    log_i = soft_cap(lin(w[p + "i"], h) + w[p + "i.b"].to(F64), cap)                                   # [T, H]
    log_f = torch.nn.functional.logsigmoid(soft_cap(lin(w[p + "f"], h) + w[p + "f.b"].to(F64), cap))
    out = mlstm_cells(q, k, v, log_i, log_f)
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


def attention_core(q, k, v, scale, softcap, size, sink, first_row=0):
    """q [R, H, dk]: the queries of the positions first_row .. first_row + R - 1; k [n, G, dk], v [n, G, dv]: the keys and
    values of the positions 0 .. n - 1. sink [H] or None. -> [R, H, dv]."""
    R, H, _ = q.shape
    n, G, dv = v.shape
    rows = first_row + torch.arange(R)
    d = rows[:, None] - torch.arange(n)[None, :]
    seen = d >= 0
    if size is not None:
        seen = seen & (d < size)
    out = torch.zeros(R, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale
        if softcap:
            s = soft_cap(s, float(softcap))
        s = s.masked_fill(~seen, -math.inf)
        top = s.max(-1, keepdim=True).values
        extra = 0.0
        if sink is not None:
            top = torch.maximum(top, sink[hd])
            extra = torch.exp(sink[hd] - top)
        e = torch.exp(s - top)
        out[:, hd] = (e / (e.sum(-1, keepdim=True) + extra)) @ v[:, g]
    return out


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
    out = attention_core(q, k, v, cfg["scale"], cfg.get("softcap"), size, w[p + "sink"].to(F64))
    out = out * torch.sigmoid(lin(w[p + "g"], h))[:, :, None]               # one gate per head
    return lin(w[p + "o"], out.reshape(T, H * dv))


# ---- state-space mixer with a short convolution -------------------------------------------------
def ssd_cells(x, B, Cm, dt, rate, D):
    """The recurrence alone. x [T, heads, dv], B and Cm [T, groups, N], dt [T, heads] (after softplus), rate and D [heads]."""
    T, Hn, dv = x.shape
    G, N = B.shape[1], B.shape[2]
    S = torch.zeros(Hn, N, dv, dtype=F64)
    y = torch.zeros(T, Hn, dv, dtype=F64)
    group = torch.arange(Hn) // (Hn // G)
    for t in range(T):
        decay = torch.exp(-rate * dt[t])
        S = decay[:, None, None] * S + dt[t][:, None, None] * B[t][group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, Cm[t][group]) + D[:, None] * x[t]
    return y


def causal_conv_silu(xbc, conv, bias):
    """xbc [T, C], conv [C, taps] (the last column is the current token's), zeros before the start."""
    taps, T = conv.shape[1], xbc.shape[0]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F64), xbc])
    mixed = torch.stack([(padded[t: t + taps].T * conv).sum(-1) for t in range(T)]) + bias
    return mixed * torch.sigmoid(mixed)


def ssd(h, w, p, cfg, eps):
    Hn, dv, N, G, parts = cfg["heads"], cfg["vdim"], cfg["state"], cfg.get("groups", 1), cfg.get("norm_groups", 1)
    inner, T = Hn * dv, h.shape[0]
    u = lin(w[p + "in"], h)
    z, xbc, dt = u[:, :inner], u[:, inner: 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    conv, bias = w[p + "conv"].to(F64), w[p + "conv.b"].to(F64)
    mixed = causal_conv_silu(xbc, conv, bias)
    x = mixed[:, :inner].view(T, Hn, dv)
    B = mixed[:, inner: inner + G * N].view(T, G, N)
    Cm = mixed[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"].to(F64))            # [T, heads]
    rate = torch.exp(w[p + "A_log"].to(F64))
    D = w[p + "D"].to(F64)
    y = ssd_cells(x, B, Cm, dt, rate, D)
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
    if MARGINS is not None and top < z.shape[1]:
        # how far the last chosen logit lies above the first one not chosen, in units of |h| |w|
        ranked = torch.sort(z, dim=-1, descending=True).values
        MARGINS.append((ranked[:, top - 1] - ranked[:, top]) / (h.norm(dim=-1) * w[p + "router"].to(F64).norm(dim=-1).max()))
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


def read_model(folder):
    """(config.json as a dict, tensors by name in float64)."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), {n: t.to(F64) for n, t in load_file(str(folder / "model.safetensors")).items()}


def generate(config: dict, w: dict, prompt: list[int], n_new: int) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token (first index on ties)."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(config, w, seq)[-1].argmax()))
    return seq[len(prompt):]
