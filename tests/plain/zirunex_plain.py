"""A plain, slow Zirunex: whole sequences, no cache, one function per mechanism.

Written from the design's equations in this file's own notation; it shares no code with the
product package: it reads model folders with the `safetensors` library, computes with dense
torch ops on the CPU (float64 unless told otherwise) and knows nothing about pages, batches or
kernels. Tests compare the engine against it.

The model: x_0 = E[token] * s. Every layer computes h = N(x) once and adds both sublayers of h,
x <- x + A(h) + F(h) (F may be absent). N is an RMS norm whose stored weight w gives the gain
1 + w. A is grouped attention: per head, RMS-normed queries and keys (plain gains), scores
q . k * c over the keys that the mask lets a position see, a softmax whose denominator holds one
extra 1, a sigmoid gate computed from h on the heads' outputs, then the output matrix. F is a
gated unit with clamped halves. The logits are H N_f(x).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ---------------------------------------------------------------------------------------------
# mechanisms


def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """Row `token` of the table, times the embedding's scale."""
    return table[tokens.long()] * scale


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def stream_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm of the residual stream: the tensor w holds the gain's offset from one: gain 1 + w."""
    return rms(x, eps) * (1.0 + w)


def head_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm of one query or key head ([..., dim]): the stored weight is the gain itself."""
    return rms(x, eps) * g


def sees(i: int, j: int, window: int, keep_first: int) -> bool:
    """Whether position i reads position j: nothing later than itself; of the earlier ones the
    last `window` (itself included) and, whatever their distance, the first `keep_first`."""
    return j <= i and (i - j < window or j < keep_first)


def sink_softmax(scores: torch.Tensor) -> torch.Tensor:
    """exp(s_j) / (1 + sum_j exp(s_j)) over the last axis: the weights sum to less than one. Scores of
    -inf (masked) get weight 0. Computed with the largest score (or 0, the sink's) taken out."""
    top = torch.clamp(scores.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(scores - top)
    return e / (torch.exp(-top) + e.sum(dim=-1, keepdim=True))


def attention_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int, keep_first: int,
                    first_position: int = 0) -> torch.Tensor:
    """q [n, H, d], k [m, G, d], v [m, G, e] -> [n, H, e]. Row r of q stands at position
    first_position + r, row j of k and v at position j; head h reads key/value head h // (H / G)."""
    n, n_heads, _ = q.shape
    m, n_groups, _ = k.shape
    per_group = n_heads // n_groups
    mask = torch.tensor([[sees(first_position + r, j, window, keep_first) for j in range(m)] for r in range(n)])
    out = torch.zeros(n, n_heads, v.shape[-1], dtype=q.dtype)
    for h in range(n_heads):
        g = h // per_group
        s = (q[:, h] @ k[:, g].T) * scale
        s = torch.where(mask, s, torch.full_like(s, -math.inf))
        out[:, h] = sink_softmax(s) @ v[:, g]
    return out


def mixer(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """The attention sublayer on normed input h [n, D]; `w` holds the tensors, `p` the layer's prefix,
    `m` the mixer's entry of the configuration."""
    n = h.shape[0]
    n_heads, n_groups, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = head_norm((h @ w[p + "mix.q"].T).view(n, n_heads, d), w[p + "mix.q.norm"], eps)
    k = head_norm((h @ w[p + "mix.k"].T).view(n, n_groups, d), w[p + "mix.k.norm"], eps)
    v = (h @ w[p + "mix.v"].T).view(n, n_groups, e)
    heads = attention_heads(q, k, v, m["scale"], m["mask"]["size"], m["mask"]["keep_first"])
    gated = heads.reshape(n, n_heads * e) * torch.sigmoid(h @ w[p + "mix.g"].T)
    return gated @ w[p + "mix.o"].T


def gated_unit(a: torch.Tensor, b: torch.Tensor, limit: float) -> torch.Tensor:
    """a is cut off above `limit`, b on both sides; the result is a * sigmoid(1.702 a) * (b + 1)."""
    a = torch.clamp(a, max=limit)
    b = torch.clamp(b, min=-limit, max=limit)
    return a * torch.sigmoid(1.702 * a) * (b + 1.0)


def feed_forward(h: torch.Tensor, w: dict, p: str, f: dict) -> torch.Tensor:
    return gated_unit(h @ w[p + "mlp.gate"].T, h @ w[p + "mlp.up"].T, f["limit"]) @ w[p + "mlp.down"].T


# ---------------------------------------------------------------------------------------------
# the model


def read_model(folder, dtype=torch.float64):
    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {name: t.to(dtype) for name, t in load_file(str(folder / "model.safetensors")).items()}
    return w, cfg


def forward(w: dict, cfg: dict, tokens, keep_layers: list | None = None) -> torch.Tensor:
    """Logits [n, V] of one whole sequence. `keep_layers` collects the stream after every layer."""
    tokens = torch.as_tensor(tokens)
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w["embed"], cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h = stream_norm(x, w[p + "norm1"], eps)
        add = mixer(h, w, p, layer["mixer"], eps)
        if layer["mlp"] is not None:
            add = add + feed_forward(h, w, p, layer["mlp"])
        x = x + add
        if keep_layers is not None:
            keep_layers.append(x.clone())
    return stream_norm(x, w["final.norm"], eps) @ w["head"].T


def generate(w: dict, cfg: dict, prompt: list[int], n_new: int) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token (first index on ties)."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(w, cfg, seq)[-1].argmax()))
    return seq[len(prompt):]
