"""Zirunex as data: its tensor names, its random initialisation, and its ModelSpec.

A decoder of parallel blocks, x + mixer(h) + feed_forward(h) with h = rms_norm(x), whose norms' weights
hold the gain's offset from one (gain 1 + w). The token table's rows are scaled on their way in; the head is a
table of its own. A layer's mixer is grouped attention with query/key norms, a window that keeps the
first tokens, a sink and an output gate (parts/attention.py: `qk_norm_attention`); its feed-forward, where
it has one, is the gated form with clamped projections (parts/mlp.py: `gated_clamped`). A layer may run
with the tensors of an earlier layer and a cache of its own: the schedule then names that layer again.

Tensor names: `embed`, `head`, `final.norm`, and for a layer i that owns its tensors `l<i>.norm1`,
`l<i>.mix.{q,k,v,g,o}`, `l<i>.mix.q.norm`, `l<i>.mix.k.norm`, `l<i>.mlp.{gate,up,down}`; matrices are stored
[out, in].
"""

from __future__ import annotations

import torch

from ..config.registry import Architecture, register_architecture
from ..config.zirunex import NAME, ZirunexConfig
from ..parts import LayerSpec, PartSpec, Runtime
from ..weights.loader import TensorSpec, WeightSpec
from .decoder import DecoderModel, ModelSpec, ScheduleEntry

# Constants that the design fixes.
SWISH_ALPHA = 1.702   # the feed-forward's gate is g * sigmoid(SWISH_ALPHA * g)
UP_OFFSET = 1.0       # ... times (u + UP_OFFSET)
# Positions enter nothing but the mask, so a sequence may be as long as the engine's options allow.
UNBOUNDED_SEQ_LEN = 1 << 30


def _layer_tensors(cfg: ZirunexConfig, i: int) -> list[TensorSpec]:
    layer, d, p = cfg.layers[i], cfg.width, f"l{i}"
    m = layer.mixer
    out = [
        TensorSpec(f"{p}.norm1", (d,)),
        TensorSpec(f"{p}.mix.q", (m.heads * m.dim, d)), TensorSpec(f"{p}.mix.k", (m.kv_heads * m.dim, d)),
        TensorSpec(f"{p}.mix.v", (m.kv_heads * m.vdim, d)),
        TensorSpec(f"{p}.mix.q.norm", (m.dim,)), TensorSpec(f"{p}.mix.k.norm", (m.dim,)),
        TensorSpec(f"{p}.mix.g", (m.heads * m.vdim, d)), TensorSpec(f"{p}.mix.o", (d, m.heads * m.vdim)),
    ]
    if layer.mlp is not None:
        f = layer.mlp.ff
        out += [TensorSpec(f"{p}.mlp.gate", (f, d)), TensorSpec(f"{p}.mlp.up", (f, d)), TensorSpec(f"{p}.mlp.down", (d, f))]
    return out


def weight_spec(cfg: ZirunexConfig) -> WeightSpec:
    tensors = [TensorSpec("embed", (cfg.vocab_size, cfg.width))]
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is None:
            tensors += _layer_tensors(cfg, i)
    tensors += [TensorSpec("final.norm", (cfg.width,)), TensorSpec("head", (cfg.vocab_size, cfg.width))]
    return WeightSpec(tensors=tuple(tensors))


def random_weights(cfg: ZirunexConfig, seed: int, std: float = 0.05, norm_std: float = 0.1) -> dict[str, torch.Tensor]:
    """Float32 draws from ONE CPU generator, in the order of `weight_spec`: matrices and tables N(0, std),
    norm weights N(0, norm_std) (offsets from a gain of one), query/key gains 1 + N(0, norm_std)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for ts in weight_spec(cfg).tensors:
        draw = torch.randn(ts.shape, generator=gen, dtype=torch.float32)
        if ts.name.endswith(".q.norm") or ts.name.endswith(".k.norm"):
            out[ts.name] = 1.0 + norm_std * draw
        elif len(ts.shape) == 1:
            out[ts.name] = norm_std * draw
        else:
            out[ts.name] = std * draw
    return out


def model_spec(cfg: ZirunexConfig) -> ModelSpec:
    rms = {"eps": cfg.norm_eps, "unit_offset": True}
    layers: list[LayerSpec | None] = []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            layers.append(None)
            continue
        m, p = layer.mixer, f"l{i}"
        mixer = PartSpec(
            "qk_norm_attention",
            {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim, "scale": m.scale,
             "window": min(m.window, UNBOUNDED_SEQ_LEN), "keep_first": min(m.keep_first, UNBOUNDED_SEQ_LEN), "sink": True, "qk_norm_eps": cfg.norm_eps,
             "qk_norm_unit_offset": False},
            {"w_q": f"{p}.mix.q", "w_k": f"{p}.mix.k", "w_v": f"{p}.mix.v", "w_gate": f"{p}.mix.g", "w_out": f"{p}.mix.o",
             "q_norm": f"{p}.mix.q.norm", "k_norm": f"{p}.mix.k.norm"})
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec(
                "gated_clamped", {"limit": layer.mlp.limit, "alpha": SWISH_ALPHA, "up_offset": UP_OFFSET},
                {"w_gate": f"{p}.mlp.gate", "w_up": f"{p}.mlp.up", "w_down": f"{p}.mlp.down"})
        layers.append(LayerSpec(block="parallel", mixer=mixer, feed_forward=feed_forward,
                                norm_1=PartSpec("rms_norm", rms, {"weight": f"{p}.norm1"}), norm_2=None))
    # the parts list holds the layers that own tensors; the schedule runs every configured layer, a borrower
    # as its lender's parts with a cache member of its own
    index, owned = {}, []
    for i, spec in enumerate(layers):
        if spec is not None:
            index[i] = len(owned)
            owned.append(spec)
    schedule = tuple(ScheduleEntry(layer=index[cfg.owner(i)], cache=i, writes_cache=True) for i in range(len(cfg.layers)))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden=cfg.width, max_seq_len=UNBOUNDED_SEQ_LEN, eos_token=None,
        embedding="embed", head="head", positions=None, layers=tuple(owned),
        final_norm=PartSpec("rms_norm", rms, {"weight": "final.norm"}), schedule=schedule,
        embedding_scale=cfg.embedding_scale)


def build(cfg: ZirunexConfig, tensors: dict[str, torch.Tensor], rt: Runtime) -> DecoderModel:
    return DecoderModel(model_spec(cfg), tensors, rt, config=cfg)


ZIRUNEX = register_architecture(Architecture(
    name=NAME, parse_config=ZirunexConfig.from_json, weight_spec=weight_spec, random_weights=random_weights,
    build=build, config_to_json=ZirunexConfig.to_json,
))
