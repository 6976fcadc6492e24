"""Bosenex as data: its tensor names, its random initialisation, and its ModelSpec.

A pre-norm decoder whose layers differ: x + mixer(rms_norm(x)), then x + feed_forward(rms_norm(x)), with plain gains.
A layer's mixer is a matrix memory with exponential gates (parts/recurrent.py: `mlstm`) or two mixers side by side
(`side_by_side`): grouped attention with rotated queries and keys, capped scores, a sliding window, a learned sink per
head and one output gate per head (parts/attention.py: `rotary_window_attention`) beside a state-space layer with a
short convolution (`ssd`). Its feed-forward, where it has one, is a gated unit with relu (parts/mlp.py: `gated_mlp`) or a
mixture of clamped gated experts with one expert that every token uses (`routed_experts`). The token table's rows are
scaled on their way in; the head is a table of its own and the logits are scaled.

Tensor names (matrices stored [out, in]): `embed`, `head`, `final.norm`, and for layer i `l<i>.norm1`, `l<i>.norm2`
(with a feed-forward), the mixer's under `l<i>.mix.` and the feed-forward's under `l<i>.mlp.`:
  mlstm     q k v g o norm i i.b f f.b
  parallel  left.{q k v sink g o}, right.{in conv conv.b dt_bias A_log D norm o}, left.out, right.out
  dense     gate up down
  moe       e<j>.{gate up down}, router, router.b, shared.{gate up down}
"""

from __future__ import annotations

import torch

from ..config.bosenex import NAME, BosenexConfig, DenseMlp, ExpertsMlp, MatrixMemoryMixer
from ..config.registry import Architecture, register_architecture
from ..parts import LayerSpec, PartSpec, Runtime
from ..weights.loader import TensorSpec, WeightSpec
from .decoder import DecoderModel, ModelSpec

# Constants that the design fixes.
SWISH_ALPHA = 1.702   # an expert's gate is g * sigmoid(SWISH_ALPHA * g)
UP_OFFSET = 1.0       # ... times (u + UP_OFFSET)
BRANCH_SHARE = 0.5    # two mixers side by side: half the sum of their normalised outputs
# The state-holding mixers have no limit and the attention's rotation none either: the engine's options bound a sequence.
UNBOUNDED_SEQ_LEN = 1 << 30


def _mixer_names(layer, p: str) -> dict[str, tuple[str, tuple[int, ...]]]:
    """The mixer part's weight name -> (tensor name, shape)."""
    def entry(name, *shape):
        return (f"{p}.mix.{name}", tuple(shape))

    m = layer.mixer
    if isinstance(m, MatrixMemoryMixer):
        return {"w_q": entry("q", m.heads * m.dim, None), "w_k": entry("k", m.heads * m.dim, None),
                "w_v": entry("v", m.heads * m.vdim, None), "w_gate": entry("g", m.heads * m.vdim, None),
                "w_out": entry("o", None, m.heads * m.vdim), "norm": entry("norm", m.heads * m.vdim),
                "w_i": entry("i", m.heads, None), "b_i": entry("i.b", m.heads), "w_f": entry("f", m.heads, None), "b_f": entry("f.b", m.heads)}
    a, s = m.left, m.right
    inner, channels = s.heads * s.vdim, s.heads * s.vdim + 2 * s.groups * s.state
    return {
        "left.w_q": entry("left.q", a.heads * a.dim, None), "left.w_k": entry("left.k", a.kv_heads * a.dim, None),
        "left.w_v": entry("left.v", a.kv_heads * a.vdim, None), "left.sink": entry("left.sink", a.heads),
        "left.w_gate": entry("left.g", a.heads, None), "left.w_out": entry("left.o", None, a.heads * a.vdim),
        "right.w_in": entry("right.in", inner + channels + s.heads, None), "right.conv": entry("right.conv", channels, s.conv),
        "right.conv_b": entry("right.conv.b", channels), "right.dt_bias": entry("right.dt_bias", s.heads),
        "right.a_log": entry("right.A_log", s.heads), "right.d_skip": entry("right.D", s.heads),
        "right.norm": entry("right.norm", inner), "right.w_out": entry("right.o", None, inner),
        "left_out": entry("left.out", -1), "right_out": entry("right.out", -1)}


def _mlp_names(layer, p: str) -> dict[str, tuple[str, tuple[int, ...]]]:
    def unit(own: str, stored: str, ff: int):
        return {f"{own}w_gate": (f"{p}.mlp.{stored}gate", (ff, None)), f"{own}w_up": (f"{p}.mlp.{stored}up", (ff, None)),
                f"{own}w_down": (f"{p}.mlp.{stored}down", (None, ff))}

    mlp = layer.mlp
    if isinstance(mlp, DenseMlp):
        return unit("", "", mlp.ff)
    out = {"router": (f"{p}.mlp.router", (mlp.experts, None)), "router_b": (f"{p}.mlp.router.b", (mlp.experts,))}
    for j in range(mlp.experts):
        out.update(unit(f"e{j}.", f"e{j}.", mlp.ff))
    if mlp.shared_ff:
        out.update(unit("shared.", "shared.", mlp.shared_ff))
    return out


def _shaped(names: dict, width: int) -> list[TensorSpec]:
    """None in a shape stands for the model width (and -1 for a vector of it)."""
    return [TensorSpec(name, tuple(width if d in (None, -1) else d for d in shape)) for name, shape in names.values()]


def weight_spec(cfg: BosenexConfig) -> WeightSpec:
    d = cfg.width
    tensors = [TensorSpec("embed", (cfg.vocab_size, d))]
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        tensors.append(TensorSpec(f"{p}.norm1", (d,)))
        if layer.mlp is not None:
            tensors.append(TensorSpec(f"{p}.norm2", (d,)))
        tensors += _shaped(_mixer_names(layer, p), d)
        if layer.mlp is not None:
            tensors += _shaped(_mlp_names(layer, p), d)
    tensors += [TensorSpec("final.norm", (d,)), TensorSpec("head", (cfg.vocab_size, d))]
    return WeightSpec(tensors=tuple(tensors))


def random_weights(cfg: BosenexConfig, seed: int, std: float = 0.05, norm_std: float = 0.1) -> dict[str, torch.Tensor]:
    """Float32 draws from ONE CPU generator, in the order of `weight_spec`: matrices and tables N(0, std); gains 1 +
    N(0, norm_std); biases, sinks, step biases and skips N(0, 1) * a size that keeps gates and steps in their
    interesting range; decay rates spread over a decade."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for ts in weight_spec(cfg).tensors:
        draw = torch.randn(ts.shape, generator=gen, dtype=torch.float32)
        last = ts.name.rsplit(".", 1)[-1]
        if len(ts.shape) == 2 and not ts.name.endswith(".conv"):
            out[ts.name] = std * draw
        elif ts.name.endswith(".conv"):
            out[ts.name] = 0.4 * draw
        elif last in ("norm1", "norm2", "norm", "out"):
            out[ts.name] = 1.0 + norm_std * draw
        elif last == "A_log":
            out[ts.name] = 0.8 * draw - 0.5
        elif last == "D":
            out[ts.name] = 1.0 + 0.3 * draw
        elif ts.name.endswith(".f.b"):
            out[ts.name] = 2.0 + draw      # forget gates that mostly keep
        else:
            out[ts.name] = 0.5 * draw      # biases, sinks, step biases
    return out


def model_spec(cfg: BosenexConfig) -> ModelSpec:
    eps = cfg.norm_eps
    rms = {"eps": eps}
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        weights = {own: name for own, (name, _) in _mixer_names(layer, p).items()}
        if isinstance(m, MatrixMemoryMixer):
            mixer = PartSpec("mlstm", {"n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "gate_cap": m.gate_cap,
                                       "norm_eps": eps}, weights)
        else:
            a, s = m.left, m.right
            left = {"kind": "rotary_window_attention", "params": {
                "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim, "scale": a.scale,
                "softcap": a.softcap, "window": min(a.window, UNBOUNDED_SEQ_LEN), "rot_dims": a.rot_dims, "rot_base": a.rot_base}}
            right = {"kind": "ssd", "params": {
                "n_heads": s.heads, "v_head_dim": s.vdim, "n_state": s.state, "n_groups": s.groups, "conv_taps": s.conv,
                "norm_groups": s.norm_groups, "norm_eps": eps}}
            mixer = PartSpec("side_by_side", {"left": left, "right": right, "eps": eps, "share": BRANCH_SHARE}, weights)
        feed_forward = norm_2 = None
        if layer.mlp is not None:
            ff_weights = {own: name for own, (name, _) in _mlp_names(layer, p).items()}
            if isinstance(layer.mlp, DenseMlp):
                feed_forward = PartSpec("gated_mlp", {"activation": "relu"}, ff_weights)
            else:
                e: ExpertsMlp = layer.mlp
                feed_forward = PartSpec("routed_experts", {
                    "n_experts": e.experts, "top": e.top, "limit": e.limit, "alpha": SWISH_ALPHA, "up_offset": UP_OFFSET,
                    "shared_limit": e.shared_limit if e.shared_ff else None}, ff_weights)
            norm_2 = PartSpec("rms_norm", rms, {"weight": f"{p}.norm2"})
        layers.append(LayerSpec(block="pre_norm", mixer=mixer, feed_forward=feed_forward,
                                norm_1=PartSpec("rms_norm", rms, {"weight": f"{p}.norm1"}), norm_2=norm_2))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden=cfg.width, max_seq_len=UNBOUNDED_SEQ_LEN, eos_token=None,
        embedding="embed", head="head", positions=None, layers=tuple(layers),
        final_norm=PartSpec("rms_norm", {"eps": eps, "gain_scale": cfg.logit_scale}, {"weight": "final.norm"}),
        embedding_scale=cfg.embedding_scale)


def build(cfg: BosenexConfig, tensors: dict[str, torch.Tensor], rt: Runtime) -> DecoderModel:
    return DecoderModel(model_spec(cfg), tensors, rt, config=cfg)


BOSENEX = register_architecture(Architecture(
    name=NAME, parse_config=BosenexConfig.from_json, weight_spec=weight_spec, random_weights=random_weights,
    build=build, config_to_json=BosenexConfig.to_json,
))
