"""The typed Zirunex configuration, read from the design's own config.json keys.

A Zirunex config.json names its model with `"architecture": "Zirunex"` and lists its layers one
by one: every entry of `layers` gives the layer's `type` (which mixer it has), the mixer's sizes
and constants (`mixer`), its feed-forward (`mlp`, or null for a layer without one), and
optionally `weights_of: j` for a layer that runs with layer j's tensors and a cache of its own.
Beside the layers stand `vocab`, `width`, `norm.eps` and `embedding.scale`. No size has a default
here: a size that is missing is an error that names it. A mechanism that a file does not mention
is not there: no `mlp` is no feed-forward, no `mask` (or no `mask.size`) is no window, no
`mask.keep_first` is no kept token, no `embedding` is a scale of one; `kv_heads` and `vdim` left out
equal `heads` and `dim`. The design has no limit on a sequence's length (positions enter nothing but
the mask), so the configuration has none.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

from .registry import ConfigError

NAME = "Zirunex"
NO_WINDOW = 1 << 30  # a window that no sequence reaches: every earlier position is seen
MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense",)


def _get(data: dict, key: str, where: str):
    if not isinstance(data, dict) or key not in data:
        raise ConfigError(f"config.json: required key {where}{key!r} is missing")
    return data[key]


def _int(data: dict, key: str, where: str, minimum: int = 1) -> int:
    value = _get(data, key, where)
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: {where}{key!r} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: {where}{key!r} must be >= {minimum}, got {value}")
    return value


def _number(data: dict, key: str, where: str, positive: bool = True) -> float:
    value = _get(data, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ConfigError(f"config.json: {where}{key!r} must be a finite number, got {value!r}")
    if positive and value <= 0:
        raise ConfigError(f"config.json: {where}{key!r} must be positive, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class AttentionMixer:
    """Grouped attention with query/key norms, a window that keeps the first tokens, a sink in the
    softmax's denominator and an output gate."""

    heads: int
    kv_heads: int
    dim: int        # size of a query or key head
    vdim: int       # size of a value head
    scale: float    # scores are (q . k) * scale
    window: int     # mask.size: position i sees j when i - j < window ...
    keep_first: int  # ... or when j < keep_first

    @staticmethod
    def from_json(data: dict, where: str) -> "AttentionMixer":
        mask = data.get("mask") if isinstance(data, dict) else None
        if mask is None:
            mask = {}
        if not isinstance(mask, dict):
            raise ConfigError(f"config.json: {where}'mask' must be an object, got {mask!r}")
        heads = _int(data, "heads", where)
        kv_heads = _int(data, "kv_heads", where) if "kv_heads" in data else heads
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: {where}'heads' ({heads}) is not a multiple of 'kv_heads' ({kv_heads})")
        return AttentionMixer(
            heads=heads, kv_heads=kv_heads, dim=_int(data, "dim", where),
            vdim=_int(data, "vdim", where) if "vdim" in data else _int(data, "dim", where),
            scale=_number(data, "scale", where),
            window=min(_int(mask, "size", where + "mask."), NO_WINDOW) if mask.get("size") is not None else NO_WINDOW,
            keep_first=min(_int(mask, "keep_first", where + "mask.", minimum=0), NO_WINDOW) if mask.get("keep_first") is not None else 0)

    def to_json(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "mask": {"keep_first": self.keep_first, "size": self.window}, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float

    @staticmethod
    def from_json(data: dict, where: str) -> "DenseMlp":
        kind = _get(data, "kind", where)
        if kind not in MLP_KINDS:
            raise ConfigError(f"config.json: {where}'kind' {kind!r} is not supported (supported: {', '.join(MLP_KINDS)})")
        return DenseMlp(ff=_int(data, "ff", where), limit=_number(data, "limit", where))

    def to_json(self) -> dict:
        return {"ff": self.ff, "kind": "dense", "limit": self.limit}


@dataclass(frozen=True)
class ZirunexLayer:
    type: str
    mixer: AttentionMixer
    mlp: DenseMlp | None
    weights_of: int | None  # the layer whose tensors this one runs with; None = its own


@dataclass(frozen=True)
class ZirunexConfig:
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[ZirunexLayer, ...]

    eos_token_id = None  # the design names no end-of-sequence token

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses."""
        j = self.layers[i].weights_of
        return i if j is None else j

    @staticmethod
    def from_json(data: dict) -> "ZirunexConfig":
        layers_json = _get(data, "layers", "")
        if not isinstance(layers_json, list) or not layers_json:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: list[ZirunexLayer] = []
        for i, entry in enumerate(layers_json):
            where = f"layers[{i}]."
            kind = _get(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}'type' {kind!r} is not supported (supported: {', '.join(MIXER_TYPES)})")
            mixer = AttentionMixer.from_json(_get(entry, "mixer", where), where + "mixer.")
            mlp_json = entry.get("mlp")
            mlp = None if mlp_json is None else DenseMlp.from_json(mlp_json, where + "mlp.")
            owner = entry.get("weights_of")
            if owner is not None:
                if isinstance(owner, bool) or not isinstance(owner, int) or not 0 <= owner < len(layers_json) or owner == i:
                    raise ConfigError(f"config.json: {where}'weights_of' must name another layer, got {owner!r}")
            layers.append(ZirunexLayer(kind, mixer, mlp, owner))
        for i, layer in enumerate(layers):
            seen, j = {i}, layer.weights_of
            while j is not None and layers[j].weights_of is not None:  # a lender that borrows itself: follow to the owner
                if j in seen:
                    raise ConfigError(f"config.json: layers[{i}].'weights_of' leads in a circle")
                seen.add(j)
                j = layers[j].weights_of
            if j is None:
                continue
            lender = layers[j]
            if (lender.type, lender.mixer, lender.mlp) != (layer.type, layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] runs with the tensors of layer {j} but describes another layer")
            layers[i] = ZirunexLayer(layer.type, layer.mixer, layer.mlp, j)
        return ZirunexConfig(
            vocab_size=_int(data, "vocab", ""), width=_int(data, "width", ""),
            norm_eps=_number(_get(data, "norm", ""), "eps", "norm."),
            embedding_scale=_number(data["embedding"], "scale", "embedding.", positive=False) if data.get("embedding") is not None else 1.0,
            layers=tuple(layers))

    def to_json(self) -> dict:
        layers = []
        for layer in self.layers:
            entry = {"mixer": layer.mixer.to_json(), "mlp": None if layer.mlp is None else layer.mlp.to_json(), "type": layer.type}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        return {"architecture": NAME, "embedding": {"scale": self.embedding_scale}, "layers": layers,
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width}
