"""The typed Bosenex configuration, read from the design's own config.json keys.

A Bosenex config.json names its model with `"architecture": "Bosenex"` and lists its layers one by one: every
entry of `layers` gives the layer's `type` (which mixer it has: `mlstm`, a matrix memory with exponential gates, or
`parallel`, an attention mixer and a state-space mixer side by side), the mixer's sizes and constants (`mixer`; for
`parallel` under `left` and `right`), and its feed-forward (`mlp`: `kind` `dense` or `moe`, or null for a layer
without one). Beside the layers stand `vocab`, `width`, `norm.eps`, `embedding.scale` and `logit_scale`. No size has
a default: a size that is missing is an error that names it. A mechanism that a file does not mention is not there:
no `mask` is no window, no `rot` no rotation, no `softcap` no cap on the scores, no `gate_cap` no cap on the gates,
no `shared` no expert that every token uses, no `embedding` / `logit_scale` a factor of one; `kv_heads`, `vdim`,
`groups` and `norm_groups` left out equal `heads`, `dim`, 1 and 1.
"""

from __future__ import annotations

from dataclasses import dataclass

from .registry import ConfigError
from .zirunex import _get, _int, _number

NAME = "Bosenex"
MIXER_TYPES = ("mlstm", "parallel")
MLP_KINDS = ("dense", "moe")


def _optional(data: dict, key: str):
    return data.get(key) if isinstance(data, dict) else None


@dataclass(frozen=True)
class MatrixMemoryMixer:
    heads: int
    dim: int         # size of a query or key head
    vdim: int        # size of a value head
    gate_cap: float  # gates are cap * tanh(x / cap); 0: no cap

    @staticmethod
    def from_json(data: dict, where: str) -> "MatrixMemoryMixer":
        dim = _int(data, "dim", where)
        return MatrixMemoryMixer(heads=_int(data, "heads", where), dim=dim,
                                 vdim=_int(data, "vdim", where) if "vdim" in data else dim,
                                 gate_cap=_number(data, "gate_cap", where) if _optional(data, "gate_cap") is not None else 0.0)

    def to_json(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.gate_cap:
            out["gate_cap"] = self.gate_cap
        return out


@dataclass(frozen=True)
class WindowAttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float     # scores are (q . k) * scale ...
    softcap: float   # ... then cap * tanh(score / cap); 0: no cap
    window: int      # position i sees j when 0 <= i - j < window; 0: every earlier position
    rot_dims: int    # the first rot_dims dimensions of a head are rotated; 0: no rotation
    rot_base: float

    @staticmethod
    def from_json(data: dict, where: str) -> "WindowAttentionMixer":
        heads = _int(data, "heads", where)
        kv_heads = _int(data, "kv_heads", where) if "kv_heads" in data else heads
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: {where}'heads' ({heads}) is not a multiple of 'kv_heads' ({kv_heads})")
        dim = _int(data, "dim", where)
        mask, rot = _optional(data, "mask"), _optional(data, "rot")
        rot_dims = _int(rot, "dims", where + "rot.", minimum=0) if rot is not None else 0
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"config.json: {where}rot.'dims' must be even and at most 'dim' ({dim}), got {rot_dims}")
        return WindowAttentionMixer(
            heads=heads, kv_heads=kv_heads, dim=dim, vdim=_int(data, "vdim", where) if "vdim" in data else dim,
            scale=_number(data, "scale", where),
            softcap=_number(data, "softcap", where) if _optional(data, "softcap") is not None else 0.0,
            window=_int(mask, "size", where + "mask.") if mask is not None and mask.get("size") is not None else 0,
            rot_dims=rot_dims, rot_base=_number(rot, "base", where + "rot.") if rot_dims else 1.0)

    def to_json(self) -> dict:
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            out["mask"] = {"size": self.window}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.softcap:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class StateSpaceMixer:
    heads: int
    vdim: int         # columns of a head: inner = heads * vdim
    state: int        # rows of a head's state
    groups: int       # heads of a group share B and C
    conv: int         # taps of the causal convolution
    norm_groups: int  # the output is normalised in this many equal parts

    @staticmethod
    def from_json(data: dict, where: str) -> "StateSpaceMixer":
        heads = _int(data, "heads", where)
        groups = _int(data, "groups", where) if "groups" in data else 1
        parts = _int(data, "norm_groups", where) if "norm_groups" in data else 1
        vdim = _int(data, "vdim", where)
        if heads % groups != 0:
            raise ConfigError(f"config.json: {where}'heads' ({heads}) is not a multiple of 'groups' ({groups})")
        if (heads * vdim) % parts != 0:
            raise ConfigError(f"config.json: {where}'norm_groups' ({parts}) does not divide heads * vdim ({heads * vdim})")
        return StateSpaceMixer(heads=heads, vdim=vdim, state=_int(data, "state", where), groups=groups,
                               conv=_int(data, "conv", where), norm_groups=parts)

    def to_json(self) -> dict:
        return {"conv": self.conv, "groups": self.groups, "heads": self.heads, "norm_groups": self.norm_groups,
                "state": self.state, "vdim": self.vdim}


@dataclass(frozen=True)
class SideBySideMixer:
    left: WindowAttentionMixer
    right: StateSpaceMixer

    @staticmethod
    def from_json(data: dict, where: str) -> "SideBySideMixer":
        return SideBySideMixer(WindowAttentionMixer.from_json(_get(data, "left", where), where + "left."),
                               StateSpaceMixer.from_json(_get(data, "right", where), where + "right."))

    def to_json(self) -> dict:
        return {"left": self.left.to_json(), "right": self.right.to_json()}


@dataclass(frozen=True)
class DenseMlp:
    ff: int

    def to_json(self) -> dict:
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class ExpertsMlp:
    experts: int
    top: int
    ff: int                   # inner width of a routed expert
    limit: float
    shared_ff: int            # inner width of the expert that every token uses; 0: none
    shared_limit: float

    def to_json(self) -> dict:
        out = {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


def _mlp_from_json(data: dict, where: str):
    kind = _get(data, "kind", where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}'kind' {kind!r} is not supported (supported: {', '.join(MLP_KINDS)})")
    if kind == "dense":
        return DenseMlp(ff=_int(data, "ff", where))
    router, expert = _get(data, "router", where), _get(data, "expert", where)
    experts, top = _int(router, "experts", where + "router."), _int(router, "top", where + "router.")
    if top > experts:
        raise ConfigError(f"config.json: {where}router.'top' ({top}) exceeds 'experts' ({experts})")
    shared = _optional(data, "shared")
    return ExpertsMlp(experts=experts, top=top, ff=_int(expert, "ff", where + "expert."),
                      limit=_number(expert, "limit", where + "expert."),
                      shared_ff=_int(shared, "ff", where + "shared.") if shared is not None else 0,
                      shared_limit=_number(shared, "limit", where + "shared.") if shared is not None else 0.0)


@dataclass(frozen=True)
class BosenexLayer:
    type: str
    mixer: MatrixMemoryMixer | SideBySideMixer
    mlp: DenseMlp | ExpertsMlp | None


@dataclass(frozen=True)
class BosenexConfig:
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    layers: tuple[BosenexLayer, ...]

    eos_token_id = None  # the design names no end-of-sequence token

    @staticmethod
    def from_json(data: dict) -> "BosenexConfig":
        layers_json = _get(data, "layers", "")
        if not isinstance(layers_json, list) or not layers_json:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_json):
            where = f"layers[{i}]."
            kind = _get(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}'type' {kind!r} is not supported (supported: {', '.join(MIXER_TYPES)})")
            mixer_json = _get(entry, "mixer", where)
            mixer = (MatrixMemoryMixer if kind == "mlstm" else SideBySideMixer).from_json(mixer_json, where + "mixer.")
            mlp_json = entry.get("mlp")
            layers.append(BosenexLayer(kind, mixer, None if mlp_json is None else _mlp_from_json(mlp_json, where + "mlp.")))
        return BosenexConfig(
            vocab_size=_int(data, "vocab", ""), width=_int(data, "width", ""),
            norm_eps=_number(_get(data, "norm", ""), "eps", "norm."),
            embedding_scale=_number(data["embedding"], "scale", "embedding.", positive=False) if data.get("embedding") is not None else 1.0,
            logit_scale=_number(data, "logit_scale", "", positive=False) if data.get("logit_scale") is not None else 1.0,
            layers=tuple(layers))

    def to_json(self) -> dict:
        layers = [{"mixer": layer.mixer.to_json(), "mlp": None if layer.mlp is None else layer.mlp.to_json(), "type": layer.type}
                  for layer in self.layers]
        return {"architecture": NAME, "embedding": {"scale": self.embedding_scale}, "layers": layers,
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width}
