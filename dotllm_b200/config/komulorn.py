"""Typed configuration of the Komulorn decoder, read from config.json's own keys.

config.json of this architecture is nested: ``layers`` lists the layers in order, each with its ``type``
("attention"), the mixer's sizes (``mixer``: ``heads``, ``kv_heads``, ``dim`` key channels and ``vdim`` value channels
a head, ``scale``, ``rot`` {``dims``, ``base``, optional ``scaling`` {factor, original, fast, slow}}, and ``kv_from``: the
index of an earlier layer whose keys and values this one reads instead of making its own) and its feed-forward
(``mlp``: ``kind`` "moe" with ``expert`` {ff}, ``router`` {experts, top} and an optional ``shared`` {ff}; null: none).
``norm.eps`` is every norm's eps, ``logit_softcap`` the cap on the logits (absent or 0: none), ``vocab`` and ``width``
the global sizes.  ``max_positions`` is optional (the design states no limit): positions up to
`DEFAULT_MAX_POSITIONS` are tabulated without it.  Every size and constant is taken from there; nothing is assumed
about their values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError
from .kubedra import _get

MIXER_TYPES = ("attention",)
DEFAULT_MAX_POSITIONS = 1 << 16


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float               # the length the frequencies were made for
    fast: float                   # turns over that length from which a frequency is kept as it is
    slow: float                   # turns up to which a frequency is divided by the factor

    @classmethod
    def from_dict(cls, d, where):
        return cls(_get(d, "factor", float, where), _get(d, "original", float, where), _get(d, "fast", float, where),
                   _get(d, "slow", float, where))

    def to_dict(self):
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int                      # key channels per head
    vdim: int                     # value channels per head
    scale: float
    rot_dims: int                 # the first that many channels of a head are rotated (0: none)
    rot_base: float
    rot_scaling: Optional[RotaryScaling] = None
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d, where):
        rot = d.get("rot") if isinstance(d, dict) else None
        scaling = rot.get("scaling") if isinstance(rot, dict) else None
        cfg = cls(_get(d, "heads", int, where), _get(d, "kv_heads", int, where), _get(d, "dim", int, where),
                  _get(d, "vdim", int, where), _get(d, "scale", float, where),
                  _get(rot, "dims", int, where + ".rot") if rot else 0,
                  _get(rot, "base", float, where + ".rot") if rot else 10000.0,
                  RotaryScaling.from_dict(scaling, where + ".rot.scaling") if scaling else None,
                  _get(d, "kv_from", int, where, required=False))
        if min(cfg.heads, cfg.kv_heads, cfg.dim, cfg.vdim) <= 0 or cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}: {cfg.heads} query heads over {cfg.kv_heads} key/value heads of "
                              f"{cfg.dim} / {cfg.vdim} channels")
        if cfg.rot_dims < 0 or cfg.rot_dims % 2 or cfg.rot_dims > cfg.dim:
            raise ConfigError(f"config.json: {where}.rot.dims = {cfg.rot_dims} must be even and at most dim = {cfg.dim}")
        return cfg

    def to_dict(self):
        out = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.rot_dims:
            out["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
            if self.rot_scaling is not None:
                out["rot"]["scaling"] = self.rot_scaling.to_dict()
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class MoeConfig:
    ff: int                       # one expert's hidden width
    experts: int
    top: int
    shared_ff: int = 0            # 0: no shared expert

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "kind", str, where)
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind = {kind!r}; known: 'moe'")
        expert, router, shared = d.get("expert"), d.get("router"), d.get("shared")
        cfg = cls(_get(expert, "ff", int, where + ".expert"), _get(router, "experts", int, where + ".router"),
                  _get(router, "top", int, where + ".router"), _get(shared, "ff", int, where + ".shared") if shared else 0)
        if cfg.ff <= 0 or not 0 < cfg.top <= cfg.experts or cfg.shared_ff < 0:
            raise ConfigError(f"config.json: {where}: {cfg.top} of {cfg.experts} experts of width {cfg.ff}")
        return cfg

    def to_dict(self):
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class KomulornLayerConfig:
    type: str
    mixer: AttentionMixerConfig
    mlp: Optional[MoeConfig]

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "type", str, where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}.type = {kind!r}; known: {list(MIXER_TYPES)}")
        if not isinstance(d.get("mixer"), dict):
            raise ConfigError(f"config.json: {where} lacks its mixer's sizes")
        return cls(kind, AttentionMixerConfig.from_dict(d["mixer"], where + ".mixer"),
                   MoeConfig.from_dict(d["mlp"], where + ".mlp") if d.get("mlp") else None)

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class KomulornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple                         # of KomulornLayerConfig
    logit_softcap: float = 0.0            # 0: the logits are not capped
    max_positions: int = DEFAULT_MAX_POSITIONS
    bos_token_id: Optional[int] = None
    eos_token_id: tuple = ()
    architecture: str = "Komulorn"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks its list of layers")
        parsed = tuple(KomulornLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(layers))
        for i, layer in enumerate(parsed):
            j = layer.mixer.kv_from
            if j is None:
                continue
            if not 0 <= j < i or parsed[j].mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {j} must name an earlier layer with keys and "
                                  f"values of its own")
            a, b = layer.mixer, parsed[j].mixer
            if (a.kv_heads, a.dim, a.vdim, a.rot_dims) != (b.kv_heads, b.dim, b.vdim, b.rot_dims):
                raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layers[{j}], whose key/value heads, "
                                  f"sizes or rotated channels differ")
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(_get(d, "vocab", int, "config"), _get(d, "width", int, "config"), _get(d.get("norm"), "eps", float, "norm"),
                  parsed, _get(d, "logit_softcap", float, "config", 0.0, required=False),
                  _get(d, "max_positions", int, "config", DEFAULT_MAX_POSITIONS, required=False),
                  _get(d, "bos_token_id", int, "config", required=False), eos)
        if min(cfg.vocab, cfg.width, cfg.max_positions) <= 0 or cfg.eps <= 0 or cfg.logit_softcap < 0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive, logit_softcap not negative")
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
