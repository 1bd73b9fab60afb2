"""Typed configuration of the Kubedra decoder, read from config.json's own keys.

config.json of this architecture is nested: ``layers`` lists the layers in order, each with its ``type``
("gla" or "latent_attention"), the mixer's sizes (``mixer``) and its feed-forward (``mlp``: ``kind`` "dense"
with ``ff``, or "moe" with ``expert`` {ff, limit}, ``router`` {experts, top} and an optional ``shared``
{ff, limit}; null: none).  ``loop`` {start, stop, times} repeats a run of layers with shared weights;
``norm.eps`` is every norm's eps; ``vocab``, ``width`` and ``max_positions`` the global sizes.  Every
size and constant is taken from there; nothing is assumed about their values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError

MIXER_TYPES = ("gla", "latent_attention")


def _get(d, key, kind, where, default=None, required=True):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json: {where} lacks required key {key!r}")
        return default
    try:
        return kind(d[key])
    except (TypeError, ValueError) as exc:
        raise ConfigError(f"config.json: {where}.{key} = {d[key]!r} is not {kind.__name__}") from exc


@dataclass(frozen=True)
class GlaMixerConfig:
    heads: int
    dim: int                      # key channels per head
    vdim: int                     # value channels per head
    tau: float
    decay_rank: Optional[int] = None      # only the random-weights mode needs it: a checkpoint's tensors give it

    @classmethod
    def from_dict(cls, d, where):
        return cls(_get(d, "heads", int, where), _get(d, "dim", int, where), _get(d, "vdim", int, where),
                   _get(d, "tau", float, where), _get(d, "decay_rank", int, where, required=False))

    def to_dict(self):
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.decay_rank is not None:
            out["decay_rank"] = self.decay_rank
        return out


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: Optional[float] = None         # None: dim^-1/2
    window: Optional[int] = None          # mask.size; None: every earlier key

    @classmethod
    def from_dict(cls, d, where):
        mask = d.get("mask") if isinstance(d, dict) else None
        return cls(_get(d, "heads", int, where), _get(d, "dim", int, where), _get(d, "vdim", int, where),
                   _get(d, "q_rank", int, where), _get(d, "kv_rank", int, where),
                   _get(d, "scale", float, where, required=False),
                   _get(mask, "size", int, where + ".mask", required=False) if mask else None)

    def to_dict(self):
        out = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "q_rank": self.q_rank, "kv_rank": self.kv_rank}
        if self.scale is not None:
            out["scale"] = self.scale
        if self.window is not None:
            out["mask"] = {"size": self.window}
        return out


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                             # "dense" or "moe"
    ff: int                               # dense: the hidden width; moe: one expert's
    limit: float = 0.0                    # moe: the experts' clamp
    experts: int = 0
    top: int = 0
    shared_ff: int = 0                    # 0: no shared expert
    shared_limit: float = 0.0

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "kind", str, where)
        if kind == "dense":
            return cls("dense", _get(d, "ff", int, where))
        if kind != "moe":
            raise ConfigError(f"config.json: {where}.kind = {kind!r}; known: 'dense', 'moe'")
        expert, router, shared = d.get("expert"), d.get("router"), d.get("shared")
        return cls("moe", _get(expert, "ff", int, where + ".expert"), _get(expert, "limit", float, where + ".expert"),
                   _get(router, "experts", int, where + ".router"), _get(router, "top", int, where + ".router"),
                   _get(shared, "ff", int, where + ".shared") if shared else 0,
                   _get(shared, "limit", float, where + ".shared") if shared else 0.0)

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
               "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


@dataclass(frozen=True)
class KubedraLayerConfig:
    type: str
    mixer: object                         # GlaMixerConfig or LatentMixerConfig
    mlp: Optional[FeedForwardConfig]

    @classmethod
    def from_dict(cls, d, where):
        kind = _get(d, "type", str, where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}.type = {kind!r}; known: {list(MIXER_TYPES)}")
        if not isinstance(d.get("mixer"), dict):
            raise ConfigError(f"config.json: {where} lacks its mixer's sizes")
        mixer = (GlaMixerConfig if kind == "gla" else LatentMixerConfig).from_dict(d["mixer"], where + ".mixer")
        mlp = FeedForwardConfig.from_dict(d["mlp"], where + ".mlp") if d.get("mlp") else None
        return cls(kind, mixer, mlp)

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class KubedraConfig:
    vocab: int
    width: int
    max_positions: int
    eps: float
    layers: tuple                         # of KubedraLayerConfig
    loop_start: int = 0                   # layers loop_start .. loop_stop - 1 run loop_times times in a row
    loop_stop: int = 0
    loop_times: int = 1
    bos_token_id: Optional[int] = None
    eos_token_id: tuple = ()
    architecture: str = "Kubedra"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks its list of layers")
        parsed = tuple(KubedraLayerConfig.from_dict(layer, f"layers[{i}]") for i, layer in enumerate(layers))
        loop = d.get("loop") or None
        start = _get(loop, "start", int, "loop") if loop else 0
        stop = _get(loop, "stop", int, "loop") if loop else 0
        times = _get(loop, "times", int, "loop") if loop else 1
        if loop and not (0 <= start <= stop <= len(parsed) and times >= 1):
            raise ConfigError(f"config.json: loop {loop!r} does not fit {len(parsed)} layers")
        eos = d.get("eos_token_id")
        eos = () if eos is None else tuple(int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(_get(d, "vocab", int, "config"), _get(d, "width", int, "config"), _get(d, "max_positions", int, "config"),
                  _get(d.get("norm"), "eps", float, "norm"), parsed, start, stop, times,
                  _get(d, "bos_token_id", int, "config", required=False), eos)
        if min(cfg.vocab, cfg.width, cfg.max_positions) <= 0 or cfg.eps <= 0:
            raise ConfigError("config.json: vocab, width, max_positions and norm.eps must be positive")
        return cfg

    def to_dict(self):
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "max_positions": self.max_positions, "norm": {"eps": self.eps},
               "layers": [layer.to_dict() for layer in self.layers]}
        if self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.bos_token_id is not None:
            out["bos_token_id"] = self.bos_token_id
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out

    def layer_runs(self):
        """(layer index, takes the embedding output in again) for every layer execution, in order."""
        n = len(self.layers)
        if self.loop_stop <= self.loop_start:
            return [(i, False) for i in range(n)]
        runs = [(i, False) for i in range(self.loop_start)]
        for p in range(self.loop_times):
            runs += [(i, p > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, False) for i in range(self.loop_stop, n)]
