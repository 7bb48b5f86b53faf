"""Typed configuration of the Finelix decoder, read from the keys of its ``config.json``.

The file is nested: ``architecture`` (a name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``layers`` (one object per layer: ``type`` names the mixer, ``mixer`` holds its sizes and constants, ``mlp``
its feed-forward or null) and ``loop`` (``start``, ``stop``, ``times``: the layers ``start .. stop - 1`` run
``times`` times in a row with the same weights; absent or null: every layer runs once).  Every size and
constant is read here; nothing about a particular model stands in code.  Errors name the key.

Mixers: ``latent_attention`` (``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``,
``rot.base``, ``rot.dims``), ``gla`` and ``gla_2`` (``heads``, ``dim``, ``vdim``, ``tau``; optional
``decay_rank``, otherwise the weight file decides the rank of the decay projection).
Feed-forwards: ``kind`` ``dense`` (``ff``) or ``moe`` (``router.experts``, ``router.top``, ``expert.ff``, optional
``shared.ff``).  Optional top-level ``max_positions`` bounds a request's length (default 131072).
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, Dict, Optional, Tuple

from ..errors import ErrorCode, PhotonError

MIXER_TYPES = ("latent_attention", "gla", "gla_2")
DEFAULT_MAX_POSITIONS = 131072


from .nested import bad as _bad, num as _num  # noqa: E402


def _check_mixer(kind: str, m: Any, where: str) -> Dict[str, Any]:
    if not isinstance(m, dict):
        raise _bad(f"'{where}' must be an object")
    out: Dict[str, Any] = {"heads": _num(m, "heads", where), "dim": _num(m, "dim", where), "vdim": _num(m, "vdim", where)}
    if kind == "latent_attention":
        for k in ("rot_dim", "kv_rank", "q_rank"):
            out[k] = _num(m, k, where)
        out["scale"] = _num(m, "scale", where, float)
        rot = m.get("rot")
        if not isinstance(rot, dict):
            raise _bad(f"'{where}.rot' must be an object with 'base' and 'dims'")
        out["rot"] = {"base": _num(rot, "base", where + ".rot", float), "dims": _num(rot, "dims", where + ".rot")}
        if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["rot_dim"]:
            raise _bad(f"'{where}.rot.dims' must be even and at most rot_dim")
    else:
        out["tau"] = _num(m, "tau", where, float)
        if m.get("decay_rank") is not None:
            out["decay_rank"] = _num(m, "decay_rank", where)
    return out


def _check_mlp(m: Any, where: str) -> Optional[Dict[str, Any]]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise _bad(f"'{where}' must be an object or null")
    kind = m.get("kind")
    if kind == "dense":
        return {"kind": "dense", "ff": _num(m, "ff", where)}
    if kind == "moe":
        router = m.get("router")
        out = {"kind": "moe",
               "router": {"experts": _num(router, "experts", where + ".router"), "top": _num(router, "top", where + ".router")},
               "expert": {"ff": _num(m.get("expert"), "ff", where + ".expert")}}
        if out["router"]["top"] > out["router"]["experts"]:
            raise _bad(f"'{where}.router.top' exceeds the number of experts")
        if m.get("shared") is not None:
            out["shared"] = {"ff": _num(m["shared"], "ff", where + ".shared")}
        return out
    raise _bad(f"key '{where}.kind' must be 'dense' or 'moe', got {kind!r}")


@dataclasses.dataclass(frozen=True)
class FinelixLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclasses.dataclass(frozen=True)
class FinelixLoop:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class FinelixConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[FinelixLayer, ...]
    loop: Optional[FinelixLoop]
    max_positions: int = DEFAULT_MAX_POSITIONS

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FinelixConfig":
        name = d.get("architecture")
        if not isinstance(name, str):
            archs = d.get("architectures")
            if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
                raise _bad("key 'architecture' must name the model class")
            name = archs[0]
        layers_in = d.get("layers")
        if not isinstance(layers_in, list) or not layers_in:
            raise _bad("key 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(l, dict) or l.get("type") not in MIXER_TYPES:
                raise _bad(f"'{where}.type' must be one of {', '.join(MIXER_TYPES)}")
            layers.append(FinelixLayer(l["type"], _check_mixer(l["type"], l.get("mixer"), where + ".mixer"),
                                       _check_mlp(l.get("mlp"), where + ".mlp")))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = FinelixLoop(_num(lp, "start", "loop", positive=False, default=0), _num(lp, "stop", "loop"),
                               _num(lp, "times", "loop"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise _bad(f"'loop' must satisfy 0 <= start < stop <= {len(layers)} layers")
        emb = d.get("embedding") if d.get("embedding") is not None else {}
        return cls(architecture=name, vocab=_num(d, "vocab", "config"), width=_num(d, "width", "config"),
                   embedding_scale=_num(emb, "scale", "embedding", float, default=1.0),
                   norm_eps=_num(d.get("norm"), "eps", "norm", float), layers=tuple(layers), loop=loop,
                   max_positions=_num(d, "max_positions", "config", default=DEFAULT_MAX_POSITIONS))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
            "loop": dataclasses.asdict(self.loop) if self.loop else None,
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d
