"""Typed configuration of the Fekopel decoder, read from the keys of its ``config.json``.

Nested like the file: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``layers`` (one object per layer:
``type`` names the mixer, ``mixer`` holds its sizes and constants, ``mlp`` its feed-forward or null) and ``loop``
(``start``, ``stop``, ``times``: layers ``start .. stop - 1`` run ``times`` times in a row with the same weights;
absent or null: every layer runs once).  Every size and constant is read here; errors name the key.

Mixers, both grouped-query attention with ``heads``, ``kv_heads``, ``dim`` (queries and keys), ``vdim`` (values),
``scale`` and ``mask`` (``size``: the window; absent: every earlier key is seen):

* ``attention``: unit-norm queries and keys, no positions, a sink in the softmax;
* ``attention_2``: weighted query/key norm, ``rot`` (``base``, ``dims``: rotation of the first ``dims`` numbers of a
  head), ``softcap``, ``mask.keep_first`` (the first keys stay visible behind the window), an output gate.

Feed-forward ``kind`` ``moe``: ``router`` (``experts``, ``top``, ``scale``, ``groups.count``, ``groups.keep``),
``expert.ff``, optional ``shared.ff``.  Optional top-level ``max_positions`` bounds a request's length.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, Dict, Optional, Tuple

from .nested import bad, num, obj

MIXER_TYPES = ("attention", "attention_2")
DEFAULT_MAX_POSITIONS = 131072


def _check_mixer(kind: str, m: Any, where: str) -> Dict[str, Any]:
    if not isinstance(m, dict):
        raise bad(f"'{where}' must be an object")
    out: Dict[str, Any] = {"heads": num(m, "heads", where), "dim": num(m, "dim", where)}
    out["kv_heads"] = num(m, "kv_heads", where, default=out["heads"])
    out["vdim"] = num(m, "vdim", where, default=out["dim"])
    out["scale"] = num(m, "scale", where, float)
    if out["heads"] % out["kv_heads"]:
        raise bad(f"'{where}.heads' must be a multiple of '{where}.kv_heads'")
    mask = obj(m, "mask", where)
    if mask is not None:
        out["mask"] = {"size": num(mask, "size", where + ".mask")}
        if kind == "attention_2" and mask.get("keep_first") is not None:
            out["mask"]["keep_first"] = num(mask, "keep_first", where + ".mask", positive=False)
            if out["mask"]["keep_first"] < 0:
                raise bad(f"key '{where}.mask.keep_first' must not be negative")
    if kind == "attention_2":
        rot = obj(m, "rot", where)
        if rot is not None:
            out["rot"] = {"base": num(rot, "base", where + ".rot", float), "dims": num(rot, "dims", where + ".rot")}
            if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["dim"]:
                raise bad(f"'{where}.rot.dims' must be even and at most dim")
        if m.get("softcap") is not None:
            out["softcap"] = num(m, "softcap", where, float)
    return out


def _check_mlp(m: Any, where: str) -> Optional[Dict[str, Any]]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise bad(f"'{where}' must be an object or null")
    if m.get("kind") != "moe":
        raise bad(f"key '{where}.kind' must be 'moe', got {m.get('kind')!r}")
    r = obj(m, "router", where, required=True)
    router: Dict[str, Any] = {"experts": num(r, "experts", where + ".router"), "top": num(r, "top", where + ".router"),
                              "scale": num(r, "scale", where + ".router", float, default=1.0)}
    if router["top"] > router["experts"]:
        raise bad(f"'{where}.router.top' exceeds the number of experts")
    g = obj(r, "groups", where + ".router")
    if g is not None:
        router["groups"] = {"count": num(g, "count", where + ".router.groups"), "keep": num(g, "keep", where + ".router.groups")}
        cnt, keep = router["groups"]["count"], router["groups"]["keep"]
        if router["experts"] % cnt or keep > cnt or keep * (router["experts"] // cnt) < router["top"]:
            raise bad(f"'{where}.router.groups': the experts must split into 'count' equal groups, and 'keep' of them "
                      "must hold at least 'top' experts")
    out = {"kind": "moe", "router": router, "expert": {"ff": num(obj(m, "expert", where, required=True), "ff", where + ".expert")}}
    if m.get("shared") is not None:
        out["shared"] = {"ff": num(obj(m, "shared", where), "ff", where + ".shared")}
    return out


@dataclasses.dataclass(frozen=True)
class FekopelLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclasses.dataclass(frozen=True)
class FekopelLoop:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class FekopelConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[FekopelLayer, ...]
    loop: Optional[FekopelLoop]
    max_positions: int = DEFAULT_MAX_POSITIONS

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FekopelConfig":
        name = d.get("architecture")
        if not isinstance(name, str):
            archs = d.get("architectures")
            if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
                raise bad("key 'architecture' must name the model class")
            name = archs[0]
        layers_in = d.get("layers")
        if not isinstance(layers_in, list) or not layers_in:
            raise bad("key 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]"
            if not isinstance(l, dict) or l.get("type") not in MIXER_TYPES:
                raise bad(f"'{where}.type' must be one of {', '.join(MIXER_TYPES)}")
            layers.append(FekopelLayer(l["type"], _check_mixer(l["type"], l.get("mixer"), where + ".mixer"),
                                       _check_mlp(l.get("mlp"), where + ".mlp")))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = FekopelLoop(num(lp, "start", "loop", positive=False, default=0), num(lp, "stop", "loop"),
                               num(lp, "times", "loop"))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise bad(f"'loop' must satisfy 0 <= start < stop <= {len(layers)} layers")
        return cls(architecture=name, vocab=num(d, "vocab", "config"), width=num(d, "width", "config"),
                   norm_eps=num(obj(d, "norm", "config", required=True), "eps", "norm", float), layers=tuple(layers),
                   loop=loop, max_positions=num(d, "max_positions", "config", default=DEFAULT_MAX_POSITIONS))

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": copy.deepcopy(l.mixer), "mlp": copy.deepcopy(l.mlp)} for l in self.layers],
            "loop": dataclasses.asdict(self.loop) if self.loop else None,
        }
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d
