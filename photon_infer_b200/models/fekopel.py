"""The Fekopel decoder as a ``ModelSpec``.

Pre-norm layers with layer norms (weight and bias): ``x += mixer(norm1(x)); x += ff(norm2(x))``.  The mixer is one of
two kinds of grouped-query attention with normed queries and keys (``parts/normed_attention.py``): ``attention``
(unit norm, no positions, a window, a sink in the softmax) or ``attention_2`` (weighted norm, rotation of part of a
head, bounded scores, a window that keeps the first keys, an output gate).  The feed-forward is a mixture of plain
experts ``W_down gelu(W_up h)`` chosen by a softmax router with groups, plus a shared expert behind a per-token gate,
or absent.  A block of layers may run several times with the same weights, each pass with a cache of its own; before
every pass but the first the embedding output is added to the stream, and before every pass a vector of that pass.
A final layer norm and an untied output head.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), ``loop.step``, and per layer ``l<i>.norm1``, ``l<i>.norm2``
(each + ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.fekopel_config import FekopelConfig
from ..config.registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer(cfg: FekopelConfig, kind: str, m: dict) -> PartSpec:
    mask = m.get("mask") or {}
    params = dict(hidden_size=cfg.width, n_q_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                  value_dim=m["vdim"], scale=m["scale"], eps=cfg.norm_eps, window=mask.get("size"))
    if kind == "attention":
        params.update(norm_weight=False, sink=True)
    else:
        rot = m.get("rot") or {}
        params.update(norm_weight=True, rot_dims=rot.get("dims", 0), rot_base=rot.get("base", 10000.0),
                      softcap=m.get("softcap"), keep_first=mask.get("keep_first", 0), output_gate=True)
    return PartSpec("normed_attention", params, "mix.")


def _feed_forward(cfg: FekopelConfig, m):
    if m is None:
        return None
    r = m["router"]
    groups = r.get("groups") or {}
    return PartSpec("moe", dict(hidden_size=cfg.width, experts=r["experts"], top=r["top"], expert_size=m["expert"]["ff"],
                                shared_size=(m.get("shared") or {}).get("ff"), activation="gelu", gated=False,
                                router_bias=False, scoring="softmax_all", groups=groups.get("count", 1),
                                keep_groups=groups.get("keep"), route_scale=r.get("scale", 1.0),
                                shared_gate=bool(m.get("shared"))), "mlp.")


def build_fekopel_spec(cfg: FekopelConfig) -> ModelSpec:
    norm = lambda name: PartSpec("layer_norm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": name,
                                                "bias_name": name + ".b"})
    layers = []
    for i, l in enumerate(cfg.layers):
        ff = _feed_forward(cfg, l.mlp)
        layers.append(LayerSpec(block=PartSpec("pre_norm", {}), norm1=norm("norm1"), mixer=_mixer(cfg, l.type, l.mixer),
                                norm2=norm("norm2") if ff is not None else None, feed_forward=ff, prefix=f"l{i}."))
    n = len(layers)
    stream_parts = {}
    if cfg.loop is None:
        run = [RunEntry(i) for i in range(n)]
    else:
        lp = cfg.loop
        stream_parts["loop"] = PartSpec("loop_add", dict(hidden_size=cfg.width, times=lp.times), "loop.")
        run = [RunEntry(i) for i in range(lp.start)]
        for t in range(lp.times):
            run += [RunEntry(i, before=("loop", t) if i == lp.start else None) for i in range(lp.start, lp.stop)]
        run += [RunEntry(i) for i in range(lp.stop, n)]
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_positions,
                     embedding_name="embed", head_name="head", final_norm=norm("final.norm"), position_encodings={},
                     layers=layers, run=run, stream_parts=stream_parts)


register_architecture("Fekopel", FekopelConfig, build_fekopel_spec, replace=True)
