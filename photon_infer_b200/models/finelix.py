"""The Finelix decoder as a ``ModelSpec``.

Embedding rows times ``embedding.scale``; parallel layers (one norm, ``x += mixer(h) + ff(h)``) whose mixer
is attention over a cached latent or gated linear attention and whose feed-forward is dense (GeGLU), a
mixture of experts with a shared expert, or absent; optionally a block of layers that is run several times
with the same weights, each pass with a cache or state of its own and entered through a projection of the
running stream joined with the embedding output; a final norm and an untied output head.

Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.in``, ``loop.step``, and per layer ``l<i>.norm1``,
``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.finelix_config import FinelixConfig
from ..config.registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def _mixer(cfg: FinelixConfig, kind: str, m: dict) -> PartSpec:
    if kind == "latent_attention":
        params = dict(hidden_size=cfg.width, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                      kv_rank=m["kv_rank"], q_rank=m["q_rank"], scale=m["scale"], eps=cfg.norm_eps,
                      rot_base=m["rot"]["base"], rot_dims=m["rot"]["dims"])
    else:
        params = dict(hidden_size=cfg.width, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], tau=m["tau"],
                      eps=cfg.norm_eps, decay_rank=m.get("decay_rank"))
    return PartSpec(kind, params, "mix.")


def _feed_forward(cfg: FinelixConfig, m):
    if m is None:
        return None
    if m["kind"] == "dense":
        return PartSpec("gated", dict(hidden_size=cfg.width, intermediate_size=m["ff"], activation="gelu_tanh",
                                      names=("gate", "up", "down")), "mlp.")
    return PartSpec("moe", dict(hidden_size=cfg.width, experts=m["router"]["experts"], top=m["router"]["top"],
                                expert_size=m["expert"]["ff"], shared_size=(m.get("shared") or {}).get("ff"),
                                activation="silu"), "mlp.")


def build_finelix_spec(cfg: FinelixConfig) -> ModelSpec:
    norm = lambda name: PartSpec("rms_norm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": name})
    layers = [LayerSpec(block=PartSpec("parallel", {}), norm1=norm("norm1"), mixer=_mixer(cfg, l.type, l.mixer),
                        norm2=None, feed_forward=_feed_forward(cfg, l.mlp), prefix=f"l{i}.")
              for i, l in enumerate(cfg.layers)]
    n = len(layers)
    stream_parts = {}
    if cfg.loop is None:
        run = [RunEntry(i) for i in range(n)]
    else:
        lp = cfg.loop
        stream_parts["loop"] = PartSpec("loop_input", dict(hidden_size=cfg.width, times=lp.times), "loop.")
        run = [RunEntry(i) for i in range(lp.start)]
        for t in range(lp.times):
            run += [RunEntry(i, before=("loop", t) if i == lp.start else None) for i in range(lp.start, lp.stop)]
        run += [RunEntry(i) for i in range(lp.stop, n)]
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_positions,
                     embedding_name="embed", head_name="head", final_norm=norm("final.norm"), position_encodings={},
                     layers=layers, run=run, embedding_scale=cfg.embedding_scale, stream_parts=stream_parts)


register_architecture("Finelix", FinelixConfig, build_finelix_spec, replace=True)
