"""Plain, slow implementation of the Finelix decoder: the oracle of its tests.

Whole sequences, no cache, no batching, one function per mechanism, float64 torch on the CPU.  It shares no code
with ``photon_infer_b200``: ``config.json`` is read as a plain dict and ``model.safetensors`` by the few lines
below.  Notation: ``h [T, H]`` rows are tokens; a weight ``W`` is stored ``[out, in]`` and applied as ``h W^T``.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        raw = data[a:b]
        if meta["dtype"] == "BF16":
            t = torch.from_numpy((np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy())
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = t.reshape(meta["shape"]).double()
    return out


# --------------------------------------------------------------------------- mechanisms

def rms_norm(x: torch.Tensor, eps: float, weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)``, times ``weight`` when given."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_half_layout(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Turns the first ``dims`` features of the last axis: feature ``i`` is paired with ``i + dims/2``, the pair
    ``(u, v)`` at position ``p`` becomes ``(u cos a - v sin a, v cos a + u sin a)``, ``a = p * base^(-2i/dims)``.
    ``x [T, ..., D]``; features from ``dims`` on pass unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    angle = positions.double().view(-1, *([1] * (x.dim() - 1))) * freq
    c, s = torch.cos(angle), torch.sin(angle)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def latent_attention(w: Dict[str, torch.Tensor], m: dict, eps: float, h: torch.Tensor) -> torch.Tensor:
    """Causal softmax attention whose keys and values are derived from one latent per token."""
    T = h.shape[0]
    n, d, r, vd, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (rms_norm(h @ w["dq"].T, eps, w["dq.norm"]) @ w["uq"].T).view(T, n, d + r)
    q_u, q_r = q[..., :d], rotate_half_layout(q[..., d:], pos, m["rot"]["base"], m["rot"]["dims"])
    kv = h @ w["dkv"].T
    c = rms_norm(kv[:, :kr], eps, w["dkv.norm"])
    k_r = rotate_half_layout(kv[:, kr:], pos, m["rot"]["base"], m["rot"]["dims"])
    k_u = (c @ w["uk"].T).view(T, n, d)
    v = (c @ w["uv"].T).view(T, n, vd)
    out = torch.zeros(T, n, vd, dtype=torch.float64)
    for t in range(T):
        for a in range(n):
            s = (k_u[: t + 1, a] @ q_u[t, a] + k_r[: t + 1] @ q_r[t, a]) * m["scale"]
            p = torch.softmax(s, dim=0)
            out[t, a] = p @ v[: t + 1, a]
    return out.reshape(T, n * vd) @ w["o"].T


def gated_linear_attention(w: Dict[str, torch.Tensor], m: dict, eps: float, h: torch.Tensor,
                           state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The recurrence ``S <- diag(a_t) S + k_t v_t^T``, ``o_t = S^T q_t`` token by token."""
    T = h.shape[0]
    n, d, vd = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T * d ** -0.5).view(T, n, d)
    k = (h @ w["k"].T).view(T, n, d)
    v = (h @ w["v"].T).view(T, n, vd)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    a = (torch.sigmoid(z) ** (1.0 / m["tau"])).view(T, n, d)
    S = torch.zeros(n, d, vd, dtype=torch.float64) if state is None else state
    o = torch.zeros(T, n, vd, dtype=torch.float64)
    for t in range(T):
        S = a[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("ndv,nd->nv", S, q[t])
    o = rms_norm(o, eps, w["norm"]).reshape(T, n * vd)
    return (o * silu(h @ w["g"].T)) @ w["o"].T


def gated_feed_forward(gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act, h: torch.Tensor) -> torch.Tensor:
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def routed_experts(w: Dict[str, torch.Tensor], m: dict, h: torch.Tensor) -> torch.Tensor:
    """Top experts by router logit, softmax over the chosen logits, plus the shared expert."""
    top = m["router"]["top"]
    z = h @ w["router"].T + w["router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))[:top]
        p = torch.softmax(z[t, chosen], dim=0)
        for j, e in enumerate(chosen):
            out[t] += p[j] * gated_feed_forward(w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], silu, h[t: t + 1])[0]
    if m.get("shared"):
        out = out + gated_feed_forward(w["shared.gate"], w["shared.up"], w["shared.down"], silu, h)
    return out


def loop_input(w_in: torch.Tensor, steps: torch.Tensor, x: torch.Tensor, x0: torch.Tensor, t: int) -> torch.Tensor:
    return torch.cat([x, x0], dim=-1) @ w_in.T + steps[t]


# --------------------------------------------------------------------------- the model

def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


class PlainFinelix:
    def __init__(self, config: dict, weights: Dict[str, torch.Tensor]):
        self.cfg, self.w = config, weights

    @classmethod
    def from_folder(cls, folder: str) -> "PlainFinelix":
        with open(os.path.join(folder, "config.json")) as f:
            cfg = json.load(f)
        return cls(cfg, read_safetensors(os.path.join(folder, "model.safetensors")))

    def run_order(self) -> List[tuple]:
        n, lp = len(self.cfg["layers"]), self.cfg.get("loop")
        if not lp:
            return [(i, None) for i in range(n)]
        order = [(i, None) for i in range(lp["start"])]
        for t in range(lp["times"]):
            order += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
        return order + [(i, None) for i in range(lp["stop"], n)]

    def layer(self, i: int, x: torch.Tensor) -> torch.Tensor:
        l, eps = self.cfg["layers"][i], self.cfg["norm"]["eps"]
        h = rms_norm(x, eps, self.w[f"l{i}.norm1"])
        mw = sub(self.w, f"l{i}.mix.")
        if l["type"] == "latent_attention":
            y = latent_attention(mw, l["mixer"], eps, h)
        else:
            y = gated_linear_attention(mw, l["mixer"], eps, h)
        mlp = l.get("mlp")
        if mlp is not None:
            fw = sub(self.w, f"l{i}.mlp.")
            y = y + (gated_feed_forward(fw["gate"], fw["up"], fw["down"], gelu_tanh, h) if mlp["kind"] == "dense"
                     else routed_experts(fw, mlp, h))
        return x + y

    def hidden(self, ids: Sequence[int], record: Optional[list] = None) -> torch.Tensor:
        x0 = self.w["embed"][torch.tensor(list(ids), dtype=torch.long)] * self.cfg.get("embedding", {}).get("scale", 1.0)
        x = x0
        for i, t in self.run_order():
            if t is not None:
                x = loop_input(self.w["loop.in"], self.w["loop.step"], x, x0, t)
            x = self.layer(i, x)
            if record is not None:
                record.append(x)
        return x

    def logits(self, ids: Sequence[int]) -> torch.Tensor:
        x = self.hidden(ids)
        return rms_norm(x, self.cfg["norm"]["eps"], self.w["final.norm"]) @ self.w["head"].T

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        ids = list(prompt)
        for _ in range(n):
            ids.append(int(torch.argmax(self.logits(ids)[-1])))
        return ids[len(prompt):]
