"""The Fekopel decoder, written plainly: one function per mechanism, float64 torch on the CPU, whole sequences
at once, no cache.  It shares no code with the package; the tests compare the package against it.

A model is ``(config, tensors)``: the dictionary of config.json and the tensors by name.

Notation: ``x [n, width]`` the residual stream of one sequence, position ``i`` of a query, ``j`` of a key.
"""
import math

import torch

F = torch.float64


def t64(t):
    return t.to(F)


# ----------------------------------------------------------------------------- norms

def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ----------------------------------------------------------------------------- positions

def rotate_first_dims(x, pos, dims, base):
    """x [n, heads, d]; the first ``dims`` numbers of a head are rotated, number i with number i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = pos.to(F)[:, None] * freq[None, :]                       # [n, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- who sees whom

def visible(n, size=None, keep_first=0):
    """[n, n] boolean: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size is not None:
        ok = ok & ((i - j < size) | (j < keep_first))
    return ok


def softmax_over_visible(s, ok, sink):
    """Rows of s [.., n, n]; with ``sink`` one more key with score 0 and no value takes part in the denominator."""
    s = s.masked_fill(~ok, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink:
        m = torch.clamp(m, min=0.0)
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink:
        den = den + torch.exp(-m)
    return e / den


# ----------------------------------------------------------------------------- mixers

def heads_of(x, n, d):
    return x.reshape(x.shape[0], n, d)


def grouped(q, k, v, scale, ok, sink=False, softcap=None):
    """q [n, H, d], k [n, G, d], v [n, G, dv] -> [n, H * dv]; query head h reads key/value head h // (H / G)."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        p = softmax_over_visible(s, ok, sink)
        out.append(p @ v[:, g])
    return torch.cat(out, dim=-1)


def mixer_attention(h, m, w, eps):
    """Unit-norm queries and keys, no positions, window, a sink in the softmax."""
    n = h.shape[0]
    q = unit_rms(heads_of(h @ w["q"].T, m["heads"], m["dim"]), eps)
    k = unit_rms(heads_of(h @ w["k"].T, m["kv_heads"], m["dim"]), eps)
    v = heads_of(h @ w["v"].T, m["kv_heads"], m["vdim"])
    mask = m.get("mask") or {}
    ok = visible(n, mask.get("size"), 0)
    return grouped(q, k, v, m["scale"], ok, sink=True) @ w["o"].T


def mixer_attention_2(h, m, w, eps):
    """Weighted query/key norm, rotation of the first dims, capped scores, window with kept first keys, output gate."""
    n = h.shape[0]
    pos = torch.arange(n)
    q = unit_rms(heads_of(h @ w["q"].T, m["heads"], m["dim"]), eps) * w["q.norm"]
    k = unit_rms(heads_of(h @ w["k"].T, m["kv_heads"], m["dim"]), eps) * w["k.norm"]
    v = heads_of(h @ w["v"].T, m["kv_heads"], m["vdim"])
    rot = m.get("rot") or {}
    q = rotate_first_dims(q, pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_first_dims(k, pos, rot.get("dims", 0), rot.get("base", 1.0))
    mask = m.get("mask") or {}
    ok = visible(n, mask.get("size"), mask.get("keep_first", 0))
    a = grouped(q, k, v, m["scale"], ok, sink=False, softcap=m.get("softcap"))
    a = a * torch.sigmoid(h @ w["g"].T)
    return a @ w["o"].T


# ----------------------------------------------------------------------------- feed-forward

def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def expert(h, up, down):
    return gelu_erf(h @ up.T) @ down.T


def route(h, m, w):
    """Returns (ids [n, top], weights [n, top])."""
    r = m["router"]
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ w["router"].T, dim=-1)                   # [n, E]
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        cnt, keep = groups["count"], groups["keep"]
        per = E // cnt
        gs = s.reshape(-1, cnt, per).max(-1).values                # [n, cnt]
        best = torch.zeros_like(gs, dtype=torch.bool)
        rest = gs.clone()
        for _ in range(keep):
            i = rest.argmax(-1, keepdim=True)
            best.scatter_(1, i, True)
            rest.scatter_(1, i, -1.0)
        allowed = best.repeat_interleave(per, dim=1)
    rest = s.masked_fill(~allowed, -1.0)
    ids = []
    for _ in range(top):
        i = rest.argmax(-1, keepdim=True)
        ids.append(i)
        rest = rest.scatter(1, i, -2.0)
    ids = torch.cat(ids, dim=1)
    chosen = s.gather(1, ids)
    weights = chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * r.get("scale", 1.0)
    return ids, weights


def moe(h, m, w):
    ids, weights = route(h, m, w)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += weights[t, j] * expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if m.get("shared"):
        gate = torch.sigmoid(h @ w["shared.sg"].T)                 # [n, 1]
        out = out + gate * expert(h, w["shared.up"], w["shared.down"])
    return out


# ----------------------------------------------------------------------------- the model

def part_weights(tensors, prefix):
    return {k[len(prefix):]: t64(v) for k, v in tensors.items() if k.startswith(prefix)}


def run_order(config):
    """[(layer, first of pass t or None)] in the order the layers run."""
    n = len(config["layers"])
    lp = config.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(lp.get("start", 0))]
    for t in range(lp["times"]):
        order += [(i, t if i == lp.get("start", 0) else None) for i in range(lp.get("start", 0), lp["stop"])]
    order += [(i, None) for i in range(lp["stop"], n)]
    return order


def forward(config, tensors, tokens, return_layers=False):
    """Logits [n, vocab] of one sequence (and the stream after every layer run)."""
    eps = config["norm"]["eps"]
    x0 = t64(tensors["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    after = []
    for i, pass_no in run_order(config):
        L = config["layers"][i]
        if pass_no is not None:
            if pass_no > 0:
                x = x + x0
            x = x + t64(tensors["loop.step"])[pass_no]
        p = f"l{i}."
        h = layer_norm(x, t64(tensors[p + "norm1"]), t64(tensors[p + "norm1.b"]), eps)
        w = part_weights(tensors, p + "mix.")
        if L["type"] == "attention":
            x = x + mixer_attention(h, L["mixer"], w, eps)
        elif L["type"] == "attention_2":
            x = x + mixer_attention_2(h, L["mixer"], w, eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            h = layer_norm(x, t64(tensors[p + "norm2"]), t64(tensors[p + "norm2.b"]), eps)
            x = x + moe(h, L["mlp"], part_weights(tensors, p + "mlp."))
        after.append(x.clone())
    y = layer_norm(x, t64(tensors["final.norm"]), t64(tensors["final.norm.b"]), eps)
    logits = y @ t64(tensors["head"]).T
    return (logits, torch.stack(after)) if return_layers else logits


# ----------------------------------------------------------------------------- a model folder

def read_folder(folder):
    """(config, tensors) of a folder with config.json and model.safetensors (bfloat16 or float32 tensors)."""
    import json
    import os
    import struct

    import numpy as np
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        if meta["dtype"] == "BF16":
            t = torch.from_numpy((np.frombuffer(data[a:b], dtype="<u2").astype(np.uint32) << 16).view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(data[a:b], dtype="<f4").copy())
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        tensors[name] = t.reshape(meta["shape"]).to(F)
    return config, tensors


def greedy(config, tensors, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(forward(config, tensors, ids)[-1])))
    return ids[len(prompt):]
