"""Each mechanism of the Fekopel decoder alone, on the device, against its plain function: the layer norm fused with
the residual sum, the entrance of a looped block by addition, the per-head norm and partial rotation of queries and
keys with the cache write, attention with a window, kept first keys, a sink and bounded scores in every kernel that
serves it (the general one, the split-key tensor-core kernel for decoded tokens, the tcgen05 kernel for prompt
portions), keys made to stand out just inside and just outside every edge, the router with groups, the plain experts
on each of their paths, the gate of the shared expert and of the mixer's output."""
import math
import types

import pytest
import torch

from helpers import rel_err
from plain import fekopel_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOLS = {torch.float32: 5e-6, torch.bfloat16: 2e-2}
i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)


def _weights(part, dtype, std, seed):
    g = torch.Generator().manual_seed(seed)
    w = {}
    for t in part.tensor_specs():
        x = std * torch.randn(t.concrete_shape(), generator=g)
        if t.init == "norm":
            x = 1.0 + x
        w[t.name] = x.to(dtype)
    part.load({k: v.to(DEV) for k, v in w.items()})
    return {k: v.double() for k, v in w.items()}


# ----------------------------------------------------------------------------- norms and stream

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [72, 50, 1024])
def test_layer_norm_with_pending_outputs(dtype, width):
    from photon_infer_b200.parts.registry import create_part
    g = torch.Generator().manual_seed(width)
    norm = create_part("norm", "layer_norm", {"size": width, "eps": 1e-5, "weight_name": "w", "bias_name": "w.b"})
    w, b = (1 + 0.2 * torch.randn(width, generator=g)).to(dtype), (0.3 * torch.randn(width, generator=g)).to(dtype)
    norm.load({"w": w.to(DEV), "w.b": b.to(DEV)})
    x = 3.0 + 2 * torch.randn(6, width, generator=g)          # a mean far from zero: the deviations must be taken from it
    a, c = torch.randn(6, width, generator=g).to(dtype), torch.randn(6, width, generator=g).to(dtype)
    res = x.to(DEV).clone()
    out = norm.add_forward((a.to(DEV), c.to(DEV)), res, dtype)
    want_x = x.double() + (a.double() + c.double())
    assert rel_err(res.cpu(), want_x) < 1e-6
    assert rel_err(out.float().cpu(), plain.layer_norm(want_x, w.double(), b.double(), 1e-5)) < (3e-6 if dtype == torch.float32 else 6e-3)
    rows = i32([4, 1])
    res2 = x.to(DEV).clone()
    out2 = norm.add_forward_rows((a.to(DEV), c.to(DEV)), res2, rows, dtype)
    assert torch.equal(res2.cpu(), x) and torch.equal(out2, out[[4, 1]])
    plain_only = norm.forward(x.to(DEV).clone(), dtype)
    assert rel_err(plain_only.float().cpu(), plain.layer_norm(x.double(), w.double(), b.double(), 1e-5)) < (3e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_loop_entrance_by_addition(dtype):
    from photon_infer_b200.parts.registry import create_part
    part = create_part("stream", "loop_add", dict(hidden_size=40, times=3))
    w = _weights(part, dtype, 0.5, 3)
    g = torch.Generator().manual_seed(4)
    x, x0 = torch.randn(5, 40, generator=g), torch.randn(5, 40, generator=g)
    a = torch.randn(5, 40, generator=g).to(dtype)
    for t in (0, 1, 2):
        out = part.forward(x.to(DEV).clone(), a.to(DEV), x0.to(DEV), t, None)
        want = x.double() + a.double() + (x0.double() if t > 0 else 0) + w["step"][t]
        assert out.dtype == torch.float32 and rel_err(out.cpu(), want) < 1e-6
    with pytest.raises(IndexError):
        part.forward(x.to(DEV), None, x0.to(DEV), 3, None)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_gate(dtype):
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    x, z = torch.randn(7, 50, generator=g).to(dtype), 3 * torch.randn(7, 90, generator=g)
    xd = x.to(DEV).clone()
    ops.gate_mul(xd, z.to(DEV)[:, 20:70])                      # a 32-bit gate in a view with a row stride
    assert rel_err(xd.float().cpu(), x.double() * torch.sigmoid(z.double()[:, 20:70])) < (1e-6 if dtype == torch.float32 else 5e-3)
    x4, z4 = torch.randn(6, 64, generator=g).to(dtype), torch.randn(6, 200, generator=g)      # rows of four: the vector path
    xd = x4.to(DEV).clone()
    ops.gate_mul(xd, z4.to(DEV)[:, 128:192])
    assert rel_err(xd.float().cpu(), x4.double() * torch.sigmoid(z4.double()[:, 128:192])) < (1e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype,rows,n,k", [(torch.bfloat16, 3, 96, 64), (torch.bfloat16, 40, 88, 56), (torch.bfloat16, 512, 6144, 256),
                                            (torch.bfloat16, 200, 6144 * 2, 128), (torch.float32, 5, 30, 20), (torch.bfloat16, 7, 33, 50)])
def test_product_with_gelu_behind_it(dtype, rows, n, k):
    """Few rows (the weight-streaming kernel), many tiles (tcgen05, on one SM and on pairs) and in between (the
    library's product, then the activation kernel): the exact gelu of every output."""
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(rows)
    x, w = torch.randn(rows, k, generator=g).to(dtype), (0.2 * torch.randn(n, k, generator=g)).to(dtype)
    got = ops.linear_act(x.to(DEV), w.to(DEV), "gelu").float().cpu()
    assert rel_err(got, plain.gelu_erf(x.double() @ w.double().T)) < (2e-6 if dtype == torch.float32 else 6e-3)
    z = torch.randn(5, 24 if dtype == torch.bfloat16 else 7, generator=g).to(dtype)      # the vector path and the plain one
    assert rel_err(ops.activation(z.to(DEV).clone(), "gelu").float().cpu(), plain.gelu_erf(z.double())) < (1e-6 if dtype == torch.float32 else 5e-3)


# ----------------------------------------------------------------------------- query/key norm, rotation, cache write

@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("shape", [dict(nq=4, nkv=2, d=64, dv=64, rot=32, weight=True), dict(nq=3, nkv=1, d=10, dv=14, rot=6, weight=True),
                                   dict(nq=2, nkv=2, d=24, dv=8, rot=24, weight=False), dict(nq=5, nkv=5, d=6, dv=9, rot=0, weight=False),
                                   dict(nq=2, nkv=1, d=128, dv=128, rot=64, weight=True)])
def test_qk_norm_rotation_and_cache_write(in_dtype, out_dtype, shape):
    from photon_infer_b200.kernels import ops
    nq, nkv, d, dv, rot = (shape[k] for k in ("nq", "nkv", "d", "dv", "rot"))
    g = torch.Generator().manual_seed(d)
    T, page, pages = 9, 4, 7
    rows = (2.0 * torch.randn(T, nq * d + nkv * d + nkv * dv + 5, generator=g)).to(in_dtype)
    pos = [0, 1, 2, 3, 1000, 1001, 40000, 7, 8]                 # large positions: the angle needs more than 32 bits of care
    slots = [5, 6, 7, 8, 20, 21, 3, -1, 0]                      # -1: nothing is stored
    qw = (1 + 0.3 * torch.randn(d, generator=g)).to(in_dtype) if shape["weight"] else None
    kw = (1 + 0.3 * torch.randn(d, generator=g)).to(in_dtype) if shape["weight"] else None
    base = 5000.0
    inv = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1)).to(DEV) if rot else None
    rd = rows.to(DEV)
    q_out = torch.empty(T, nq * d, dtype=out_dtype, device=DEV)
    kc = torch.zeros(pages, nkv, page, d, dtype=out_dtype, device=DEV)
    vc = torch.zeros(pages, nkv, page, dv, dtype=out_dtype, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.qk_norm_rope_write(rd[:, :nq * d], rd[:, nq * d:(nq + nkv) * d], rd[:, (nq + nkv) * d:(nq + nkv) * d + nkv * dv], q_out,
                           qw.to(DEV) if qw is not None else None, kw.to(DEV) if kw is not None else None, 1e-6, i32(pos), inv, rot,
                           i32(slots), kc, vc, nq, nkv, d, dv, err)
    assert err.cpu().tolist()[0] == 0
    x = rows.double()
    P = torch.tensor(pos)
    q = plain.unit_rms(x[:, :nq * d].reshape(T, nq, d), 1e-6) * (qw.double() if qw is not None else 1.0)
    k = plain.unit_rms(x[:, nq * d:(nq + nkv) * d].reshape(T, nkv, d), 1e-6) * (kw.double() if kw is not None else 1.0)
    q, k = plain.rotate_first_dims(q, P, rot, base), plain.rotate_first_dims(k, P, rot, base)
    v = x[:, (nq + nkv) * d:(nq + nkv) * d + nkv * dv].reshape(T, nkv, dv)
    tol = 2e-6 if out_dtype == torch.float32 else 5e-3
    assert rel_err(q_out.float().cpu().reshape(T, nq, d), q) < tol
    for t, s in enumerate(slots):
        if s < 0:
            continue
        assert rel_err(kc[s // page, :, s % page].float().cpu(), k[t]) < tol
        assert rel_err(vc[s // page, :, s % page].float().cpu(), v[t]) < tol
    used = {s for s in slots if s >= 0}
    for s in range(pages * page):
        if s not in used:
            assert float(kc[s // page, :, s % page].abs().max()) == 0.0


# ----------------------------------------------------------------------------- attention kernels

def _oracle(q, k, v, pos, scale, window, keep, sink, cap):
    """q [n, H, d], k [L, G, d], v [L, G, dv], pos [n] -> [n, H * dv] by the plain softmax over the visible keys."""
    L = k.shape[0]
    i, j = torch.tensor(pos)[:, None], torch.arange(L)[None, :]
    ok = j <= i
    if window:
        ok = ok & ((i - j < window) | (j < keep))
    H, G = q.shape[1], k.shape[1]
    out = []
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        out.append(plain.softmax_over_visible(s, ok, sink) @ v[:, h // (H // G)])
    return torch.cat(out, dim=-1)


class _Step:
    """Requests with keys and values already in a paged cache (pages scattered over the pool, stale numbers in the
    pages' unused slots), and a step that brings the last ``n`` tokens of each."""

    def __init__(self, lengths, counts, nq, nkv, d, dv, page, dtype, seed, std=1.0):
        from photon_infer_b200.parts.base import GroupView, StepContext
        g = torch.Generator().manual_seed(seed)
        self.lengths, self.counts = lengths, counts
        S = len(lengths)
        per = max(-(-L // page) for L in lengths) + 1
        order = torch.randperm(S * per, generator=g).tolist()
        self.k = [(std * torch.randn(L, nkv, d, generator=g)).to(dtype) for L in lengths]
        self.v = [torch.randn(L, nkv, dv, generator=g).to(dtype) for L in lengths]
        self.q = [(std * torch.randn(n, nq, d, generator=g)).to(dtype) for n in counts]
        self.kc = (100.0 * torch.randn(S * per, nkv, page, d, generator=g)).to(dtype)      # stale numbers everywhere
        self.vc = (100.0 * torch.randn(S * per, nkv, page, dv, generator=g)).to(dtype)
        self.table = [[order[s * per + i] if i * page < lengths[s] else -1 for i in range(per)] for s in range(S)]
        self.page, self.dtype, self.dims = page, dtype, (nq, nkv, d, dv)
        self.pos = [list(range(L - n, L)) for L, n in zip(lengths, counts)]
        self._ctx = None

    def place(self):
        for s, L in enumerate(self.lengths):
            for p in range(L):
                pg = self.table[s][p // self.page]
                self.kc[pg, :, p % self.page] = self.k[s][p]
                self.vc[pg, :, p % self.page] = self.v[s][p]

    def ctx(self):
        from photon_infer_b200.parts.base import GroupView, StepContext
        self.place()
        S, T = len(self.lengths), sum(self.counts)
        width = max(8, -(-len(self.table[0]) // 8) * 8)
        bt = [row + [-1] * (width - len(row)) for row in self.table]
        pos = [p for ps in self.pos for p in ps]
        seq = [s for s, n in enumerate(self.counts) for _ in range(n)]
        cu = [0]
        for n in self.counts:
            cu.append(cu[-1] + n)
        starts = [L - n for L, n in zip(self.lengths, self.counts)]
        self.kcd, self.vcd = self.kc.to(DEV), self.vc.to(DEV)
        return StepContext(T, S, self.dtype, i32([0] * T), i32(pos), i32(seq), i32(cu), i32(self.lengths), i32(list(range(S))),
                           [GroupView(i32(bt), i32([0] * T), self.page, self.kc.shape[0], width)], self.counts, self.lengths,
                           starts, max(self.counts), max(self.lengths), torch.zeros(4, dtype=torch.int32, device=DEV))

    def want(self, scale, window, keep, sink, cap):
        return torch.cat([_oracle(self.q[s].double(), self.k[s].double(), self.v[s].double(), self.pos[s], scale, window, keep,
                                  sink, cap) for s in range(len(self.lengths))])

    def run(self, kernel, scale, window, keep, sink, cap, splits=1, gate=None):
        from photon_infer_b200.kernels import ops
        from photon_infer_b200.parts.attention import attend_tensor_cores
        from photon_infer_b200.parts.base import LayerCache
        nq, nkv, d, dv = self.dims
        ctx = self.ctx()
        q = torch.cat(self.q).reshape(-1, nq * d).to(DEV)
        out = torch.full((q.shape[0], nq * dv), float("nan"), dtype=self.dtype, device=DEV)
        if gate is not None:
            wide = torch.zeros(q.shape[0], nq * dv + 16, dtype=self.dtype, device=DEV)     # a view with a row stride, 16-byte aligned rows
            wide[:, 8:8 + nq * dv] = gate.to(DEV)
            gate = wide[:, 8:8 + nq * dv]
        if kernel == "general":
            ops.paged_attention(q, out, self.kcd, self.vcd, ctx.groups[0].block_table, ctx.token_seq, ctx.positions, nq, nkv, d,
                                window, scale, ctx.error_flag, value_dim=dv, splits=splits, keep_first=keep, sink=sink, softcap=cap,
                                gate=gate)
        else:
            mixer = types.SimpleNamespace(n_q=nq, n_kv=nkv, head_dim=d, window=window, scale=scale, _max_groups=None)
            attend_tensor_cores(mixer, q, out, ctx, LayerCache(group=0, k=self.kcd, v=self.vcd), keep_first=keep, sink=sink, softcap=cap,
                                gate=gate)
        torch.cuda.synchronize()
        assert ctx.error_flag.cpu().tolist()[0] == 0
        return out.float().cpu()


RULES = [dict(window=None, keep=0, sink=False, cap=None), dict(window=24, keep=0, sink=True, cap=None),
         dict(window=40, keep=5, sink=False, cap=6.0), dict(window=8, keep=11, sink=False, cap=None),
         dict(window=3, keep=1, sink=True, cap=9.0), dict(window=70, keep=0, sink=True, cap=4.0),
         dict(window=64, keep=64, sink=False, cap=None), dict(window=130, keep=70, sink=True, cap=2.5)]
# a whole short prompt, the end of a long one, single decoded tokens near and far, two tokens
LENGTHS, COUNTS = [33, 150, 97, 200, 1, 300], [33, 50, 1, 2, 1, 1]


@pytest.mark.parametrize("rule", RULES, ids=lambda r: f"w{r['window']}k{r['keep']}s{int(r['sink'])}c{r['cap']}")
@pytest.mark.parametrize("heads", [(2, 1), (6, 2), (2, 2), (8, 1), (5, 1)])
@pytest.mark.parametrize("kernel,dtype,d,dv,page", [("general", torch.float32, 10, 14, 8), ("general", torch.float32, 64, 64, 16),
                                                    ("general", torch.bfloat16, 24, 8, 16), ("tensor", torch.bfloat16, 64, 64, 16),
                                                    ("tensor", torch.bfloat16, 128, 128, 16), ("tensor", torch.bfloat16, 64, 64, 64),
                                                    ("tensor", torch.bfloat16, 32, 32, 8), ("tensor", torch.bfloat16, 48, 48, 16),
                                                    ("tensor", torch.bfloat16, 96, 96, 32), ("general", torch.bfloat16, 256, 64, 16)])
def test_attention_rules_in_every_kernel(rule, heads, kernel, dtype, d, dv, page):
    nq, nkv = heads
    st = _Step(LENGTHS, COUNTS, nq, nkv, d, dv, page, dtype, seed=nq * 100 + d, std=1.0 if d < 64 else 0.5)
    scale = 1.3 / math.sqrt(d)
    # with bounded scores (the second kind of mixer) the heads' outputs are gated in the kernel's epilogue as well
    gate = (2.0 * torch.randn(sum(COUNTS), nq * dv, generator=torch.Generator().manual_seed(d))).to(dtype) if rule["cap"] else None
    got = st.run("general" if kernel == "general" else "tc", scale, rule["window"], rule["keep"], rule["sink"], rule["cap"], gate=gate)
    want = st.want(scale, rule["window"], rule["keep"], rule["sink"], rule["cap"])
    if gate is not None:
        want = want * torch.sigmoid(gate.double())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    per_row = (got.double() - want).abs().amax(dim=1) / float(want.abs().max())
    assert float(per_row.max()) < tol, f"rows off: {(per_row >= tol).nonzero().flatten().tolist()[:10]}, worst {float(per_row.max()):.3g}"


@pytest.mark.parametrize("rule", RULES[1:6], ids=lambda r: f"w{r['window']}k{r['keep']}s{int(r['sink'])}c{r['cap']}")
def test_attention_with_keys_split_over_blocks(rule):
    """Decoded tokens only, long contexts: the general kernel shares a token's keys out over blocks and merges; the
    sink enters the merged denominator once."""
    st = _Step([700, 1, 333, 520], [1, 1, 1, 1], 4, 2, 24, 8, 16, torch.bfloat16, seed=3)
    want = st.want(0.3, rule["window"], rule["keep"], rule["sink"], rule["cap"])
    gate = (2.0 * torch.randn(4, 4 * 8, generator=torch.Generator().manual_seed(8))).to(torch.bfloat16)
    for splits in (1, 3, 64):
        got = st.run("general", 0.3, rule["window"], rule["keep"], rule["sink"], rule["cap"], splits=splits)
        assert rel_err(got, want) < 2e-2
        got = st.run("general", 0.3, rule["window"], rule["keep"], rule["sink"], rule["cap"], splits=splits, gate=gate)
        assert rel_err(got, want * torch.sigmoid(gate.double())) < 2e-2


@pytest.mark.parametrize("kernel,dtype,d,page", [("general", torch.float32, 12, 8), ("general", torch.bfloat16, 64, 16),
                                                 ("tensor", torch.bfloat16, 64, 16), ("tensor", torch.bfloat16, 128, 32)])
@pytest.mark.parametrize("count", [1, 40])
@pytest.mark.parametrize("sink", [False, True])
def test_keys_that_stand_out_at_every_edge(kernel, dtype, d, page, count, sink):
    """Random keys score about 0.  One key at a time is made to score high for the LAST token of a request of 333
    tokens (decoded alone, or the end of a portion of 40): far back (no window), the first and the last key the
    window holds, the key just behind it, the last kept first key and the one after it, keys at both sides of a
    page border.  The output must be that key's value where the rules let the token see it, and the oracle's
    output where they do not."""
    L, window, keep = 333, 96, 6
    i = L - 1
    places = {"far": (1, None, 0), "window_first": (i - window + 1, window, 0), "window_behind": (i - window, window, 0),
              "self": (i, window, 0), "kept_last": (keep - 1, window, keep), "kept_behind": (keep, window, keep),
              "page_low": ((i - 40) // page * page - 1, window, keep), "page_high": ((i - 40) // page * page, window, keep)}
    for name, (j, w, kf) in places.items():
        st = _Step([L, 50], [count, 1], 2, 1, d, d, page, dtype, seed=len(name), std=0.05)
        qdir = st.q[0][-1, 0].double()
        st.k[0][j, 0] = (qdir / qdir.norm() * 40.0).to(dtype)          # this key's score with head 0 of the last token: large
        marker = torch.full((d,), 7.0).to(dtype)
        st.v[0][j, 0] = marker
        scale = 1.0 / float(qdir.norm())                               # score = 40
        got = st.run("general" if kernel == "general" else "tc", scale, w, kf, sink, None)
        want = st.want(scale, w, kf, sink, None)
        visible = j <= i and (w is None or i - j < w or j < kf)
        row = got[count - 1, :d]
        assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 2e-2), name
        if visible:
            assert float((row - 7.0).abs().max()) < 0.1, f"{name}: key {j} must be seen"
        else:
            assert float(row.abs().max()) < 3.0, f"{name}: key {j} must not be seen"


# ----------------------------------------------------------------------------- the mixer as a whole

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
@pytest.mark.parametrize("shape", [dict(heads=4, kv_heads=2, dim=64, vdim=64, size=24, keep_first=5, rot=(5000.0, 16), softcap=6.0),
                                   dict(heads=3, kv_heads=1, dim=10, vdim=14, size=7, keep_first=9, rot=(100.0, 10), softcap=None),
                                   dict(heads=2, kv_heads=2, dim=128, vdim=128, size=None, keep_first=None, rot=None, softcap=3.0)])
def test_mixer_in_portions(dtype, kind, shape):
    """One request through the mixer in steps of 30, 2, 1, 1, 17, 1 tokens against the plain mixer over the whole
    sequence."""
    from photon_infer_b200.config.fekopel_config import FekopelConfig
    from photon_infer_b200.models.fekopel import _mixer
    from photon_infer_b200.parts.base import GroupView, LayerCache, StepContext
    from photon_infer_b200.parts.registry import create_part
    H = 48
    m = dict(heads=shape["heads"], kv_heads=shape["kv_heads"], dim=shape["dim"], vdim=shape["vdim"], scale=0.9 / math.sqrt(shape["dim"]))
    if shape["size"]:
        m["mask"] = dict(size=shape["size"])
        if kind == "attention_2" and shape["keep_first"] is not None:
            m["mask"]["keep_first"] = shape["keep_first"]
    if kind == "attention_2":
        if shape["rot"]:
            m["rot"] = dict(base=shape["rot"][0], dims=shape["rot"][1])
        if shape["softcap"]:
            m["softcap"] = shape["softcap"]
    cfg = types.SimpleNamespace(width=H, norm_eps=1e-5)
    spec = _mixer(cfg, kind, m)
    att = create_part("mixer", spec.kind, spec.params)
    w = _weights(att, dtype, 0.3, 5)
    n, page = 52, 16
    h = torch.randn(n, H, generator=torch.Generator().manual_seed(6)).to(dtype)
    want = (plain.mixer_attention if kind == "attention" else plain.mixer_attention_2)(h.double(), m, w, 1e-5)
    pages = -(-n // page)
    cs = att.cache_spec()
    kc = torch.zeros(pages, cs.n_kv_heads, page, cs.head_dim, dtype=dtype, device=DEV)
    vc = torch.zeros(pages, cs.n_kv_heads, page, cs.value_dim or cs.head_dim, dtype=dtype, device=DEV)
    got, p = [], 0
    for cnt in (30, 2, 1, 1, 17, 1):
        pos = list(range(p, p + cnt))
        ctx = StepContext(cnt, 1, dtype, i32([0] * cnt), i32(pos), i32([0] * cnt), i32([0, cnt]), i32([p + cnt]), i32([0]),
                          [GroupView(i32([list(range(pages)) + [-1] * (8 - pages)]), i32(pos), page, pages, 8)], [cnt], [p + cnt], [p],
                          cnt, p + cnt, torch.zeros(4, dtype=torch.int32, device=DEV))
        got.append(att.forward(h[p:p + cnt].to(DEV), ctx, LayerCache(group=0, k=kc, v=vc)).float().cpu())
        assert ctx.error_flag.cpu().tolist()[0] == 0
        p += cnt
    assert rel_err(torch.cat(got), want) < (2e-5 if dtype == torch.float32 else 2.5e-2)


# ----------------------------------------------------------------------------- router and experts

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [dict(E=16, top=4, groups=(4, 3), scale=1.5), dict(E=6, top=2, groups=(3, 1), scale=0.5),
                                   dict(E=5, top=5, groups=None, scale=2.0), dict(E=8, top=1, groups=(8, 2), scale=1.0),
                                   dict(E=12, top=3, groups=(1, 1), scale=1.0),
                                   dict(E=40, top=3, groups=(5, 2), scale=0.7), dict(E=32, top=32, groups=(4, 4), scale=1.0),
                                   dict(E=140, top=2, groups=(70, 3), scale=1.0)])   # more experts than lanes: one thread walks them
def test_router_with_groups(dtype, shape):
    from photon_infer_b200.kernels import ops
    E, top, H, T = shape["E"], shape["top"], 40, 64
    g = torch.Generator().manual_seed(E)
    h = torch.randn(T, H, generator=g).to(dtype)
    wr = (0.5 * torch.randn(E, H, generator=g)).to(dtype)
    wsg = torch.randn(1, H, generator=g).to(dtype)
    m = dict(router=dict(experts=E, top=top, scale=shape["scale"]))
    if shape["groups"]:
        m["router"]["groups"] = dict(count=shape["groups"][0], keep=shape["groups"][1])
    cnt, keep = shape["groups"] or (1, 1)
    ids, weights, counts, gate = ops.moe_route(h.to(DEV), wr.to(DEV), None, top, "softmax_all", cnt, keep, shape["scale"], wsg.to(DEV))
    want_ids, want_w = plain.route(h.double(), m, {"router": wr.double()})
    assert torch.equal(ids.cpu().long(), want_ids)
    assert rel_err(weights.cpu(), want_w) < 1e-5
    assert rel_err(gate.cpu(), torch.sigmoid(h.double() @ wsg.double().T)[:, 0]) < 1e-5
    assert counts.cpu().tolist() == torch.bincount(want_ids.flatten(), minlength=E).tolist()


def test_router_ties_go_to_the_lower_index():
    """Equal rows of the router give equal scores: the lower expert wins in the choice of groups and of experts."""
    from photon_infer_b200.kernels import ops
    h = torch.randn(5, 16, generator=torch.Generator().manual_seed(1))
    row = torch.randn(16, generator=torch.Generator().manual_seed(2))
    wr = row.repeat(8, 1)
    ids, weights, _ = ops.moe_route(h.to(DEV), wr.to(DEV), None, 3, "softmax_all", 4, 2, 1.0)
    assert ids.cpu().tolist() == [[0, 1, 2]] * 5
    assert rel_err(weights.cpu(), torch.full((5, 3), 1.0 / 3).double()) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [3, 40, 300])                 # one product per pair; the grouped kernel; the library's grouped product
@pytest.mark.parametrize("shape", [dict(E=6, top=2, ff=24, shared=40, groups=(3, 2), H=64), dict(E=4, top=4, ff=16, shared=None, groups=None, H=48),
                                   dict(E=7, top=3, ff=10, shared=14, groups=None, H=50)])
def test_plain_experts_on_every_path(dtype, rows, shape):
    from photon_infer_b200.config.fekopel_config import FekopelConfig
    from photon_infer_b200.models.fekopel import _feed_forward
    from photon_infer_b200.parts.registry import create_part
    m = dict(kind="moe", router=dict(experts=shape["E"], top=shape["top"], scale=1.5), expert=dict(ff=shape["ff"]))
    if shape["groups"]:
        m["router"]["groups"] = dict(count=shape["groups"][0], keep=shape["groups"][1])
    if shape["shared"]:
        m["shared"] = dict(ff=shape["shared"])
    spec = _feed_forward(types.SimpleNamespace(width=shape["H"]), m)
    ff = create_part("feed_forward", spec.kind, spec.params)
    w = _weights(ff, dtype, 0.3, 11)
    h = torch.randn(rows, shape["H"], generator=torch.Generator().manual_seed(12)).to(dtype)
    got = ff.forward(h.to(DEV), None).float().cpu()
    want = plain.moe(h.double(), m, w)
    per_row = (got.double() - want).abs().amax(dim=1) / float(want.abs().max())
    if dtype == torch.float32:
        assert float(per_row.max()) < 1e-5
    else:
        # bfloat16 products of bfloat16 inputs agree with the oracle on the experts (the router sees the same numbers)
        assert float(per_row.max()) < 2.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [5, 70, 400])
def test_experts_that_nobody_chooses(dtype, rows):
    """Two of eight experts never win (their router rows point away from every input): their groups of rows are
    empty on every path, and the others' results do not move."""
    from photon_infer_b200.models.fekopel import _feed_forward
    from photon_infer_b200.parts.registry import create_part
    H = 64
    m = dict(kind="moe", router=dict(experts=8, top=1, scale=1.0), expert=dict(ff=32))
    spec = _feed_forward(types.SimpleNamespace(width=H), m)
    ff = create_part("feed_forward", spec.kind, spec.params)
    g = torch.Generator().manual_seed(21)
    w = {t.name: (0.3 * torch.randn(t.concrete_shape(), generator=g)) for t in ff.tensor_specs()}
    w["router"][:, 0] = 2.0
    w["router"][3, 0] = w["router"][5, 0] = -2.0
    w = {k: v.to(dtype) for k, v in w.items()}
    ff.load({k: v.to(DEV) for k, v in w.items()})
    h = torch.randn(rows, H, generator=g)
    h[:, 0] = 5.0
    h = h.to(dtype)
    wd = {k: v.double() for k, v in w.items()}
    ids, _ = plain.route(h.double(), m, wd)
    assert not ((ids == 3) | (ids == 5)).any()
    got = ff.forward(h.to(DEV), None).float().cpu()
    assert rel_err(got, plain.moe(h.double(), m, wd)) < (1e-5 if dtype == torch.float32 else 2.5e-2)
