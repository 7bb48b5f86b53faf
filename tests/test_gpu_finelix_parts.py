"""Each mechanism of the Finelix decoder alone, on the device, against its plain function: the norm that adds two
pending outputs, the gated feed-forward with gelu, the entrance of a looped block, attention over a cached latent
(in portions, with keys that are made to stand out far back, at page borders and at the start), gated linear
attention (in portions down to one token, with its state in slots that are used again), the routed experts and the
sort that feeds them, and the per-head products."""
import math

import pytest
import torch

from helpers import rel_err
from plain import finelix_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOLS = {torch.float32: 5e-6, torch.bfloat16: 2e-2}


def _ctx(tokens_per_seq, starts, page_size, dtype, pages_per_seq=8, slots=None):
    """A hand-made StepContext: request i owns pages i * pages_per_seq .. in order."""
    from photon_infer_b200.parts.base import GroupView, StepContext
    T, S = sum(tokens_per_seq), len(tokens_per_seq)
    pos, seq, sm = [], [], []
    for s, (n, st) in enumerate(zip(tokens_per_seq, starts)):
        for p in range(st, st + n):
            pos.append(p); seq.append(s); sm.append((s * pages_per_seq + p // page_size) * page_size + p % page_size)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    bt = i32([[s * pages_per_seq + i for i in range(pages_per_seq)] for s in range(S)])
    cu = [0]
    for n in tokens_per_seq:
        cu.append(cu[-1] + n)
    ends = [a + b for a, b in zip(tokens_per_seq, starts)]
    return StepContext(T, S, dtype, i32([0] * T), i32(pos), i32(seq), i32(cu), i32(ends),
                       i32(list(range(S)) if slots is None else slots),
                       [GroupView(bt, i32(sm), page_size, S * pages_per_seq, pages_per_seq)], tokens_per_seq, ends, starts,
                       max(tokens_per_seq), max(ends), torch.zeros(4, dtype=torch.int32, device=DEV))


def _weights(part, dtype, std, seed):
    g = torch.Generator().manual_seed(seed)
    w = {}
    for t in part.tensor_specs():
        shape = t.concrete_shape()
        x = std * torch.randn(shape, generator=g)
        if t.init == "norm":
            x = 1.0 + x
        w[t.name] = x.to(dtype)
    part.load({k: v.to(DEV) for k, v in w.items()})
    return {k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_adds_two_pending_outputs(dtype):
    from photon_infer_b200.parts.registry import create_part
    torch.manual_seed(0)
    norm = create_part("norm", "rms_norm", {"size": 72, "eps": 1e-5, "weight_name": "w"})
    w = (1 + 0.1 * torch.randn(72)).to(dtype)
    norm.load({"w": w.to(DEV)})
    x, a, b = torch.randn(6, 72), torch.randn(6, 72).to(dtype), torch.randn(6, 72).to(dtype)
    res = x.to(DEV).clone()
    out = norm.add_forward((a.to(DEV), b.to(DEV)), res, dtype)
    want_x = x.double() + (a.double() + b.double())
    assert rel_err(res.cpu(), want_x) < 1e-6
    assert rel_err(out.float().cpu(), plain.rms_norm(want_x, 1e-5, w.double())) < (2e-6 if dtype == torch.float32 else 6e-3)
    rows = torch.tensor([4, 1], dtype=torch.int32, device=DEV)
    res2 = x.to(DEV).clone()
    out2 = norm.add_forward_rows((a.to(DEV), b.to(DEV)), res2, rows, dtype)
    assert torch.equal(res2.cpu(), x) and torch.equal(out2, out[[4, 1]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [3, 40])
def test_gated_feed_forward_with_gelu(dtype, rows):
    from photon_infer_b200.parts.registry import create_part
    ff = create_part("feed_forward", "gated", dict(hidden_size=56, intermediate_size=88, activation="gelu_tanh",
                                                   names=("gate", "up", "down")))
    w = _weights(ff, dtype, 0.2, 1)
    h = torch.randn(rows, 56, generator=torch.Generator().manual_seed(2)).to(dtype)
    out = ff.forward(h.to(DEV), None)
    want = plain.gated_feed_forward(w["gate"], w["up"], w["down"], plain.gelu_tanh, h.double())
    assert rel_err(out.float().cpu(), want) < TOLS[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_loop_input(dtype):
    from photon_infer_b200.parts.registry import create_part
    part = create_part("stream", "loop_input", dict(hidden_size=40, times=3))
    w = _weights(part, dtype, 0.15, 3)
    g = torch.Generator().manual_seed(4)
    x, x0 = torch.randn(5, 40, generator=g), torch.randn(5, 40, generator=g)
    a, b = torch.randn(5, 40, generator=g).to(dtype), torch.randn(5, 40, generator=g).to(dtype)
    for t in (0, 2):
        out = part.forward(x.to(DEV).clone(), (a.to(DEV), b.to(DEV)), x0.to(DEV), t, None)
        want = plain.loop_input(w["in"], w["step"], x.double() + a.double() + b.double(), x0.double(), t)
        assert out.dtype == torch.float32 and rel_err(out.cpu(), want) < TOLS[dtype]
    with pytest.raises(IndexError):
        part.forward(x.to(DEV), None, x0.to(DEV), 3, None)


def _latent_part(dtype, heads=3, dim=16, rot=8, vdim=20, kv_rank=32, q_rank=24, H=48, base=10000.0, seed=5, rot_dims=None):
    from photon_infer_b200.parts.registry import create_part
    rot_dims = rot if rot_dims is None else rot_dims
    m = dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=(dim + rot) ** -0.5,
             rot=dict(base=base, dims=rot_dims))
    att = create_part("mixer", "latent_attention", dict(hidden_size=H, heads=heads, dim=dim, rot_dim=rot, vdim=vdim,
                                                        kv_rank=kv_rank, q_rank=q_rank, scale=m["scale"], eps=1e-5,
                                                        rot_base=base, rot_dims=rot_dims))
    return att, m, _weights(att, dtype, 0.3, seed)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [dict(), dict(heads=1, dim=24, rot=16, vdim=8, kv_rank=40, q_rank=8, base=1e6),
                                   dict(heads=2, dim=8, rot=16, vdim=8, kv_rank=24, q_rank=16, rot_dims=8),   # part of the rotated features turns
                                   dict(heads=3, dim=16, rot=16, vdim=20, kv_rank=32, q_rank=24)])            # widths of 16s: tensor-core decode
@pytest.mark.parametrize("long", [False, True])
def test_latent_attention_two_requests_in_portions(dtype, shape, long):
    """The mixer alone: two requests, each fed in three steps (a long portion, two tokens, single tokens), against
    dense attention over the whole sequence.  Only one row of kv_rank + rot_dim numbers per token is cached."""
    from photon_infer_b200.parts.base import LayerCache
    att, m, w = _latent_part(dtype, **shape)
    spec = att.cache_spec()
    assert (spec.n_kv_heads, spec.head_dim, spec.values) == (1, m["kv_rank"] + m["rot_dim"], False) and att.state_spec() is None
    ps = 4
    lens = [27, 14] if not long else [125, 60]
    g = torch.Generator().manual_seed(6)
    hs = [torch.randn(L, 48, generator=g).to(dtype) for L in lens]
    want = [plain.latent_attention(w, m, 1e-5, h.double()) for h in hs]
    cache = LayerCache(group=0, k=torch.full((64, 1, ps, spec.head_dim), float("nan"), dtype=dtype, device=DEV))
    got, starts = [[], []], [0, 0]
    # long: portions of 32 tokens and more take the products-and-softmax path in bfloat16, beside short ones in one step
    for cut in ([(17, 5), (2, 2), (1, 1), (7, 6)] if not long else [(40, 33), (2, 2), (48, 1), (35, 24)]):
        ctx = _ctx(list(cut), list(starts), ps, dtype, pages_per_seq=32)
        h = torch.cat([hs[i][starts[i]:starts[i] + cut[i]] for i in range(2)]).to(DEV)
        out = att.forward(h, ctx, cache).float().cpu()
        got[0].append(out[:cut[0]]); got[1].append(out[cut[0]:])
        starts = [starts[i] + cut[i] for i in range(2)]
        assert ctx.error_flag.cpu().tolist()[0] == 0
    for i in range(2):
        assert rel_err(torch.cat(got[i]), want[i]) < (1e-5 if dtype == torch.float32 else 2.5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("target", [0, 1, 15, 16, 17, 31, 32, 255, 256, 400, 598, 599])
def test_latent_rows_far_back_at_page_borders_and_at_the_start(dtype, target):
    """The attention kernel over rows that are key and value at once: among 600 cached rows ONE is made to fit the
    query (its score stands 12 above the rest), so the result is that row's head, whichever page it lies in: the
    first rows, the last, both sides of page borders, hundreds of rows back.  A decoded token (one row) and a
    portion whose last token asks."""
    from photon_infer_b200.kernels import ops
    heads, width, dv, ps, n = 5, 40, 28, 16, 600
    g = torch.Generator().manual_seed(target)
    rows = torch.randn(n, width, generator=g)
    rows = rows / rows.norm(dim=1, keepdim=True)
    q = torch.randn(heads, width, generator=g)
    q = q / q.norm(dim=1, keepdim=True)
    rows[target] = q.mean(0) / q.mean(0).norm()
    qs = 14.0 * rows[target].expand(heads, width).clone() + 0.1 * q
    pages = (n + ps - 1) // ps
    perm = torch.randperm(pages, generator=g)                                # the pages lie scattered in the pool
    cache = torch.zeros(pages, 1, ps, width)
    for p in range(n):
        cache[perm[p // ps], 0, p % ps] = rows[p]
    cache = cache.to(dtype).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    bt = i32([perm.tolist() + [-1] * 3])
    scores = (qs.to(dtype).double() @ cache.cpu().double().view(-1, width)[[int(perm[p // ps]) * ps + p % ps for p in range(n)]].T)
    want = torch.softmax(scores, dim=1) @ rows.to(dtype).double()[:, :dv]
    assert float(torch.softmax(scores, dim=1)[:, target].min()) > 0.5         # the test is about that row
    for tokens in (1, 3):
        qq = torch.zeros(tokens, heads * width)
        qq[-1] = qs.reshape(-1)
        out = torch.empty(tokens, heads * dv, dtype=dtype, device=DEV)
        err = torch.zeros(4, dtype=torch.int32, device=DEV)
        for splits in (1, 5, 64):                                                # the keys of a token shared out over blocks
            out.zero_()
            ops.paged_attention(qq.to(dtype).to(DEV), out, cache, cache, bt, i32([0] * tokens), i32(list(range(n - tokens, n))),
                                heads, 1, width, None, 1.0, err, value_dim=dv, splits=splits)
            assert err.cpu().tolist()[0] == 0
            assert rel_err(out[-1].float().cpu().view(heads, dv), want) < (1e-5 if dtype == torch.float32 else 1e-2)
    # one row less in the context: the row at the end is not seen by the token before it
    if target == n - 1:
        out = torch.empty(1, heads * dv, dtype=dtype, device=DEV)
        ops.paged_attention(qs.reshape(1, -1).to(dtype).to(DEV), out, cache, cache, bt, i32([0]), i32([n - 2]), heads, 1, width,
                            None, 1.0, None, value_dim=dv)
        want2 = torch.softmax(scores[:, :n - 1], dim=1) @ rows.to(dtype).double()[:n - 1, :dv]
        assert rel_err(out.float().cpu().view(heads, dv), want2) < (1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("heads", [5, 16, 20])
@pytest.mark.parametrize("target", [0, 1, 63, 64, 65, 127, 128, 300, 598, 599])
def test_latent_rows_on_the_tensor_cores(heads, target):
    """The same made-to-stand-out row for the tensor-core kernel of decoded tokens (one block per token and 64 rows): the
    borders of its blocks of 64 rows, the first rows and the last, with heads that fill part of a tile, one tile, and
    more; two tokens of different requests and lengths in one call."""
    from photon_infer_b200.kernels import ops
    width, dv, ps, n = 48, 32, 16, 600
    g = torch.Generator().manual_seed(1000 + target)
    rows = torch.randn(n, width, generator=g)
    rows = rows / rows.norm(dim=1, keepdim=True)
    q = torch.randn(heads, width, generator=g)
    rows[target] = q.mean(0) / q.mean(0).norm()
    qs = 14.0 * rows[target].expand(heads, width).clone() + 0.1 * q / q.norm(dim=1, keepdim=True)
    pages = (n + ps - 1) // ps
    perm = torch.randperm(pages, generator=g)
    cache = torch.zeros(pages, 1, ps, width)
    for p in range(n):
        cache[perm[p // ps], 0, p % ps] = rows[p]
    cache = cache.bfloat16().to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    bt = i32([perm.tolist(), perm.tolist()])
    rb, qb = rows.bfloat16().double(), qs.bfloat16().double()
    short = max(target + 1, 70)                                            # the second token's request is shorter
    qq = torch.stack([qs.reshape(-1), qs.reshape(-1)]).bfloat16().to(DEV)
    out = torch.empty(2, heads * dv, dtype=torch.bfloat16, device=DEV)
    err = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.latent_decode_attention(qq, out, cache, bt, i32([0, 1]), i32([n - 1, short - 1]), heads, width, dv, 1.0, n, err)
    assert err.cpu().tolist()[0] == 0
    for row, length in ((0, n), (1, short)):
        want = torch.softmax(qb @ rb[:length].T, dim=1) @ rb[:length, :dv]
        assert rel_err(out[row].float().cpu().view(heads, dv), want) < 1.5e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 16, 24, 4.0), (1, 72, 40, 16.0), (4, 8, 8, 1.0), (3, 12, 10, 2.0), (2, 128, 64, 8.0)])
@pytest.mark.parametrize("long", [False, True])
def test_gated_linear_attention_in_portions_and_slots_used_again(dtype, shape, long):
    """Two requests through the mixer in portions (long, two tokens, single tokens), their states in slots 2 and 0 of
    four; then a third request in slot 2 after it was cleared: the state is carried between steps, belongs to the
    slot and starts at zero.  ``long``: portions of 128 tokens and more, which in bfloat16 run their chunks of 64 side
    by side (from a zero state and from a carried one, with a last chunk that is not full), beside short ones."""
    from photon_infer_b200.parts.base import LayerCache
    from photon_infer_b200.parts.registry import create_part
    heads, dim, vdim, tau = shape
    H = 40
    mixer = create_part("mixer", "gla", dict(hidden_size=H, heads=heads, dim=dim, vdim=vdim, tau=tau, eps=1e-5, decay_rank=8))
    w = _weights(mixer, dtype, 0.3, 7)
    m = dict(heads=heads, dim=dim, vdim=vdim, tau=tau)
    assert mixer.cache_spec() is None and mixer.state_spec().shape == (heads, dim, vdim)
    state = torch.full((4, heads, dim, vdim), 3.0, dtype=torch.float32, device=DEV)      # stale values of earlier owners
    cache = LayerCache(state=state)
    g = torch.Generator().manual_seed(8)
    lens = [33, 21] if not long else [341, 150]
    hs = [torch.randn(L, H, generator=g).to(dtype) for L in lens]
    want = [plain.gated_linear_attention(w, m, 1e-5, h.double()) for h in hs]
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2
    slots = [2, 0]
    for s in slots:
        state[s].zero_()                                                             # what the slot pool does at hand-out
    got, starts = [[], []], [0, 0]
    for cut in ([(19, 4), (2, 2), (1, 1), (1, 1), (10, 13)] if not long else [(170, 4), (2, 2), (1, 128), (168, 16)]):
        ctx = _ctx(list(cut), list(starts), 16, dtype, slots=slots, pages_per_seq=32)
        h = torch.cat([hs[i][starts[i]:starts[i] + cut[i]] for i in range(2)]).to(DEV)
        out = mixer.forward(h, ctx, cache).float().cpu()
        got[0].append(out[:cut[0]]); got[1].append(out[cut[0]:])
        starts = [starts[i] + cut[i] for i in range(2)]
    for i in range(2):
        assert rel_err(torch.cat(got[i]), want[i]) < tol
    assert torch.all(state[1] == 3.0) and torch.all(state[3] == 3.0)                 # slots of others are untouched
    state[2].zero_()
    h3 = torch.randn(9, H, generator=g).to(dtype)
    out = mixer.forward(h3.to(DEV), _ctx([9], [0], 16, dtype, slots=[2]), cache).float().cpu()
    assert rel_err(out, plain.gated_linear_attention(w, m, 1e-5, h3.double())) < tol


def test_gated_linear_attention_forgets_at_the_rate_of_its_decay():
    """A decay that is made strong on purpose (large negative bias, tau 1) wipes the state within a few tokens, a weak
    one keeps it: the output at the last token does or does not depend on the first tokens."""
    from photon_infer_b200.parts.base import LayerCache
    from photon_infer_b200.parts.registry import create_part
    H, heads, dim, vdim = 32, 2, 16, 16
    g = torch.Generator().manual_seed(9)
    h = torch.randn(40, H, generator=g)
    h2 = h.clone(); h2[:8] = torch.randn(8, H, generator=g)
    outs = {}
    for bias in (-8.0, 8.0):
        mixer = create_part("mixer", "gla", dict(hidden_size=H, heads=heads, dim=dim, vdim=vdim, tau=1.0, eps=1e-5, decay_rank=4))
        w = _weights(mixer, torch.float32, 0.2, 10)
        w["a2.b"] = torch.full_like(w["a2.b"], bias)
        mixer.load({k: v.float().to(DEV) for k, v in w.items()})
        for name, x in (("a", h), ("b", h2)):
            state = torch.zeros(1, heads, dim, vdim, device=DEV)
            out = mixer.forward(x.to(DEV), _ctx([40], [0], 16, torch.float32, slots=[0]), LayerCache(state=state)).cpu()
            want = plain.gated_linear_attention(w, dict(heads=heads, dim=dim, vdim=vdim, tau=1.0), 1e-5, x.double())
            assert rel_err(out, want) < 2e-5
            outs[(bias, name)] = out[-1]
    assert rel_err(outs[(-8.0, "a")], outs[(-8.0, "b")].double()) < 1e-5            # forgotten
    assert rel_err(outs[(8.0, "a")], outs[(8.0, "b")].double()) > 1e-2              # remembered


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 2, 32, 48, 37), (3, 3, 40, None, 5), (5, 1, 24, 16, 1), (9, 4, 8, 8, 70)])
def test_routed_experts(dtype, shape):
    from photon_infer_b200.parts.registry import create_part
    experts, top, ff_size, shared, rows = shape
    H = 56
    ff = create_part("feed_forward", "moe", dict(hidden_size=H, experts=experts, top=top, expert_size=ff_size, shared_size=shared))
    w = _weights(ff, dtype, 0.25, 11)
    # router logits well apart (the steps between them beat the rounding of bfloat16 activations)
    w["router"] = (w["router"] * 6).to(dtype).double()
    ff.load({k: v.to(dtype).to(DEV) for k, v in w.items()})
    h = torch.randn(rows, H, generator=torch.Generator().manual_seed(12)).to(dtype)
    out = ff.forward(h.to(DEV), None)
    m = dict(router=dict(experts=experts, top=top), shared=dict(ff=shared) if shared else None)
    want = plain.routed_experts(w, m, h.double())
    per_row = (out.float().cpu().double() - want).abs().amax(dim=1) / float(want.abs().max())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert int((per_row > tol).sum()) <= (0 if dtype == torch.float32 else max(1, rows // 20)), float(per_row.max())


def test_sort_by_expert_is_stable_and_complete():
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(13)
    T, H, E, top = 300, 32, 7, 3
    h, wr, b = torch.randn(T, H, generator=g), torch.randn(E, H, generator=g), torch.randn(E, generator=g)
    ids, weights, counts = ops.moe_route(h.to(DEV), wr.to(DEV), b.to(DEV), top)
    z = h.double() @ wr.double().T + b.double()
    tv, ti = torch.topk(z, top, dim=1)
    assert torch.equal(ids.cpu().long(), ti) and rel_err(weights.cpu(), torch.softmax(tv, dim=1)) < 1e-5
    assert torch.equal(counts.cpu().long(), torch.bincount(ti.flatten(), minlength=E))
    offsets, srt, place, tiles, num_tiles, max_tiles = ops.moe_align(ids, counts)
    flat = ids.cpu().flatten().long()
    order = torch.sort(flat, stable=True).indices
    assert torch.equal(srt.cpu().long(), order)
    assert torch.equal(place.cpu().long()[order], torch.arange(T * top))
    assert offsets.cpu().tolist() == [0] + torch.cumsum(counts.cpu(), 0).tolist()
    n_t = int(num_tiles.cpu())
    assert n_t <= max_tiles
    covered = []
    for e, r0, n in tiles.cpu()[:n_t].tolist():
        assert 0 < n <= ops.moe_tile_rows() and all(int(flat[order[r]]) == e for r in range(r0, r0 + n))
        covered += list(range(r0, r0 + n))
    assert covered == list(range(T * top))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 7, 50])
def test_products_per_head(dtype, rows):
    from photon_infer_b200.kernels import ops
    g = torch.Generator().manual_seed(14)
    heads, K, N = 3, 20, 36
    x = torch.randn(rows, heads, K + 4, generator=g).to(dtype)
    w = (0.3 * torch.randn(heads, N, K, generator=g)).to(dtype)
    out = torch.zeros(rows, heads, N + 8, dtype=dtype, device=DEV)
    ops.head_linear(x.to(DEV)[:, :, :K], w.to(DEV), out[:, :, :N])
    want = torch.einsum("thk,hnk->thn", x[:, :, :K].double(), w.double())
    assert rel_err(out[:, :, :N].float().cpu(), want) < TOLS[dtype]
    assert torch.all(out[:, :, N:] == 0)
