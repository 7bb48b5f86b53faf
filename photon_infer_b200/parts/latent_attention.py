"""Attention over a cached latent (multi-head latent attention).

Queries go through a latent of their own: ``c_q = rmsnorm(W_dq h)``, ``q = W_uq c_q``, every head laid out as
``[dim unrotated | rot_dim rotated]``.  Keys and values come from ONE latent per token: ``W_dkv h`` has
``kv_rank + rot_dim`` rows, the first ``kv_rank`` (RMS-normed) are the latent ``c``, the last ``rot_dim`` (not
normed, rotated by the token's position) are a key part ``k_r`` that all heads share.  Head ``h`` has the
unrotated key ``W_uk[h] c`` and the value ``W_uv[h] c``; its score against a key is
``(q_u . W_uk[h] c + q_r . k_r) * scale``, softmax over the keys up to the token's own position.

Only ``[c ; k_r]`` is cached, one row of ``kv_rank + rot_dim`` numbers per token and layer, and neither keys nor
values are ever formed: ``q_u . W_uk[h] c = (W_uk[h]^T q_u) . c``, so the queries are taken into the latent space
once per step (``head_linear``), attention runs with ONE key/value head whose key rows are ``[c ; k_r]`` and
whose values are the first ``kv_rank`` numbers of the same rows, and ``W_uv[h]`` is applied to the head's
weighted sum of latents.  A prompt portion, a decoded token and a mixed batch are the same case.

The rotation turns the first ``rot_dims`` numbers of the rotated part, feature ``i`` paired with
``i + rot_dims / 2``, by the angle ``position * base^(-2i / rot_dims)``; the rest passes unchanged.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, PagedCacheSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer


class LatentAttention(Mixer):
    kernel_modules = ("latent", "attention")

    def __init__(self, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int,
                 scale: float, eps: float, rot_base: float, rot_dims: Optional[int] = None, window: Optional[int] = None):
        self.hidden_size, self.heads, self.dim, self.rot_dim, self.vdim = hidden_size, heads, dim, rot_dim, vdim
        self.kv_rank, self.q_rank = kv_rank, q_rank
        self.scale, self.eps = float(scale), float(eps)
        self.rot_base = float(rot_base)
        self.rot_dims = rot_dim if rot_dims is None else int(rot_dims)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= rot_dim:
            raise ValueError("the rotated features must be an even number of at most rot_dim")
        self.window = window
        self.width = kv_rank + rot_dim          # one cached row
        half = self.rot_dims // 2
        self.inv_freq_host = torch.tensor([self.rot_base ** (-2.0 * i / self.rot_dims) for i in range(half)],
                                          dtype=torch.float64).to(torch.float32)
        self.inv_freq: Optional[torch.Tensor] = None
        self.w_down = self.w_uq = self.w_absorb = self.w_uv = self.w_o = None
        self.q_norm = self.kv_norm = None

    def required_kernels(self, dtype):
        mods = list(self.kernel_modules)
        if dtype == torch.bfloat16:
            mods.extend(["gemm_skinny", "gemm_tc", "gemm_tc2"])
        return mods

    def tensor_specs(self) -> List[TensorSpec]:
        H, n, d, r, v = self.hidden_size, self.heads, self.dim, self.rot_dim, self.vdim
        return [TensorSpec("dq", (self.q_rank, H)), TensorSpec("dq.norm", (self.q_rank,), role="vector", init="norm"),
                TensorSpec("uq", (n * (d + r), self.q_rank)),
                TensorSpec("dkv", (self.kv_rank + r, H)), TensorSpec("dkv.norm", (self.kv_rank,), role="vector", init="norm"),
                TensorSpec("uk", (n * d, self.kv_rank)), TensorSpec("uv", (n * v, self.kv_rank)),
                TensorSpec("o", (H, n * v))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n, d, v = self.heads, self.dim, self.vdim
        self.w_down = torch.cat([tensors["dq"], tensors["dkv"]], dim=0).contiguous()      # h is read once
        self.q_norm, self.kv_norm = tensors["dq.norm"].contiguous(), tensors["dkv.norm"].contiguous()
        self.w_uq = tensors["uq"].contiguous()
        # W_uk[h]^T as the [out, in] matrix of the product that takes a head's unrotated query into the latent space
        self.w_absorb = tensors["uk"].view(n, d, self.kv_rank).transpose(1, 2).contiguous()   # [heads, kv_rank, dim]
        self.w_uv = tensors["uv"].view(n, v, self.kv_rank).contiguous()                       # [heads, vdim, kv_rank]
        self.w_o = tensors["o"].contiguous()
        self.inv_freq = self.inv_freq_host.to(self.w_o.device)

    def weight_bytes(self) -> int:
        ws = (self.w_down, self.w_uq, self.w_absorb, self.w_uv, self.w_o)
        return sum(w.numel() * w.element_size() for w in ws)

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(1, self.width, self.window, values=False)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        n, d, r, kr = self.heads, self.dim, self.rot_dim, self.kv_rank
        group = ctx.groups[cache.group]
        down = project(h, self.w_down)                                   # [T, q_rank + kv_rank + rot]
        cq = torch.empty((T, self.q_rank), dtype=h.dtype, device=h.device)
        ops.latent_prep(down, self.q_rank, kr, r, self.rot_dims, self.q_norm, self.kv_norm, self.eps, ctx.positions,
                        self.inv_freq, group.slot_mapping, cq, cache.k, ctx.error_flag)
        q = project(cq, self.w_uq)                                       # [T, heads * (dim + rot)]
        q_lat = torch.empty((T, n, self.width), dtype=h.dtype, device=h.device)
        ops.head_linear(q.view(T, n, d + r)[:, :, :d], self.w_absorb, q_lat[:, :, :kr])
        ops.latent_q_rope(q, n, d, r, self.rot_dims, ctx.positions, self.inv_freq, q_lat, kr)
        o_lat = torch.empty((T, n * kr), dtype=h.dtype, device=h.device)
        self.attend(q_lat, o_lat, ctx, cache)
        o = torch.empty((T, n, self.vdim), dtype=h.dtype, device=h.device)
        ops.head_linear(o_lat.view(T, n, kr), self.w_uv, o)
        return project(o.view(T, n * self.vdim), self.w_o)


    def attend(self, q_lat: torch.Tensor, o_lat: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        """Decoded tokens, short portions and the float32 run: the paged kernel, whose sums depend only on a token's
        position.  A long bfloat16 portion: the request's cached rows are gathered into one matrix and attention
        is three steps per slab of queries, scores = Q C^T (library product, 32-bit out), a causal softmax over the
        rows, and P C[:, :kv_rank] (library product); a slab ends at the last key its queries may see."""
        T, n, kr = q_lat.shape[0], self.heads, self.kv_rank
        group = ctx.groups[cache.group]
        lens = list(ctx.host_query_lens) or [T]
        long_rows = [q_lat.dtype == torch.bfloat16 and self.window is None and m >= LIBRARY_MIN_TOKENS for m in lens]
        t = 0
        pending = None                                  # a run of neighbouring requests for the paged kernel
        for s, m in enumerate(lens):
            if long_rows[s]:
                if pending is not None:
                    self._paged(q_lat, o_lat, ctx, cache, pending, t)
                    pending = None
                self._dense(q_lat[t:t + m], o_lat[t:t + m], ctx.host_start_positions[s], group.block_table[s], cache, ctx)
            elif pending is None:
                pending = t
            t += m
        if pending is not None:
            self._paged(q_lat, o_lat, ctx, cache, pending, T)

    def _paged(self, q_lat, o_lat, ctx, cache, a: int, b: int) -> None:
        n = self.heads
        group = ctx.groups[cache.group]
        q2 = q_lat[a:b].view(b - a, n * self.width)
        shares = -(-max(ctx.max_context_len, 1) // 64)
        if self.window is None and ops.latent_decode_supported(q2, self.width, self.kv_rank) \
                and (b - a) * n * shares * (self.kv_rank + 2) * 4 <= DECODE_SHARES_BYTES:
            # bfloat16 with widths that fit the tensor cores' tiles: one block per token and 64 cached rows
            ops.latent_decode_attention(q2, o_lat[a:b], cache.k, group.block_table, ctx.token_seq[a:b], ctx.positions[a:b], n,
                                        self.width, self.kv_rank, self.scale, ctx.max_context_len, ctx.error_flag)
            return
        splits = 1
        if q_lat.dtype == torch.bfloat16:
            # few tokens with long contexts: share every token's key tiles out until the GPU is full (the float32 run keeps
            # one block per token, whose sums depend on the token's position alone)
            chunks = -(-n // max(1, min(n, 4096 // self.width)))
            tiles = -(-max(ctx.max_context_len, 1) // 32)
            splits = max(1, min(4 * ops.sm_count(q_lat.device) // max(1, (b - a) * chunks), tiles, 64))
        ops.paged_attention(q_lat[a:b].view(b - a, n * self.width), o_lat[a:b], cache.k, cache.k, group.block_table,
                            ctx.token_seq[a:b], ctx.positions[a:b], n, 1, self.width, self.window, self.scale,
                            ctx.error_flag, value_dim=self.kv_rank, splits=splits)

    def _dense(self, q, o, start: int, table: torch.Tensor, cache: LayerCache, ctx: StepContext) -> None:
        m, n, kr = q.shape[0], self.heads, self.kv_rank
        rows = ops.gather_rows(cache.k, table, start + m, ctx.error_flag)            # [context, width]
        slab = max(1, min(m, SCORE_BYTES // (4 * n * (start + m))))
        for t0 in range(0, m, slab):
            t1 = min(m, t0 + slab)
            keys = start + t1                                                          # the last query of the slab sees these
            scores = torch.mm(q[t0:t1].view((t1 - t0) * n, self.width), rows[:keys].t(), out_dtype=torch.float32)
            probs = torch.empty(scores.shape, dtype=q.dtype, device=q.device)
            ops.causal_softmax_rows(scores, probs, n, start + t0, self.scale)
            torch.mm(probs, rows[:keys, :kr], out=o[t0:t1].view((t1 - t0) * n, kr))


#: The tensor-core decode kernel leaves one share per token, head and 64 rows of the longest context the step allows;
#: beyond this many bytes of shares the step takes the general kernel, which bounds its shares by the GPU's size.
DECODE_SHARES_BYTES = 512 << 20
#: A request that brings at least this many tokens to a bfloat16 step takes the products-and-softmax path.
LIBRARY_MIN_TOKENS = 32
#: Bytes of 32-bit scores held at a time on that path (the queries are cut into slabs that fit).
SCORE_BYTES = 64 << 20

register_mixer("latent_attention", LatentAttention)
