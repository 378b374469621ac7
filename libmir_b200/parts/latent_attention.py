"""Latent attention: queries, keys and values come through low-rank latents, and the cache holds one vector per
token.

With h the mixer's input, H heads, per head d unrotated and r rotated query / key dims and e value dims:
    c_q = rmsnorm(W_dq h) * n_q;   q = W_uq c_q                    per head [d unrotated | r rotated]
    [c' | k_r] = W_dkv h;   c = rmsnorm(c') * n_kv                 the latent (kv_rank wide) and one rotated key part
                                                                   (r wide, not normed) shared by all heads
    k_h = [W_uk,h c | rot(k_r)],  v_h = W_uv,h c,  q_h = [q_h unrotated | rot(q_h rotated)]
    a_h = softmax_j<=i(q_h . k_h,j * scale) v_h,j;   out = W_o (concat_h a_h * sigmoid(W_g h))
Only c and rot(k_r) are cached: one row [kv_rank + r] per token.  The up-projections never run on cached tokens:
    q_h . k_h,j = (W_uk,h^T q_h unrotated) . c_j + rot(q_h rotated) . rot(k_r)_j
so each query head becomes a vector of kv_rank + r numbers and attention is what a model with one key head of that
width would run, with the first kv_rank numbers of a cached row as its value; W_uv,h is applied to the attended
latent afterwards.  Norms, angles, scores and the softmax are 32-bit; the rotation is the mixer's position part
(layout, frequencies and magnitude are its constants).
Kernels: csrc/latent_attention.cu (latent_prepare, rope_rows, head_linear) and the paged attention kernels.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import PagedKv, ParamSpec
from ..registry import build_part
from .base import Mixer


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class LatentAttention(Mixer):
    graph_safe = True
    takes_normed_residual = True       # x enters one product only

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if min(s.heads, s.head_dim, s.value_dim, s.q_rank, s.kv_rank) <= 0 or s.rotary_dim < 0 or s.rotary_dim % 2:
            raise ValueError("latent attention needs heads, head_dim, value_dim and both ranks above zero and an even "
                             "rotary_dim")
        self.position = build_part(s.position, env) if (s.position is not None and s.rotary_dim) else None
        if self.position is not None and self.position.rotary_dim != s.rotary_dim:
            raise ValueError("the position part must rotate exactly the rotary dims")
        self.key_width = s.kv_rank + s.rotary_dim                  # of a cached row and of a folded query head
        self.out_width = s.heads * s.value_dim
        # segments of the packed projection of h: name -> first column
        self.segments, cursor = {}, 0
        for name, width in (("dq", s.q_rank), ("dkv", self.key_width), ("g", self.out_width if s.gate else 0)):
            self.segments[name] = cursor
            cursor = _pad8(cursor + width)
        self.packed_width = cursor
        self.w_in = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.q_norm = self.kv_norm = None

    def cache_requirement(self):
        # one vector per token: the latent is read as key and as value, so no value rows are kept
        return PagedKv(1, self.key_width, None, 0)

    def parameters(self):
        s = self.spec
        matrix = lambda rows, columns: ParamSpec((rows, columns), accept_transposed=False)
        table = {
            "dq": matrix(s.q_rank, s.hidden_size), "dq.norm": ParamSpec((s.q_rank,), init="ones", store="float32"),
            "uq": matrix(s.heads * (s.head_dim + s.rotary_dim), s.q_rank),
            "dkv": matrix(self.key_width, s.hidden_size), "dkv.norm": ParamSpec((s.kv_rank,), init="ones", store="float32"),
            "uk": matrix(s.heads * s.head_dim, s.kv_rank), "uv": matrix(s.heads * s.value_dim, s.kv_rank),
            "o": matrix(s.hidden_size, self.out_width),
        }
        if s.gate:
            table["g"] = matrix(self.out_width, s.hidden_size)
        return table

    def bind(self, tensors):
        s = self.spec
        w_in = torch.zeros((self.packed_width, s.hidden_size), dtype=tensors["dq"].dtype, device=tensors["dq"].device)
        for name in ("dq", "dkv") + (("g",) if s.gate else ()):
            w_in[self.segments[name]:self.segments[name] + tensors[name].shape[0]] = tensors[name]
        self.w_in = w_in
        self.w_uq = tensors["uq"].contiguous()
        # per head [in, out]: the key up-projection is applied transposed (to the query), the value one as it is
        self.w_uk = tensors["uk"].view(s.heads, s.head_dim, s.kv_rank).contiguous()
        self.w_uv = tensors["uv"].view(s.heads, s.value_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.q_norm, self.kv_norm = tensors["dq.norm"].contiguous(), tensors["dkv.norm"].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_uq, self.w_uk, self.w_uv, self.w_o))

    def forward(self, ctx, cache, x, residual, overwrite=False):
        """residual += W_o (...) (or residual = with `overwrite`, for a mixer that combines several branches)."""
        s = self.spec
        tokens = x.shape[0]
        dtype = self.env.dtype
        group = ctx.groups[cache.group]
        table = self.position.table if self.position is not None else None
        magnitude = self.position.magnitude if self.position is not None else 1.0
        interleaved = self.position.interleaved if self.position is not None else False
        packed = ctx.alloc((tokens, self.packed_width), dtype)
        kernels.linear(x, self.w_in, packed, alloc=ctx.alloc)
        latent_q = ctx.alloc((tokens, s.q_rank), dtype)
        kernels.latent_prepare(packed, self.segments["dq"], s.q_rank, self.segments["dkv"], s.kv_rank, s.rotary_dim,
                               self.q_norm, self.kv_norm, s.norm_eps, ctx.positions,
                               group.slot_mapping if cache.writes else None, table, magnitude, interleaved, latent_q,
                               cache.k_pages)
        per_head = s.head_dim + s.rotary_dim
        q = ctx.alloc((tokens, s.heads * per_head), dtype)
        kernels.linear(latent_q, self.w_uq, q, alloc=ctx.alloc)
        q = q.view(tokens, s.heads, per_head)
        folded = ctx.alloc((tokens, s.heads, self.key_width), dtype)
        kernels.head_linear(q[:, :, :s.head_dim], self.w_uk, folded[:, :, :s.kv_rank])
        if s.rotary_dim:
            kernels.rope_rows(q[:, :, s.head_dim:], folded[:, :, s.kv_rank:], ctx.positions, table, magnitude, interleaved)
        attended = ctx.alloc((tokens, s.heads * s.kv_rank), dtype)
        self.attend(ctx, group, cache, folded.view(tokens, s.heads * self.key_width), attended)
        mixed = ctx.alloc((tokens, self.out_width), dtype)
        gate = packed[:, self.segments["g"]:self.segments["g"] + self.out_width] if s.gate else None
        kernels.head_linear(attended.view(tokens, s.heads, s.kv_rank), self.w_uv, mixed.view(tokens, s.heads, s.value_dim),
                            gate)
        if overwrite:
            kernels.linear(mixed, self.w_o, residual, alloc=ctx.alloc)
        else:
            ctx.accumulate(mixed, self.w_o, residual)

    def attend(self, ctx, group, cache, folded, out):
        """Every packed row's folded query heads over its request's cached rows: one key head of kv_rank + rotary
        dims whose first kv_rank dims are the value."""
        s = self.spec
        if self.env.dtype == torch.bfloat16 and kernels.latent_attention_takes(self.key_width, s.kv_rank):
            # tensor cores: the (token, head) pairs of a request are the rows of one query matrix over its keys
            max_pairs = max(1, ctx.max_portion) * s.heads
            per_partition, partitions = kernels.latent_attention_plan(ctx.num_rows, max_pairs, ctx.max_context)
            kernels.latent_attention(folded, out, cache.k_pages, group.block_table, ctx.query_starts, ctx.context_lens,
                                     cache.page_size, s.heads, self.key_width, s.kv_rank, s.scale, max_pairs,
                                     per_partition, partitions, ctx.alloc)
            return
        kernels.paged_attention_generic(folded, out, cache.k_pages, None, group.block_table, ctx.row_of_token,
                                        ctx.positions, cache.page_size, s.heads, 1, self.key_width, s.scale, None,
                                        value_dim=s.kv_rank, values_in_keys=True)
