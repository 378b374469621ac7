"""The gated delta rule: a recurrent mixer with a matrix state per head, short convolutions before it and a gated
per-head norm after it.

With h the mixer's input [T, hidden], G key heads of width D and H value heads of width V (value head i uses key
head i // (H / G)):
    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     causal per-channel convolution over the
                                                                          request's own tokens, zeros before its start
    q, k    = unit vectors per head (x / sqrt(sum x^2 + 1e-6)); q also times D^-1/2
    beta    = sigmoid(W_b h)                                              one per value head
    g       = exp(-exp(A_log) * softplus(a + dt_bias))                    a = W_a h, one per head           (decay "head")
                                                                          a = W_a2 (W_a1 h), per head and key channel ("channel")
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q    per value head, S [D, V], in this order
    y       = o / rms(o) * norm * act(gate)                               gate = W_g h with silu, or W_g2 (W_g1 h) with sigmoid
    out     = W_o y
Per request the mixer keeps two fixed-size states in the request's slot: S of every head (32-bit) and the last
taps - 1 inputs of the convolutions.  Everything between the projections and the output projection is 32-bit
(csrc/delta_rule.cu); the projections run in the engine's dtype.  All projections that read h are one product on
row-stacked weights, each segment padded to a multiple of eight rows so that the views into the packed result stay
16-byte aligned.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import CacheBundle, FixedState, ParamSpec
from .base import Mixer


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class GatedDeltaRule(Mixer):
    graph_safe = True          # the batch is read from device tensors only; padding rows (position < 0) are skipped
    takes_normed_residual = True   # x is used by one product only, which can take a folded norm over

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError("heads must be divisible by kv_heads")
        if s.decay not in ("head", "channel") or s.gate not in ("silu", "sigmoid"):
            raise ValueError(f"unknown decay {s.decay!r} or gate {s.gate!r}")
        if s.key_dim > 256:
            raise ValueError("the recurrence kernel takes key heads up to 256 wide")
        self.qk_width = s.kv_heads * s.key_dim
        self.v_width = s.heads * s.value_dim
        self.conv_channels = 2 * self.qk_width + self.v_width
        self.decay_width = s.heads * s.key_dim if s.decay == "channel" else s.heads
        # segments of the packed projection: name -> (first column, columns)
        self.segments, cursor = {}, 0
        first = ("a1", s.decay_rank) if s.decay == "channel" else ("a", s.heads)
        second = ("g1", s.gate_rank) if s.gate == "sigmoid" else ("g", self.v_width)
        for name, width in (("q", self.qk_width), ("k", self.qk_width), ("v", self.v_width), ("b", s.heads), first, second):
            if name == "q" or name == "k" or name == "v":
                self.segments[name] = (cursor, width)          # q | k | v stay side by side for the convolution
                cursor += width
                if name == "v":
                    cursor = _pad8(cursor)
            else:
                self.segments[name] = (cursor, width)
                cursor = _pad8(cursor + width)
        self.packed_width = cursor
        self.w_in = self.w_conv = self.w_a2 = self.w_g2 = self.w_second = self.w_o = None
        self.a_log = self.dt_bias = self.norm = None

    def cache_requirement(self):
        s = self.spec
        return CacheBundle(None, (FixedState((s.heads, s.value_dim, s.key_dim), "float32"),
                                  FixedState((max(s.conv_taps - 1, 0), self.conv_channels), "float32")))

    def parameters(self):
        s = self.spec
        table = {
            "q": ParamSpec((self.qk_width, s.hidden_size)), "q.conv": ParamSpec((self.qk_width, s.conv_taps), accept_transposed=False),
            "k": ParamSpec((self.qk_width, s.hidden_size)), "k.conv": ParamSpec((self.qk_width, s.conv_taps), accept_transposed=False),
            "v": ParamSpec((self.v_width, s.hidden_size)), "v.conv": ParamSpec((self.v_width, s.conv_taps), accept_transposed=False),
            "b": ParamSpec((s.heads, s.hidden_size)),
            "A_log": ParamSpec((s.heads,), init="zeros", store="float32"),
            "dt_bias": ParamSpec((self.decay_width,), init="zeros", store="float32"),
            "norm": ParamSpec((s.value_dim,), init="ones", store="float32"),
            "o": ParamSpec((s.hidden_size, self.v_width)),
        }
        if s.decay == "channel":
            table["a1"] = ParamSpec((s.decay_rank, s.hidden_size))
            table["a2"] = ParamSpec((self.decay_width, s.decay_rank))
        else:
            table["a"] = ParamSpec((s.heads, s.hidden_size))
        if s.gate == "sigmoid":
            table["g1"] = ParamSpec((s.gate_rank, s.hidden_size))
            table["g2"] = ParamSpec((self.v_width, s.gate_rank))
        else:
            table["g"] = ParamSpec((self.v_width, s.hidden_size))
        return table

    def bind(self, tensors):
        s = self.spec
        w_in = torch.zeros((self.packed_width, s.hidden_size), dtype=tensors["q"].dtype, device=tensors["q"].device)
        for name, (first, width) in self.segments.items():
            w_in[first:first + width] = tensors[name]
        self.w_in = w_in
        self.w_conv = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        self.a_log, self.dt_bias, self.norm = (tensors[n].contiguous() for n in ("A_log", "dt_bias", "norm"))

        def second_stage(weight, rank):          # [out, rank] -> [out, rank rounded up to 8], zero columns added
            padded = torch.zeros((weight.shape[0], _pad8(rank)), dtype=weight.dtype, device=weight.device)
            padded[:, :rank] = weight
            return padded
        if s.decay == "channel":
            self.w_a2 = second_stage(tensors["a2"], s.decay_rank)
        if s.gate == "sigmoid":
            self.w_g2 = second_stage(tensors["g2"], s.gate_rank)
        self.w_second = None
        if s.decay == "channel" and s.gate == "sigmoid":
            # both second stages as one product on the neighbouring segments a1 | g1 of the packed projection: the
            # weights side by side on the diagonal, zeros elsewhere; the result is 32-bit [decays | gates]
            ranks = self.w_a2.shape[1] + self.w_g2.shape[1]
            both = torch.zeros((self.decay_width + self.v_width, ranks), dtype=self.w_a2.dtype, device=self.w_a2.device)
            both[:self.decay_width, :self.w_a2.shape[1]] = self.w_a2
            both[self.decay_width:, self.w_a2.shape[1]:] = self.w_g2
            if self.segments["g1"][0] == self.segments["a1"][0] + self.w_a2.shape[1]:
                self.w_second, self.w_a2, self.w_g2 = both, None, None

    def weight_bytes(self):
        tensors = (self.w_in, self.w_conv, self.w_a2, self.w_g2, self.w_second, self.w_o, self.a_log, self.dt_bias, self.norm)
        return sum(t.numel() * t.element_size() for t in tensors if t is not None)

    def forward(self, ctx, cache, x, residual, overwrite=False):
        """residual += W_o y (or residual = W_o y with `overwrite`, for a mixer that combines several branches)."""
        s = self.spec
        tokens = x.shape[0]
        state, tail = cache.states[0], cache.states[1]
        packed = ctx.alloc((tokens, self.packed_width), self.env.dtype)
        kernels.linear(x, self.w_in, packed, alloc=ctx.alloc)
        segment = lambda name, width=None: packed[:, self.segments[name][0]:self.segments[name][0] + (width or self.segments[name][1])]
        if self.w_second is not None:
            second = ctx.alloc((tokens, self.decay_width + self.v_width), torch.float32)
            kernels.linear(segment("a1", self.w_second.shape[1]), self.w_second, second, alloc=ctx.alloc)
            decay, gate = second[:, :self.decay_width], second[:, self.decay_width:]
        else:
            if s.decay == "channel":
                decay = ctx.alloc((tokens, self.decay_width), torch.float32)       # 32-bit: it enters the recurrence
                kernels.linear(segment("a1", self.w_a2.shape[1]), self.w_a2, decay, alloc=ctx.alloc)
            else:
                decay = segment("a")
            if s.gate == "sigmoid":
                gate = ctx.alloc((tokens, self.v_width), self.env.dtype)
                kernels.linear(segment("g1", self.w_g2.shape[1]), self.w_g2, gate, alloc=ctx.alloc)
            else:
                gate = segment("g")
        # all tokens in parallel: convolutions, unit vectors, sigmoid and the decays; then the recurrence
        prepared = ctx.alloc((tokens, self.conv_channels), torch.float32)
        beta = ctx.alloc((tokens, s.heads), torch.float32)
        decays = ctx.alloc((tokens, self.decay_width), torch.float32)
        kernels.delta_rule_prepare(packed[:, :self.conv_channels], self.w_conv, tail, segment("b"), decay, self.dt_bias,
                                   self.a_log, ctx.row_of_token, ctx.query_starts, ctx.state_slots, ctx.positions,
                                   prepared, beta, decays, s.heads, s.kv_heads, s.key_dim, s.value_dim)
        read = ctx.alloc((tokens, self.v_width), torch.float32)
        kernels.delta_rule_scan(prepared, beta, decays, state, ctx.query_starts, ctx.state_slots, ctx.positions, read,
                                s.heads, s.kv_heads, s.key_dim, s.value_dim)
        mixed = ctx.alloc((tokens, self.v_width), self.env.dtype)
        kernels.gated_head_norm(read, gate, self.norm, mixed, s.heads, s.value_dim, s.norm_eps, s.gate == "sigmoid")
        if overwrite:
            kernels.linear(mixed, self.w_o, residual, alloc=ctx.alloc)
        else:
            ctx.accumulate(mixed, self.w_o, residual)
