"""The wkv mixer: time mixing with a matrix state per head.

With h the mixer's input and h' the input of the token before (zeros before a request's first token), H heads of
width d:
    x_s = h + (h' - h) * mu_s                       s in r, k, v, g, w: five blends, one per projection
    r, k, v = W_r x_r, W_k x_k, W_v x_v             per head [d];   gate = silu(W_g x_g)
    w = exp(-exp(W_w2 tanh(W_w1 x_w) + w0))         a decay per head and key channel
    o_t = (S_t-1 + diag(u) k_t v_t^T)^T r_t         per head, S [key channel, value channel]; the bonus u only for
    S_t = diag(w_t) S_t-1 + k_t v_t^T               the current token
    out = W_o ((o / rms(o) per head) * norm * gate)
Per request the mixer keeps two fixed-size states in the request's slot: S of every head (32-bit) and the last input
h.  The decays (from the second low-rank product on), the bonus term, the state and the recurrence are 32-bit
(csrc/wkv.cu); the projections run in the engine's dtype.  The low-rank pair's rank is padded to a multiple of eight
with zeros so that its rows stay 16-byte aligned.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import CacheBundle, FixedState, ParamSpec
from .base import Mixer

MIXES = ("r", "k", "v", "g", "w")


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class Wkv(Mixer):
    graph_safe = True          # the batch is read from device tensors only; padding rows (position < 0) are skipped

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if min(s.heads, s.head_dim, s.decay_rank) <= 0:
            raise ValueError("wkv needs heads, head_dim and decay_rank above zero")
        if s.head_dim > 256:
            raise ValueError("the recurrence kernel takes heads up to 256 wide")
        self.width = s.heads * s.head_dim
        self.mu = self.w_r = self.w_k = self.w_v = self.w_g = self.w_1 = self.w_2 = self.w_o = None
        self.decay_bias = self.bonus = self.norm = None

    def cache_requirement(self):
        s = self.spec
        return CacheBundle(None, (FixedState((s.heads, s.head_dim, s.head_dim), "float32"),
                                  FixedState((s.hidden_size,), "float32")))

    def parameters(self):
        s = self.spec
        matrix = lambda rows, columns: ParamSpec((rows, columns), accept_transposed=False)
        table = {f"mu.{name}": ParamSpec((s.hidden_size,), init="zeros", store="float32") for name in MIXES}
        table.update({name: matrix(self.width, s.hidden_size) for name in ("r", "k", "v", "g")})
        table.update({
            "w1": matrix(s.decay_rank, s.hidden_size), "w2": matrix(self.width, s.decay_rank),
            "w0": ParamSpec((self.width,), init="zeros", store="float32"),
            "u": ParamSpec((s.heads, s.head_dim), init="zeros", store="float32", accept_transposed=False),
            "norm": ParamSpec((self.width,), init="ones", store="float32"),
            "o": matrix(s.hidden_size, self.width),
        })
        return table

    def bind(self, tensors):
        s = self.spec
        self.mu = torch.stack([tensors[f"mu.{name}"] for name in MIXES]).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = (tensors[name].contiguous() for name in ("r", "k", "v", "g"))
        rank = _pad8(s.decay_rank)
        w_1 = torch.zeros((rank, s.hidden_size), dtype=tensors["w1"].dtype, device=tensors["w1"].device)
        w_1[:s.decay_rank] = tensors["w1"]
        w_2 = torch.zeros((self.width, rank), dtype=tensors["w2"].dtype, device=tensors["w2"].device)
        w_2[:, :s.decay_rank] = tensors["w2"]
        self.w_1, self.w_2 = w_1, w_2
        self.w_o = tensors["o"].contiguous()
        self.decay_bias = tensors["w0"].contiguous()
        self.bonus = tensors["u"].reshape(-1).contiguous()
        self.norm = tensors["norm"].contiguous()

    def weight_bytes(self):
        tensors = (self.mu, self.w_r, self.w_k, self.w_v, self.w_g, self.w_1, self.w_2, self.w_o, self.decay_bias,
                   self.bonus, self.norm)
        return sum(t.numel() * t.element_size() for t in tensors)

    def forward(self, ctx, cache, x, residual, overwrite=False):
        """residual += W_o y (or residual = W_o y with `overwrite`, for a mixer that combines several branches)."""
        s = self.spec
        tokens = x.shape[0]
        dtype = self.env.dtype
        state, tail = cache.states[0], cache.states[1]
        mixes = ctx.alloc((len(MIXES), tokens, s.hidden_size), dtype)
        kernels.wkv_mix(x, tail, self.mu, ctx.row_of_token, ctx.query_starts, ctx.state_slots, ctx.positions, mixes,
                        single_tokens_only=ctx.decode_only)
        projected = ctx.alloc((4, tokens, self.width), dtype)
        for index, weight in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)):
            kernels.linear(mixes[index], weight, projected[index], alloc=ctx.alloc)
        low = ctx.alloc((tokens, self.w_1.shape[0]), dtype)
        kernels.linear(mixes[4], self.w_1, low, alloc=ctx.alloc)
        kernels.tanh(low)
        decay_raw = ctx.alloc((tokens, self.width), torch.float32)        # 32-bit: it enters the recurrence
        kernels.linear(low, self.w_2, decay_raw, alloc=ctx.alloc)
        read = ctx.alloc((tokens, self.width), torch.float32)
        kernels.wkv_scan(projected[0], projected[1], projected[2], decay_raw, self.decay_bias, self.bonus, state,
                         ctx.query_starts, ctx.state_slots, ctx.positions, read, s.heads, s.head_dim)
        mixed = ctx.alloc((tokens, self.width), dtype)
        kernels.gated_head_norm(read, projected[3], self.norm, mixed, s.heads, s.head_dim, s.norm_eps, False)
        if overwrite:
            kernels.linear(mixed, self.w_o, residual, alloc=ctx.alloc)
        else:
            ctx.accumulate(mixed, self.w_o, residual)
