"""A recurrent mixer with a decaying matrix state per head (RWKV-style time mixing).

With ``h'`` the input of the token before (zeros at a sequence's start), each of r, k, v, g, w
reads its own mix ``h + (h' - h) * mu_s``.  ``r, k, v = Wr, Wk, Wv`` of their mixes (``heads x d``),
``gate = silu(Wg mix_g)``, and the decay per head and key channel is ``exp(-exp(Ww2 tanh(Ww1
mix_w) + w0))``.  Per head, with state ``S [d, d]`` (zero at the start):

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          S_t = diag(decay_t) S_(t-1) + k_t v_t^T

Each head's ``o`` is brought to unit root mean square, the heads are concatenated, multiplied by
a weight and by the gate, and ``residual += Wo (.)``.

Per request the part keeps ``S`` of every head and the last token's ``h`` in one float32 state
slot; a step hands a request's tokens in order, so prompts cut anywhere continue exactly.
The inner width of the decay's two products is the stored tensor's.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import MATRIX, NORM_WEIGHT, NORM_ZERO, FixedStateSpec, Part, WeightSpec, as_float32, register_part

MIXES = ("r", "k", "v", "g", "w")


class WkvMixer(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, norm_eps: float,
                 decay_rank: Optional[int] = None):
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        self.eps = float(norm_eps)
        # inner width of the decay's products: the stored tensor's own size unless given (random
        # weights need it)
        self.decay_rank = None if decay_rank is None else int(decay_rank)
        self.n = self.num_heads * self.head_dim
        self.prev_offset = self.num_heads * self.head_dim * self.head_dim
        self.mu = self.w = self.w1 = self.w2 = self.w0 = self.u = self.norm = self.w_o = None

    def weight_specs(self):
        h, n = self.hidden_size, self.n
        specs = {f"mu.{s}": WeightSpec((h,), NORM_ZERO) for s in MIXES}
        specs.update({s: WeightSpec((n, h), MATRIX) for s in ("r", "k", "v", "g")})
        specs.update({"w1": WeightSpec((self.decay_rank, h), MATRIX), "w2": WeightSpec((n, self.decay_rank), MATRIX),
                      "w0": WeightSpec((n,), NORM_ZERO), "u": WeightSpec((self.num_heads, self.head_dim), NORM_ZERO),
                      "norm": WeightSpec((n,), NORM_WEIGHT), "o": WeightSpec((h, n), MATRIX)})
        return specs

    def load_weights(self, tensors, ops):
        self.mu = torch.stack([as_float32(tensors[f"mu.{s}"]) for s in MIXES]).contiguous()
        self.w = [ops.pack_linear(tensors[s]) for s in ("r", "k", "v", "g")]
        self.w1, self.w2 = ops.pack_linear(tensors["w1"]), ops.pack_linear(tensors["w2"])
        if self.w1.shape[0] != self.w2.shape[1]:
            raise ValueError(f"the decay's two matrices disagree on their inner width: {tuple(self.w1.shape)} "
                             f"and {tuple(self.w2.shape)}")
        self.w0 = as_float32(tensors["w0"]).contiguous()
        self.u = as_float32(tensors["u"]).contiguous().view(-1)
        self.norm = as_float32(tensors["norm"]).contiguous()
        self.w_o = ops.pack_linear(tensors["o"])

    def cache_spec(self):
        return FixedStateSpec((self.prev_offset + self.hidden_size,), torch.float32)

    def forward(self, ops, h, residual, step, cache):
        t, n, dev = h.shape[0], self.n, h.device
        mixes = torch.empty((len(MIXES), t, self.hidden_size), dtype=h.dtype, device=dev)
        ops.token_shift_mix(h, self.mu, step, cache, self.prev_offset, mixes)
        proj = torch.empty((5, t, n), dtype=torch.float32, device=dev)          # r, k, v, g, decay argument
        for i in range(4):
            ops.linear(mixes[i], self.w[i], proj[i])
        low = torch.empty((t, self.w1.shape[0]), dtype=torch.float32, device=dev)
        ops.linear(mixes[4], self.w1, low)
        low_act = torch.empty(low.shape, dtype=h.dtype, device=dev)
        ops.tanh_rows(low, low_act)
        ops.linear(low_act, self.w2, proj[4])
        out = torch.empty((t, n), dtype=h.dtype, device=dev)
        ops.wkv_recurrence(proj[0], proj[1], proj[2], proj[3], proj[4], self.w0, self.u, self.norm, self.eps,
                           h, step, cache, self.prev_offset, out, self.num_heads, self.head_dim)
        ops.linear(out, self.w_o, residual, accumulate=True, may_defer=True)


register_part("mixer", "wkv", WkvMixer)
