"""Grouped-query attention with a learned bias per (head, distance), a window that keeps a
request's first tokens, an output gate and projections with biases.

For token ``i`` and query head ``a`` (kv head ``a // (heads / kv_heads)``):

* ``q, k, v = Wq h + bq, Wk h + bk, Wv h + bv``; ``q`` and ``k`` are brought to unit root mean
  square per head (``x / sqrt(mean(x^2) + eps)``, no weight); there is no rotation.
* key ``j <= i`` is visible when ``i - j < window`` or ``j < keep_first``.
* ``score = (q . k) * scale + B[row(i - j), a]``; ``B`` is the layer's own table.  ``row(n) = n``
  below half the table's rows ``R``; from there on rows are spaced evenly in ``ln n`` up to
  ``far``: ``row(n) = min(R - 1, R/2 + floor(ln(n / (R/2)) / ln(far / (R/2)) * (R - R/2)))``.
  The kernels get the table expanded by distance, ``[heads, far + 1]`` float32 (every distance
  from ``far`` on reads the last row), so they never take a logarithm.
* float32 softmax over the visible keys, weighted sum of the values (head size ``v_head_dim``).
* the concatenated heads times ``sigmoid(Wg h)``, element by element, then ``residual += Wo (.)``.

A layer with ``own_kv=False`` has no key/value projections: it reads the cache slot that another
layer wrote (normed keys, values) with its own queries, mask, table and gate.  The slot keeps
what the widest reader needs: ``cache_window`` / ``cache_keep_first``.

All of ``Wq, Wk, Wv, Wg`` run as one product; the bias is added, heads are normed and stored by
the kernel behind it, and the gate is applied in the attention kernel's last step.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import MATRIX, PagedKVSpec, Part, WeightSpec, as_float32, register_part


def distance_rows(num_rows: int, far: int) -> list[int]:
    """Row of the bias table for every distance ``0 .. far`` (the last entry serves all beyond)."""
    half = num_rows // 2
    if half < 1 or far <= half:
        raise ValueError(f"a distance table of {num_rows} rows cannot reach to {far}")
    rows = []
    for n in range(far + 1):
        if n < half:
            rows.append(n)
        else:
            rows.append(min(num_rows - 1, half + int(math.floor(
                math.log(n / half) / math.log(far / half) * (num_rows - half)))))
    return rows


class GatedBiasAttention(Part):
    category = "mixer"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 v_head_dim: int, scale: float, qk_norm_eps: float, window: Optional[int],
                 keep_first: int, bias_far: int, bias_rows: Optional[int] = None, own_kv: bool = True,
                 cache_window: Optional[int] = None, cache_keep_first: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_kv_heads} kv heads evenly")
        if window is not None and window < 1:
            raise ValueError(f"window must be positive, got {window}")
        self.hidden_size = int(hidden_size)
        self.num_heads, self.num_kv_heads = int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale, self.eps = float(scale), float(qk_norm_eps)
        self.window = None if window is None else int(window)
        self.keep_first = int(keep_first)
        # rows of the bias table: the stored tensor's own size unless given (random weights need it)
        self.bias_rows = None if bias_rows is None else int(bias_rows)
        self.bias_far = int(bias_far)
        self.own_kv = bool(own_kv)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        self.cache_keep_first = self.keep_first if cache_keep_first is None else int(cache_keep_first)
        self.nq = self.num_heads * self.head_dim
        self.nk = self.num_kv_heads * self.head_dim
        self.nv = self.num_kv_heads * self.v_head_dim
        self.ng = self.num_heads * self.v_head_dim
        self.w_in = self.bias = self.w_o = self.dist_bias = None

    def weight_specs(self):
        h = self.hidden_size
        specs = {"q": WeightSpec((self.nq, h), MATRIX), "q.b": WeightSpec((self.nq,), MATRIX)}
        if self.own_kv:
            specs.update({"k": WeightSpec((self.nk, h), MATRIX), "k.b": WeightSpec((self.nk,), MATRIX),
                          "v": WeightSpec((self.nv, h), MATRIX), "v.b": WeightSpec((self.nv,), MATRIX)})
        specs.update({"rel": WeightSpec((self.bias_rows, self.num_heads), MATRIX),
                      "g": WeightSpec((self.ng, h), MATRIX), "o": WeightSpec((h, self.ng), MATRIX)})
        return specs

    def load_weights(self, tensors, ops):
        names = ["q", "k", "v"] if self.own_kv else ["q"]
        mats = [tensors[n] for n in names] + [tensors["g"]]
        if len({m.dtype for m in mats}) > 1:          # mixed storage: widen, never narrow
            mats = [m.to(torch.float32) for m in mats]
        self.w_in = ops.pack_linear(torch.cat(mats, dim=0))
        self.bias = torch.cat([as_float32(tensors[n + ".b"]) for n in names]).contiguous()
        self.w_o = ops.pack_linear(tensors["o"])
        rel = as_float32(tensors["rel"])               # [rows, heads]
        rows = torch.as_tensor(distance_rows(rel.shape[0], self.bias_far), dtype=torch.long, device=rel.device)
        self.dist_bias = rel[rows].t().contiguous()    # [heads, far + 1]

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.cache_window,
                           None if self.v_head_dim == self.head_dim else self.v_head_dim,
                           self.cache_keep_first)

    def forward(self, ops, h, residual, step, cache):
        t = h.shape[0]
        if cache.writes != self.own_kv:
            raise ValueError("a layer with key/value projections writes its cache slot, one without reads another's")
        proj = torch.empty((t, self.w_in.shape[0]), dtype=torch.float32, device=h.device)
        ops.linear(h, self.w_in, proj)
        q = torch.empty((t, self.nq), dtype=h.dtype, device=h.device)
        ops.qkv_bias_norm_store(proj, self.bias, None, None, self.eps, step, cache, q,
                                self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim)
        gate = proj[:, proj.shape[1] - self.ng:]
        out = torch.empty((t, self.ng), dtype=h.dtype, device=h.device)
        ops.biased_attention(q, step, cache, out, self.num_heads, self.num_kv_heads, self.head_dim,
                             self.v_head_dim, self.window, self.keep_first, self.scale,
                             self.dist_bias, gate)
        ops.linear(out, self.w_o, residual, accumulate=True)


register_part("mixer", "gated_bias_attention", GatedBiasAttention)
