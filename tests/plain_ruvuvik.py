"""A plain, slow statement of the Ruvuvik decoder in PyTorch on the CPU, one function per mechanism.

It shares no code with the package: it reads ``config.json`` as a dictionary and the tensors by
their checkpoint names, and loops over tokens and keys where a loop says it most plainly.
Everything runs in one dtype (float64 by default), over one whole sequence at a time; the
recurrent mixer can also be carried from one piece of a sequence to the next.

Notation: ``T`` tokens, model width ``W``, ``H`` query heads, ``G`` key/value heads, head sizes
``dk`` (queries, keys) and ``dv`` (values), latent width ``R``, rotated width ``dr``.
"""
from __future__ import annotations

import math

import torch


# ---- small pieces -------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over the root of (mean of squares + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_plain(x, weight, eps):
    return unit_rms(x, eps) * weight


def norm_one_plus(x, weight, eps):
    """The model's norm: the stored weight is the factor minus one."""
    return unit_rms(x, eps) * (1.0 + weight)


def softplus(z: float) -> float:
    return math.log1p(math.exp(-abs(z))) + max(z, 0.0)


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.exp(neg) - 1.0 - neg) + 0.5 * z)


def rotate_pairs(x: torch.Tensor, positions, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` elements of every head turned pair by pair; element 2i
    goes with 2i + 1, by the angle position * base^(-2i / dims).  The rest passes."""
    out = x.clone()
    for r, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[r, :, 2 * i], x[r, :, 2 * i + 1]
            out[r, :, 2 * i] = u * c - v * s
            out[r, :, 2 * i + 1] = v * c + u * s
    return out


def softmax_rows(scores: torch.Tensor, extra: float | None = None) -> torch.Tensor:
    """Weights of one query over its visible keys; ``extra`` is a logit that only enlarges the
    denominator."""
    m = scores.max().item() if extra is None else max(scores.max().item(), extra)
    e = torch.exp(scores - m)
    den = e.sum() + (0.0 if extra is None else math.exp(extra - m))
    return e / den


def attend(q, keys, values, positions, scale, chunk=None, cap=None, head_scale=None, sink=None):
    """Causal softmax attention of queries ``q`` [T, H, dk] at ``positions`` over ``keys`` [S, G, dk]
    and ``values`` [S, G, dv] at positions 0 .. S-1.  A query at i sees j <= i of its own chunk
    (``j // chunk == i // chunk``); the score is (q . k) * scale [* head_scale[h]], then
    cap * tanh(score / cap); ``sink`` [H] adds one logit without a value to the denominator."""
    t, nh, _ = q.shape
    g = keys.shape[1]
    out = torch.zeros((t, nh, values.shape[2]), dtype=q.dtype)
    for r, i in enumerate(positions):
        lo = 0 if chunk is None else (i // chunk) * chunk
        for a in range(nh):
            kv = a // (nh // g)
            s = (keys[lo:i + 1, kv] @ q[r, a]) * scale
            if head_scale is not None:
                s = s * head_scale[a]
            if cap is not None:
                s = cap * torch.tanh(s / cap)
            out[r, a] = softmax_rows(s, None if sink is None else float(sink[a])) @ values[lo:i + 1, kv]
    return out


# ---- mixers --------------------------------------------------------------------------------
def chunked_attention(h, w, p, m, eps, first_position=0, past=None):
    """Grouped-query attention inside chunks of ``mask.size`` positions.  ``past``: (keys, values)
    of the positions before ``first_position``; returns the output and the grown (keys, values)."""
    t = h.shape[0]
    nh, g, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = list(range(first_position, first_position + t))
    q = norm_plain(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(t, nh, dk)
    k = norm_plain(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(t, g, dk)
    v = (h @ w[p + "v"].T).view(t, g, dv)
    q = rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"])
    if past is not None:
        k, v = torch.cat([past[0], k]), torch.cat([past[1], v])
    gate = torch.sigmoid(h @ w[p + "g"].T)                        # [T, H]
    chunk = m["mask"]["size"] if m.get("mask") else None
    out = attend(q, k, v, pos, m["scale"], chunk, m.get("softcap"), w[p + "temp"]) * gate[:, :, None]
    return out.reshape(t, nh * dv) @ w[p + "o"].T, (k, v)


def latent_attention(h, w, p, m, eps, first_position=0, past=None):
    """Attention whose keys and values are made from one latent row per token plus one rotated
    key part that all heads share; the softmax has a sink.  ``past``: (latents, rotated parts)."""
    t = h.shape[0]
    nh, dk, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = list(range(first_position, first_position + t))
    q = (h @ w[p + "q"].T).view(t, nh, dk + dr)
    q_plain = q[:, :, :dk]
    q_rot = rotate_pairs(q[:, :, dk:], pos, m["rot"]["dims"], m["rot"]["base"])
    down = h @ w[p + "dkv"].T
    c = norm_plain(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, rank:].reshape(t, 1, dr), pos, m["rot"]["dims"], m["rot"]["base"])[:, 0]
    if past is not None:
        c, k_rot = torch.cat([past[0], c]), torch.cat([past[1], k_rot])
    # every head's key: its own plain part followed by the shared rotated part
    keys = torch.cat([(c @ w[p + "uk"].T).view(-1, nh, dk), k_rot[:, None, :].expand(-1, nh, -1)], dim=2)
    values = (c @ w[p + "uv"].T).view(-1, nh, dv)
    out = attend(torch.cat([q_plain, q_rot], dim=2), keys, values, pos, m["scale"], sink=w[p + "sink"])
    return out.reshape(t, nh * dv) @ w[p + "o"].T, (c, k_rot)


def wkv(h, w, p, m, eps, state=None):
    """Time mixing with a decaying matrix state per head.  ``state``: (previous token's input,
    S [heads, d, d]) or None for the start of a sequence; returns the output and the new state."""
    t, width = h.shape
    nh, d = m["heads"], m["dim"]
    prev, s = (torch.zeros(width, dtype=h.dtype), torch.zeros((nh, d, d), dtype=h.dtype)) if state is None else state
    s = s.clone()
    out = torch.zeros((t, nh * d), dtype=h.dtype)
    for r in range(t):
        x = h[r]
        mix = {n: x + (prev - x) * w[p + "mu." + n] for n in "rkvgw"}
        rr = (w[p + "r"] @ mix["r"]).view(nh, d)
        kk = (w[p + "k"] @ mix["k"]).view(nh, d)
        vv = (w[p + "v"] @ mix["v"]).view(nh, d)
        g = w[p + "g"] @ mix["g"]
        gate = g * torch.sigmoid(g)
        decay = torch.exp(-torch.exp(w[p + "w2"] @ torch.tanh(w[p + "w1"] @ mix["w"]) + w[p + "w0"])).view(nh, d)
        heads = []
        for a in range(nh):
            kv = torch.outer(kk[a], vv[a])
            o = (s[a] + w[p + "u"][a][:, None] * kv).T @ rr[a]
            s[a] = decay[a][:, None] * s[a] + kv
            heads.append(unit_rms(o, eps))
        out[r] = torch.cat(heads) * w[p + "norm"] * gate
        prev = x
    return out @ w[p + "o"].T, (prev, s)


MIXERS = {"attention": chunked_attention, "latent_attention": latent_attention}


def feed_forward(h, w, p):
    act = w[p + "act"]
    return xielu(h @ w[p + "up"].T, float(act[0]), float(act[1])) @ w[p + "down"].T


# ---- the model ------------------------------------------------------------------------------
def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, carry=None, keep_layers=False):
    """Logits [T, vocab] of one sequence's next ``tokens``.  ``carry`` is what an earlier call
    returned for the tokens before these (None at the start); returns (logits, carry[, residual
    stream after every layer])."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    first, caches = (0, [None] * len(cfg["layers"])) if carry is None else carry
    caches = list(caches)
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    x = norm_one_plus(x, w["embed.norm"], eps)
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        h = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "wkv":
            y, caches[i] = wkv(h, w, p + "mix.", layer["mixer"], eps, caches[i])
        else:
            y, caches[i] = MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps, first, caches[i])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + feed_forward(norm_one_plus(x, w[p + "norm2"], eps), w, p + "mlp.")
        after.append(x)
    logits = norm_one_plus(x, w["final.norm"], eps) @ w["head"].T
    carry = (first + len(tokens), caches)
    return (logits, carry, torch.stack(after)) if keep_layers else (logits, carry)


def load_folder(model_dir: str):
    """``(config dictionary, {tensor name: tensor})`` of a model folder, read with the standard
    library and torch alone."""
    import json
    import os
    import struct
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        data = fh.read()
    weights = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        lo, hi = ent["data_offsets"]
        weights[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=kinds[ent["dtype"]]).view(ent["shape"]).clone()
    return cfg, weights


def greedy(cfg, weights, prompt, count: int):
    """``count`` tokens chosen by the largest logit (ties: the lowest id), from ``prompt`` on."""
    logits, carry = forward(cfg, weights, prompt)
    out = []
    for _ in range(count):
        out.append(int(torch.argmax(logits[-1])))
        logits, carry = forward(cfg, weights, [out[-1]], carry=carry)
    return out
