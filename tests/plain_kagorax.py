"""A plain, slow statement of the Kagorax decoder in PyTorch on the CPU, one function per mechanism.

It shares no code with the package: it reads ``config.json`` as a dictionary and the tensors by
their checkpoint names, and loops where a loop says it most plainly.  Everything runs in one
dtype (float64 by default), over one whole sequence at a time.

Notation: ``T`` tokens, model width ``W``, ``H`` query heads, ``G`` key/value heads, head sizes
``dk`` (queries, keys) and ``dv`` (values).
"""
from __future__ import annotations

import math

import torch


# ---- small pieces -------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over the root of (mean of squares + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def sinusoid_rows(positions, width: int, dtype) -> torch.Tensor:
    """Row p: element 2i = sin(p / 10000^(2i/W)), element 2i+1 = cos of the same angle."""
    out = torch.zeros((len(positions), width), dtype=dtype)
    for r, p in enumerate(positions):
        for i in range((width + 1) // 2):
            angle = p * 10000.0 ** (-2.0 * i / width)
            out[r, 2 * i] = math.sin(angle)
            if 2 * i + 1 < width:
                out[r, 2 * i + 1] = math.cos(angle)
    return out


def embed(table: torch.Tensor, tokens, scale: float, first_position: int = 0) -> torch.Tensor:
    x = table[torch.as_tensor(list(tokens), dtype=torch.long)] * scale
    return x + sinusoid_rows(range(first_position, first_position + len(tokens)), table.shape[1], x.dtype)


# ---- distance bias ------------------------------------------------------------------------
def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the bias table for a key ``n`` positions back: one row per distance below half the
    table, then rows spaced evenly in the logarithm of the distance up to ``far``, the last row
    for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    return j <= i and (i - j < window or j < keep_first)


# ---- the mixer ----------------------------------------------------------------------------
def attention_keys_values(h, w, prefix, mixer, eps):
    """Keys (unit RMS per head) and values of every token: [T, G, dk], [T, G, dv]."""
    t = h.shape[0]
    g, dk, dv = mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(t, g, dk)
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(t, g, dv)
    return unit_rms(k, eps), v


def attend(q, keys, values, rel, heads_per_kv: int, scale: float, window: int, keep_first: int, far: int,
           first_position: int = 0):
    """Softmax attention of queries ``q`` [T, H, dk] at positions ``first_position ..`` over
    ``keys`` [S, G, dk] and ``values`` [S, G, dv] at positions ``0 ..``; ``rel`` [rows, H]."""
    t, nh, _ = q.shape
    out = torch.zeros((t, nh, values.shape[2]), dtype=q.dtype)
    for r in range(t):
        i = first_position + r
        js = [j for j in range(i + 1) if visible(i, j, window, keep_first)]
        rows = [distance_bucket(i - j, rel.shape[0], far) for j in js]
        for a in range(nh):
            kv = a // heads_per_kv
            s = keys[js, kv] @ q[r, a] * scale + rel[rows, a]
            p = torch.softmax(s, dim=0)
            out[r, a] = p @ values[js, kv]
    return out


def attention(h, w, prefix, mixer, eps, keys, values):
    """The mixer's output for all tokens of one sequence, given the keys and values to use."""
    t = h.shape[0]
    nh, g, dk, dv = mixer["heads"], mixer["kv_heads"], mixer["dim"], mixer["vdim"]
    q = unit_rms((h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(t, nh, dk), eps)
    heads = attend(q, keys, values, w[prefix + "rel"], nh // g, mixer["scale"], mixer["mask"]["size"],
                   mixer["mask"]["keep_first"], mixer["bias_max"])
    gate = torch.sigmoid(h @ w[prefix + "g"].T)
    return (heads.reshape(t, nh * dv) * gate) @ w[prefix + "o"].T


# ---- the feed-forward ---------------------------------------------------------------------
def gated_ffn(x, w, prefix):
    return (silu(x @ w[prefix + "gate"].T) * (x @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def routed_experts(h, w, prefix, mlp):
    """Per token: the ``top`` experts of largest sigmoid score, each fed the token times its
    score; plus the shared expert times a sigmoid gate of its own."""
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.sigmoid(h @ w[prefix + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = sorted(range(n), key=lambda e: (-float(scores[t, e]), e))[:top]
        for e in chosen:
            out[t] += gated_ffn(scores[t, e] * h[t:t + 1], w, f"{prefix}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_ffn(h, w, prefix + "shared.") * torch.sigmoid(h @ w[prefix + "shared.sg"].T)
    return out


# ---- the model ----------------------------------------------------------------------------
def forward(cfg: dict, w: dict, tokens, dtype=torch.float64, trace=None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from its first token.  ``trace`` (a list) receives the
    residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = embed(w["embed"], tokens, cfg["embedding"]["scale"])
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        mixer = layer["mixer"]
        if layer["type"] != "attention":
            raise ValueError(f"layer {i}: unknown mixer {layer['type']!r}")
        if "kv_from" in mixer:
            keys, values = kept[mixer["kv_from"]]
        else:
            keys, values = kept[i] = attention_keys_values(h, w, p + "mix.", mixer, eps)
        y = attention(h, w, p + "mix.", mixer, eps, keys, values)
        if layer.get("mlp") is not None:
            y = y + routed_experts(h, w, p + "mlp.", layer["mlp"])
        x = x + y
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].T


def load_folder(path: str):
    """``(config dictionary, {name: tensor})`` of a model folder, read without the package."""
    import json
    import os
    import struct
    with open(os.path.join(path, "config.json")) as fh:
        cfg = json.load(fh)
    with open(os.path.join(path, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        data = fh.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32}
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        a, b = ent["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[ent["dtype"]]).view(ent["shape"]).clone()
    return cfg, out


def greedy(cfg, w, prompt, n_new: int, dtype=torch.float64):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(torch.argmax(forward(cfg, w, tokens, dtype)[-1])))
    return tokens[len(prompt):]
