"""Small Ruvuvik configurations with random weights, written as model folders by the tests.

The weights are drawn here with torch's generator (not with the package's), large enough that
every mechanism moves the logits: score factors and caps that bend the scores, sinks that take a
share of the softmax, decays spread between fast and slow, activations on both of their branches.
Everything is stored in bfloat16, so the plain implementation and the engine read the same values.
"""
from __future__ import annotations

import json
import os

import torch

from tinyinfer_b200.weights.safetensors_io import write_safetensors


def attention(heads, kv_heads, dim, vdim, chunk, rot_dims, base, scale, softcap):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                           "mask": {"size": chunk}, "rot": {"dims": rot_dims, "base": base},
                                           "scale": scale, "softcap": softcap}}


def latent(heads, dim, rot_dim, vdim, kv_rank, base, scale):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                                                  "kv_rank": kv_rank, "rot": {"dims": rot_dim, "base": base},
                                                  "scale": scale}}


def wkv(heads, dim):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}}


def layer(entry, ff=None, weights_of=None):
    out = dict(entry, mlp=None if ff is None else {"kind": "dense", "ff": ff})
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


_A0 = latent(3, 8, 4, 12, 20, 10000.0, 0.3)
_A1 = wkv(2, 12)
_A2 = attention(4, 2, 12, 8, 7, 6, 1000.0, 0.29, 5.0)
# every size differs between the mixers; a chunk shorter than a page, a rotation over half a head,
# value heads of their own size, a layer without a feed-forward, layers that run another's tensors
SMALL_A = {"architecture": "Ruvuvik", "vocab": 131, "width": 48, "norm": {"eps": 1e-6}, "layers": [
    layer(_A0, 40), layer(_A1), layer(_A2, 24), layer(_A1, weights_of=1), layer(_A2, 24, weights_of=2),
    layer(_A0, 40, weights_of=0)]}
# values that make branches coincide: one head, as many kv heads as heads, a chunk longer than any
# prompt, a rotation over the whole head, one recurrent head as wide as the model
SMALL_B = {"architecture": "Ruvuvik", "vocab": 97, "width": 32, "norm": {"eps": 1e-5}, "layers": [
    layer(attention(1, 1, 16, 16, 4096, 16, 500.0, 0.25, 50.0), 32),
    layer(wkv(1, 32), 16),
    layer(latent(1, 16, 2, 16, 16, 30.0, 0.2), 32),
    layer(attention(2, 2, 8, 8, 64, 2, 7.0, 0.35, 2.0))]}
# sizes that tensor-core kernels take (head sizes 64 and 128, widths that are multiples of 64),
# chunks that end inside pages
SMALL_C = {"architecture": "Ruvuvik", "vocab": 1009, "width": 128, "norm": {"eps": 2e-6}, "layers": [
    layer(wkv(2, 64), 192),
    layer(attention(4, 2, 64, 64, 72, 32, 20000.0, 0.125, 8.0), 128),
    layer(latent(4, 32, 32, 32, 96, 5000.0, 0.13), 192),
    layer(attention(2, 1, 128, 128, 100, 128, 300000.0, 0.09, 12.0), 128),
    layer(wkv(2, 64), 192, weights_of=0)]}

SMALL = {"A": (SMALL_A, 5), "B": (SMALL_B, 8), "C": (SMALL_C, 16)}     # configuration, decay's inner width


def mixer_weights(kind: str, m: dict, width: int, g: torch.Generator, decay_rank: int = 4) -> dict:
    """Tensors of one mixer under their local names."""
    def mat(rows, cols, gain=1.0):
        return (torch.randn((rows, cols), generator=g) * gain / cols ** 0.5).to(torch.bfloat16)

    def vec(n, std, mean=0.0):
        return (mean + torch.randn((n,), generator=g) * std).to(torch.bfloat16)

    w = {}
    if kind == "attention":
        nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        w.update({"q": mat(nq, width, 2.0), "k": mat(nk, width, 2.0), "v": mat(nv, width),
                  "q.norm": vec(nq, 0.3, 1.5), "k.norm": vec(nk, 0.3, 1.5), "temp": vec(m["heads"], 0.5, 2.0),
                  "g": mat(m["heads"], width, 3.0), "o": mat(width, m["heads"] * m["vdim"])})
    elif kind == "latent_attention":
        nh, row = m["heads"], m["kv_rank"] + m["rot_dim"]
        w.update({"q": mat(nh * (m["dim"] + m["rot_dim"]), width, 3.0), "dkv": mat(row, width, 2.0),
                  "dkv.norm": vec(m["kv_rank"], 0.3, 1.0), "uk": mat(nh * m["dim"], m["kv_rank"], 2.0),
                  "uv": mat(nh * m["vdim"], m["kv_rank"]), "sink": vec(nh, 1.0, 1.0),
                  "o": mat(width, nh * m["vdim"])})
    else:
        n = m["heads"] * m["dim"]
        for s in "rkvgw":
            w["mu." + s] = torch.rand((width,), generator=g).to(torch.bfloat16)
        w.update({"r": mat(n, width, 1.5), "k": mat(n, width, 1.5), "v": mat(n, width, 1.5), "g": mat(n, width, 2.0),
                  "w1": mat(decay_rank, width, 2.0), "w2": mat(n, decay_rank, 2.0), "w0": vec(n, 1.5, -1.5),
                  "u": vec(n, 0.5, 0.3).view(m["heads"], m["dim"]), "norm": vec(n, 0.2, 1.0), "o": mat(width, n)})
    return w


def random_weights(cfg: dict, decay_rank: int, seed: int) -> dict:
    g = torch.Generator().manual_seed(seed)
    width = cfg["width"]
    small = lambda n: (0.2 * torch.randn((n,), generator=g)).to(torch.bfloat16)
    w = {"embed": (torch.randn((cfg["vocab"], width), generator=g) * 0.5).to(torch.bfloat16),
         "embed.norm": small(width), "final.norm": small(width),
         "head": (torch.randn((cfg["vocab"], width), generator=g) / width ** 0.5).to(torch.bfloat16)}
    for i, entry in enumerate(cfg["layers"]):
        if "weights_of" in entry:
            continue
        p = f"l{i}."
        w[p + "norm1"] = small(width)
        for name, t in mixer_weights(entry["type"], entry["mixer"], width, g, decay_rank).items():
            w[p + "mix." + name] = t
        if entry["mlp"] is not None:
            ff = entry["mlp"]["ff"]
            w[p + "norm2"] = small(width)
            w[p + "mlp.up"] = (torch.randn((ff, width), generator=g) * 1.5 / width ** 0.5).to(torch.bfloat16)
            w[p + "mlp.down"] = (torch.randn((width, ff), generator=g) / ff ** 0.5).to(torch.bfloat16)
            w[p + "mlp.act"] = torch.randn((2,), generator=g).to(torch.bfloat16)
    return w


def write_model(folder: str, cfg: dict, decay_rank: int, seed: int) -> str:
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_weights(cfg, decay_rank, seed))
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return folder


def make_model(tmp_path, name: str, seed: int = 5) -> str:
    cfg, rank = SMALL[name]
    d = os.path.join(str(tmp_path), f"ruvuvik_{name}_{seed}")
    if not os.path.isdir(d):
        write_model(d, cfg, rank, seed)
    return d
