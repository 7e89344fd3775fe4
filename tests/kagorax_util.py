"""Small Kagorax configurations with random weights, written as model folders by the tests.

The weights are drawn here with torch's generator (not with the package's), large enough that
every mechanism moves the logits: biases of the projections, the distance table, the router.
Matrices are stored in bfloat16, so the plain implementation and the engine read the same values.
"""
from __future__ import annotations

import json
import os

import torch

from tinyinfer_b200.weights.safetensors_io import write_safetensors


def _mixer(heads, kv_heads, dim, vdim, scale, bias_max, size, keep_first, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "bias_max": bias_max, "mask": {"size": size, "keep_first": keep_first}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, shared_ff=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff is not None:
        m["shared"] = {"ff": shared_ff}
    return m


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


# every size differs between layers where the design allows it: value heads of their own size, a
# reader of another layer's keys with a wider window and more kept tokens than the owner's, a layer
# without a feed-forward, one without a shared expert, one kv head, no kept tokens
SMALL_A = {
    "architecture": "Kagorax", "vocab": 211, "width": 64, "embedding": {"scale": 6.5}, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mixer(4, 2, 16, 24, 0.31, 40, 20, 3), _moe(4, 2, 32, 48)),
        _layer(_mixer(4, 2, 16, 24, 0.22, 64, 33, 5, kv_from=0), None),
        _layer(_mixer(6, 1, 32, 32, 0.17, 100, 9, 0), _moe(3, 1, 16)),
    ]}
ROWS_A = [8, 12, 6]

# values that make branches coincide: one head, all experts chosen, a window longer than any
# prompt, a table of four rows
SMALL_B = {
    "architecture": "Kagorax", "vocab": 97, "width": 32, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_mixer(1, 1, 8, 8, 0.5, 16, 1000, 1), _moe(2, 2, 8, 8)),
        _layer(_mixer(1, 1, 8, 8, 0.4, 12, 1000, 0, kv_from=0), _moe(2, 1, 8, 24)),
    ]}
ROWS_B = [4, 6]

# sizes that the tensor-core kernels take (head size 64, widths that are multiples of 32)
SMALL_C = {
    "architecture": "Kagorax", "vocab": 1008, "width": 128, "embedding": {"scale": 11.0}, "norm": {"eps": 2e-6},
    "layers": [
        _layer(_mixer(8, 2, 64, 64, 0.125, 200, 48, 4), _moe(8, 2, 64, 96)),
        _layer(_mixer(8, 2, 64, 64, 0.11, 120, 70, 2), _moe(6, 3, 32, 64)),
        _layer(_mixer(8, 2, 64, 64, 0.2, 300, 100, 7, kv_from=1), _moe(8, 1, 64)),
    ]}
ROWS_C = [16, 10, 32]

# head size 128: prompt portions take the tcgen05 attention kernel; windows shorter than the prompts,
# so that tiles of kept first tokens are walked apart from the window's
SMALL_D = {
    "architecture": "Kagorax", "vocab": 500, "width": 128, "embedding": {"scale": 9.0}, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mixer(2, 1, 128, 128, 0.09, 260, 150, 3), _moe(4, 2, 32, 32)),
        _layer(_mixer(4, 2, 128, 128, 0.1, 90, 40, 130), _moe(4, 1, 64)),
        _layer(_mixer(4, 2, 128, 128, 0.08, 500, 260, 1, kv_from=1), None),
    ]}
ROWS_D = [12, 8, 20]

# sizes that no tensor-core kernel takes (a width that is no multiple of 32, head sizes that are no
# multiples of 16, an odd table): every call must find its general kernel, in both precisions
SMALL_E = {
    "architecture": "Kagorax", "vocab": 301, "width": 72, "embedding": {"scale": 5.0}, "norm": {"eps": 3e-6},
    "layers": [
        _layer(_mixer(3, 1, 40, 24, 0.16, 77, 50, 2), _moe(5, 2, 24, 40)),
        _layer(_mixer(6, 3, 8, 8, 0.35, 30, 19, 9), _moe(3, 3, 56)),
        _layer(_mixer(6, 3, 8, 8, 0.3, 45, 64, 0, kv_from=1), _moe(7, 1, 8, 8)),
    ]}
ROWS_E = [9, 6, 14]

SMALL = {"A": (SMALL_A, ROWS_A), "B": (SMALL_B, ROWS_B), "C": (SMALL_C, ROWS_C), "D": (SMALL_D, ROWS_D),
         "E": (SMALL_E, ROWS_E)}


def random_weights(cfg: dict, table_rows, seed: int) -> dict:
    g = torch.Generator().manual_seed(seed)
    width = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return (torch.randn((rows, cols), generator=g) * gain / cols ** 0.5).to(torch.bfloat16)

    def vec(n, std):
        return (torch.randn((n,), generator=g) * std).to(torch.bfloat16)

    w = {"embed": (torch.randn((cfg["vocab"], width), generator=g) * 0.3).to(torch.bfloat16),
         "final.norm": (1.0 + 0.1 * torch.randn((width,), generator=g)).to(torch.bfloat16)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        w[p + "norm1"] = (1.0 + 0.1 * torch.randn((width,), generator=g)).to(torch.bfloat16)
        nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        w[p + "mix.q"], w[p + "mix.q.b"] = mat(nq, width, 2.0), vec(nq, 0.5)
        if "kv_from" not in m:
            w[p + "mix.k"], w[p + "mix.k.b"] = mat(nk, width, 2.0), vec(nk, 0.5)
            w[p + "mix.v"], w[p + "mix.v.b"] = mat(nv, width), vec(nv, 0.3)
        w[p + "mix.rel"] = (torch.randn((table_rows[i], m["heads"]), generator=g) * 1.5).to(torch.bfloat16)
        w[p + "mix.g"] = mat(m["heads"] * m["vdim"], width, 2.0)
        w[p + "mix.o"] = mat(width, m["heads"] * m["vdim"])
        mlp = layer["mlp"]
        if mlp is None:
            continue
        q = p + "mlp."
        ff = mlp["expert"]["ff"]
        w[q + "router"] = mat(mlp["router"]["experts"], width, 3.0)
        for e in range(mlp["router"]["experts"]):
            w[f"{q}e{e}.gate"], w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = mat(ff, width, 1.5), mat(ff, width, 1.5), mat(width, ff, 1.5)
        if mlp.get("shared") is not None:
            sf = mlp["shared"]["ff"]
            w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"] = mat(sf, width), mat(sf, width), mat(width, sf)
            w[q + "shared.sg"] = mat(1, width, 2.0)
    return w


def write_model(folder: str, cfg: dict, table_rows, seed: int) -> str:
    os.makedirs(folder, exist_ok=True)
    write_safetensors(os.path.join(folder, "model.safetensors"), random_weights(cfg, table_rows, seed))
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return folder


def make_model(tmp_path, name: str, seed: int = 3) -> str:
    cfg, rows = SMALL[name]
    d = os.path.join(str(tmp_path), f"kagorax_{name}_{seed}")
    if not os.path.isdir(d):
        write_model(d, cfg, rows, seed)
    return d
