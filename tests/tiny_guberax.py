"""Tiny Guberax configurations and weights for the tests.

The configurations differ in every size and option, and avoid coincidences that would hide a
mix-up: value sizes that are not twice the map size, groups of 1, 2 and 4 query heads, rotated
parts shorter than a map, layers with and without feed-forward, with and without convolution,
window, kept first tokens, rotation and frequency scaling, repeated ranges that start at layer 0 or
later and run two or three times, and layers of one model that differ from each other.
"""
from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def _mixer(heads, kv_heads, dim, vdim, conv=0, diff=0.3, mask=None, rot=None, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
           "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if conv:
        out["conv"] = conv
    if mask is not None:
        out["mask"] = mask
    if rot is not None:
        out["rot"] = rot
    return out


def _layer(mixer, ff):
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


SCALED = {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 32}

# P: small and odd everywhere; the second layer has no feed-forward and other sizes than the first
GUB_P = {
    "architecture": "Guberax", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
    "loop": {"start": 1, "stop": 2, "times": 3},
    "layers": [
        _layer(_mixer(4, 2, 6, 10, conv=3, diff=0.25, mask={"size": 9, "keep_first": 2},
                      rot={"base": 100.0, "dims": 4, "scaling": SCALED}), 52),
        _layer(_mixer(3, 3, 10, 7, conv=2, diff=0.4, mask={"size": 5, "keep_first": 0},
                      rot={"base": 10000.0, "dims": 10}), 0),
        _layer(_mixer(2, 1, 8, 12, conv=0, diff=0.1, mask=None, rot=None), 36),
    ],
}

# Q: sizes that the tensor-core kernels take, windows wider and narrower than a page, the
# repeated range from layer 0, no soft cap
GUB_Q = {
    "architecture": "Guberax", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        _layer(_mixer(4, 1, 32, 32, conv=4, diff=0.35, mask={"size": 70, "keep_first": 3},
                      rot={"base": 200000.0, "dims": 16, "scaling": SCALED}), 192),
        _layer(_mixer(4, 2, 32, 64, conv=3, diff=0.35, mask={"size": 70, "keep_first": 3},
                      rot={"base": 200000.0, "dims": 32}), 192),
        _layer(_mixer(2, 2, 64, 64, conv=4, diff=0.2, mask={"size": 33, "keep_first": 1},
                      rot={"base": 200000.0, "dims": 64}), 192),
    ],
}

# R: one layer, no repeated range, no window: everything optional is absent
GUB_R = {
    "architecture": "Guberax", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [_layer(_mixer(2, 1, 16, 24), 48)],
}

CONFIGS = {"P": (GUB_P, 11), "Q": (GUB_Q, 12), "R": (GUB_R, 13)}


def tensor_shapes(config) -> dict:
    """Every tensor of a model of this configuration with its shape (written out here, not taken
    from the library)."""
    width = config["width"]
    out = {"embed": (config["vocab"], width), "final.norm": (width,), "head": (config["vocab"], width)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        q, k, v = m["heads"] * 2 * m["dim"], m["kv_heads"] * 2 * m["dim"], m["kv_heads"] * m["vdim"]
        out[p + "norm1"] = (width,)
        out.update({p + "mix.q": (q, width), p + "mix.k": (k, width), p + "mix.v": (v, width),
                    p + "mix.o": (width, m["heads"] * m["vdim"])})
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[p + "mix." + name] = (m["dim"],)
        if m.get("conv"):
            out.update({p + "mix.q.conv": (q, m["conv"]), p + "mix.k.conv": (k, m["conv"]),
                        p + "mix.v.conv": (v, m["conv"])})
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, width), p + "mlp.up": (ff, width), p + "mlp.down": (width, ff)})
    return out


def random_weights(config, seed: int, dtype=torch.bfloat16) -> dict:
    """Weights of a size at which every mechanism matters at these widths: projections that give
    queries and keys of order 1, taps of order 1 / sqrt(taps), norm weights and gate vectors well
    away from zero."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        if name.endswith("norm1") or name == "final.norm":
            t = 0.3 * torch.randn(shape, generator=gen)
        elif name.endswith(".conv"):
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif name.rsplit(".", 1)[-1] in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.4 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        out[name] = t.to(dtype)
    return out


def write_folder(folder, config, weights) -> Path:
    from llm_b200.weights.safetensors_io import write_safetensors
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    write_safetensors(folder / "model.safetensors", {k: v.contiguous() for k, v in weights.items()}, {"format": "pt"})
    return folder


def make_folder(tmp_path, which: str, dtype=torch.bfloat16, change=None, weights_change=None):
    """Write the folder of tiny configuration `which`; `change(config)` may alter a copy of the
    configuration first, `weights_change(weights)` the weights."""
    raw, seed = CONFIGS[which]
    config = copy.deepcopy(raw)
    if change is not None:
        change(config)
    weights = random_weights(config, seed, dtype)
    if weights_change is not None:
        weights_change(weights)
    return write_folder(Path(tmp_path) / f"gub_{which}_{str(dtype).split('.')[-1]}", config, weights)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
