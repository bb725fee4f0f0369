"""Tiny Mefolorn configurations and weights for the tests.

The configurations differ in every size and option and avoid coincidences that would hide a mix-up:
value sizes that differ from the key sizes, latents of other sizes than the heads, groups of 1, 2
and 4 query heads, rotated parts shorter than a head, one, two and three gate blocks, one to four
taps, windows shorter and longer than a page and than the prompts, layers with and without a
feed-forward, layer orders that start with either kind, scales that are not 1.
"""
from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import torch


def _latent(heads, dim, vdim, q_rank, kv_rank, window, scale=None):
    out = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
           "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window:
        out["mask"] = {"size": window}
    return out


def _left(heads, kv_heads, dim, vdim, window, rot=None, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
           "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window:
        out["mask"] = {"size": window}
    if rot is not None:
        out["rot"] = rot
    return out


def _pair(left, width, blocks, conv, left_scale, right_scale):
    return {"left": left, "right": {"width": width, "blocks": blocks, "conv": conv},
            "left_scale": left_scale, "right_scale": right_scale}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# P: small and odd everywhere; a layer without feed-forward; the pair first
MEF_P = {
    "architecture": "Mefolorn", "vocab": 97, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
    "layers": [
        _layer("parallel", _pair(_left(4, 2, 6, 10, 9, rot={"base": 100.0, "dims": 4}), 24, 3, 3, 0.7, 1.2), 52),
        _layer("latent_attention", _latent(3, 10, 7, 12, 9, 5), 0),
        _layer("parallel", _pair(_left(2, 2, 8, 5, 33, rot={"base": 10000.0, "dims": 8}, scale=0.2), 14, 1, 1, 1.3, 0.4), 36),
        _layer("latent_attention", _latent(2, 4, 12, 20, 34, 21, scale=0.3), 44),
    ],
}

# Q: sizes that tensor-core kernels take; windows wider and narrower than a page; the latent first
MEF_Q = {
    "architecture": "Mefolorn", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
    "layers": [
        _layer("latent_attention", _latent(4, 32, 64, 48, 64, 70), 192),
        _layer("parallel", _pair(_left(4, 2, 64, 32, 40, rot={"base": 200000.0, "dims": 32}), 96, 3, 4, 0.5, 0.8), 192),
        _layer("latent_attention", _latent(8, 16, 16, 64, 32, 130), 192),
        _layer("parallel", _pair(_left(4, 1, 32, 64, 100, rot={"base": 5000.0, "dims": 32}), 128, 2, 2, 0.9, 0.6), 192),
    ],
}

# R: one layer of each kind, no window, no rotation, no embedding scale: everything optional is absent
MEF_R = {
    "architecture": "Mefolorn", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [
        _layer("parallel", _pair(_left(2, 1, 16, 24, 0), 32, 2, 4, 1.0, 1.0), 48),
        _layer("latent_attention", _latent(2, 8, 8, 16, 16, 0), 48),
    ],
}

CONFIGS = {"P": (MEF_P, 21), "Q": (MEF_Q, 22), "R": (MEF_R, 23)}


def tensor_shapes(config) -> dict:
    """Every tensor of a model of this configuration with its shape (written out here, not taken
    from the library)."""
    width = config["width"]
    out = {"embed": (config["vocab"], width)}

    def norm(name):
        out.update({name: (width,), name + ".b": (width,), name + ".alpha": ()})

    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        norm(p + "norm1")
        if layer["type"] == "latent_attention":
            h = m["heads"]
            out.update({p + "mix.dq": (m["q_rank"], width), p + "mix.dq.norm": (m["q_rank"],),
                        p + "mix.uq": (h * m["dim"], m["q_rank"]), p + "mix.dkv": (m["kv_rank"], width),
                        p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (h * m["dim"], m["kv_rank"]),
                        p + "mix.uv": (h * m["vdim"], m["kv_rank"]), p + "mix.sink": (h,), p + "mix.g": (h, width),
                        p + "mix.o": (width, h * m["vdim"])})
        else:
            l, r = m["left"], m["right"]
            q, k, v = l["heads"] * l["dim"], l["kv_heads"] * l["dim"], l["kv_heads"] * l["vdim"]
            lp, rp = p + "mix.left.", p + "mix.right."
            out.update({lp + "q": (q, width), lp + "k": (k, width), lp + "v": (v, width), lp + "q.norm": (q,),
                        lp + "k.norm": (k,), lp + "talk": (l["heads"], l["heads"]), lp + "pb": (l["heads"],),
                        lp + "o": (width, l["heads"] * l["vdim"])})
            c, part = r["width"], r["width"] // r["blocks"]
            out.update({rp + "y": (c, width), rp + "y.b": (c,), rp + "x": (c, width), rp + "x.b": (c,),
                        rp + "conv": (c, r["conv"]), rp + "conv.b": (c,), rp + "ra": (r["blocks"], part, part),
                        rp + "ra.b": (r["blocks"], part), rp + "ri": (r["blocks"], part, part),
                        rp + "ri.b": (r["blocks"], part), rp + "lam": (c,), rp + "o": (width, c)})
        if layer.get("mlp"):
            norm(p + "norm2")
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, width), p + "mlp.up": (ff, width), p + "mlp.down": (width, ff)})
    norm("final.norm")
    return out


def random_weights(config, seed: int, dtype=torch.bfloat16) -> dict:
    """Weights of a size at which every mechanism matters: projections that give values of order 1,
    norm weights, biases, sinks, head biases and decay parameters well away from zero, a mixing
    matrix that is neither the identity nor small."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            t = torch.tensor(0.4) + 0.2 * torch.rand((), generator=gen)
        elif last in ("norm1", "norm2") or name in ("final.norm",) or name.endswith(".norm"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last == "b":
            t = 0.2 * torch.randn(shape, generator=gen)
        elif last == "conv":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif last in ("sink", "pb", "lam"):
            t = torch.randn(shape, generator=gen)
        elif last == "talk":
            t = torch.eye(shape[0]) + 0.5 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
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
    return write_folder(Path(tmp_path) / f"mef_{which}_{str(dtype).split('.')[-1]}", config, weights)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=gen).tolist()
