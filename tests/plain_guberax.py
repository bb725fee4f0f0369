"""A plain, slow statement of the Guberax decoder: one function per mechanism, whole sequences,
32-bit arithmetic, no cache. The tests compare the library with it; nothing here is imported by
the `llm_b200` package and nothing of the package is used here (the model folder is read with
this file's own safetensors reader).

Notation: x is the residual stream [T, width]; positions count from 0.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}


def read_model_folder(folder):
    """(config dictionary, {tensor name: float32 tensor}) of a model folder."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    weights = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        data = torch.frombuffer(bytearray(raw[8 + n + a:8 + n + b]), dtype=_DTYPES[meta["dtype"]])
        weights[name] = data.reshape(meta["shape"]).to(torch.float32)
    return config, weights


# ----------------------------------------------------------------------------- mechanisms

def offset_norm(x, weight, eps):
    """x * (1 + weight) / r, r = the root of (the mean of x's squares + eps)."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (1.0 + weight)


def unit_norm(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def short_conv(u, taps):
    """u [T, C], taps [C, n]: y[t] = sum_j taps[:, j] * u[t - n + 1 + j], u = 0 before the start."""
    n = taps.shape[1]
    y = torch.zeros_like(u)
    for t in range(u.shape[0]):
        for j in range(n):
            src = t - n + 1 + j
            if src >= 0:
                y[t] += taps[:, j] * u[src]
    return y


def rotation_frequencies(rot):
    """f_i = base^(-2i/dims), then the band-wise slow-down of long wavelengths."""
    dims = rot["dims"]
    out = []
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        s = rot.get("scaling")
        if s:
            wavelength = 2.0 * math.pi / f
            if wavelength > s["original"] / s["low"]:
                f = f / s["factor"]
            elif wavelength >= s["original"] / s["high"]:
                blend = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
                f = (1.0 - blend) * f / s["factor"] + blend * f
        out.append(f)
    return out


def rotate(x, rot, positions):
    """x [T, units, dim]: elements (2i, 2i+1), i < dims/2, of every unit turn by position * f_i."""
    freqs = rotation_frequencies(rot)
    out = x.clone()
    for t, p in enumerate(positions):
        for i, f in enumerate(freqs):
            angle = p * f
            c, s = math.cos(angle), math.sin(angle)
            u, v = x[t, :, 2 * i], x[t, :, 2 * i + 1]
            out[t, :, 2 * i] = u * c - v * s
            out[t, :, 2 * i + 1] = v * c + u * s
    return out


def visible(i, j, mask):
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if not mask or not mask.get("size"):
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


def softmax_attention(q, k, v, scale, mask):
    """q [T, d], k [T, d], v [T, dv] of one map of one head -> [T, dv]."""
    n = q.shape[0]
    scores = (q @ k.T) * scale
    see = torch.tensor([[visible(i, j, mask) for j in range(n)] for i in range(n)])
    scores = scores.masked_fill(~see, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def diff_lambda(w, prefix, diff):
    return float(torch.exp((w[prefix + "lq1"] * w[prefix + "lk1"]).sum())
                 - torch.exp((w[prefix + "lq2"] * w[prefix + "lk2"]).sum()) + diff)


def mixer(h, w, prefix, m, eps):
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q, k, v = h @ w[prefix + "q"].T, h @ w[prefix + "k"].T, h @ w[prefix + "v"].T
    if m.get("conv"):
        q = short_conv(q, w[prefix + "q.conv"])
        k = short_conv(k, w[prefix + "k.conv"])
        v = short_conv(v, w[prefix + "v.conv"])
    q, k, v = q.view(n, heads * 2, dim), k.view(n, groups * 2, dim), v.view(n, groups, vdim)
    if m.get("rot"):
        q, k = rotate(q, m["rot"], range(n)), rotate(k, m["rot"], range(n))
    lam = diff_lambda(w, prefix, m["diff"])
    outs = []
    for head in range(heads):
        g = head // (heads // groups)
        a1 = softmax_attention(q[:, 2 * head], k[:, 2 * g], v[:, g], m["scale"], m.get("mask"))
        a2 = softmax_attention(q[:, 2 * head + 1], k[:, 2 * g + 1], v[:, g], m["scale"], m.get("mask"))
        outs.append(unit_norm(a1 - lam * a2, eps) * (1.0 - m["diff"]))
    return torch.cat(outs, dim=-1) @ w[prefix + "o"].T


def feed_forward(h, w, prefix):
    gate = h @ w[prefix + "gate"].T
    return ((gate * torch.sigmoid(gate)) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def layer_runs(config):
    """[(layer, whether the embedding output is added before it)] in running order."""
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, False) for i in range(loop["start"])]
    for again in range(loop["times"]):
        runs += [(i, again > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(config, w, tokens, streams=None):
    """Logits [T, vocab] of a whole sequence. `streams` (a list) receives x after every layer run."""
    eps = config["norm"]["eps"]
    x0 = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    for i, add in layer_runs(config):
        if add:
            x = x + x0
        layer = config["layers"][i]
        h = offset_norm(x, w[f"l{i}.norm1"], eps)
        update = mixer(h, w, f"l{i}.mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            update = update + feed_forward(h, w, f"l{i}.mlp.")
        x = x + update
        if streams is not None:
            streams.append(x.clone())
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def greedy(config, w, prompt, n_new):
    tokens, out = list(prompt), []
    for _ in range(n_new):
        logits = forward(config, w, tokens)[-1]
        best = int((logits == logits.max()).nonzero()[0])
        out.append(best)
        tokens.append(best)
    return out
