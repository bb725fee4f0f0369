"""A plain, slow statement of the Mefolorn decoder: one function per mechanism, whole sequences,
32-bit arithmetic, no cache and no state. The tests compare the library with it; nothing here is
imported by the `llm_b200` package and nothing of the package is used here (the model folder is
read with this file's own safetensors reader).

Notation: x is the residual stream [T, width]; positions count from 0; W x is written x @ W.T.
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

def tanh_norm(x, alpha, weight, bias):
    """tanh(alpha x) * weight + bias, element by element: no statistic of the row enters."""
    return torch.tanh(alpha * x) * weight + bias


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def visible(n: int, window):
    """[n, n] booleans: query i sees key j if 0 <= i - j (and i - j < window, where there is one)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = j <= i
    if window:
        seen &= (i - j) < window
    return seen


def sink_softmax_attention(q, k, v, scale, window, sink):
    """One head. q, k [T, d], v [T, dv]. weights = e^s / (sum over visible keys of e^s + e^sink):
    the sink is one more term of the denominator, with no key, no value and no scale."""
    n = q.shape[0]
    scores = (q @ k.T) * scale
    scores = scores.masked_fill(~visible(n, window), float("-inf"))
    top = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink)
    e = torch.exp(scores - top)
    return (e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))) @ v


def latent_attention(h, w, prefix, m, eps):
    """Queries through a normed latent; keys and values of every head made from one normed latent
    c per position; windowed softmax with a sink per head; a sigmoid gate per head read from the
    mixer's input; output projection."""
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    window = (m.get("mask") or {}).get("size", 0)
    cq = rms_norm(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps)
    q = (cq @ w[prefix + "uq"].T).view(-1, heads, dim)
    c = rms_norm(h @ w[prefix + "dkv"].T, w[prefix + "dkv.norm"], eps)
    k = (c @ w[prefix + "uk"].T).view(-1, heads, dim)
    v = (c @ w[prefix + "uv"].T).view(-1, heads, vdim)
    gate = torch.sigmoid(h @ w[prefix + "g"].T)                      # [T, heads]
    outs = []
    for head in range(heads):
        o = sink_softmax_attention(q[:, head], k[:, head], v[:, head], m["scale"], window, w[prefix + "sink"][head])
        outs.append(o * gate[:, head:head + 1])
    return torch.cat(outs, dim=-1) @ w[prefix + "o"].T


def rotate_half(x, rot):
    """x [T, heads, d]: element i < n/2 of a head pairs with element i + n/2 (n = rot.dims); the
    pair (a, b) at position p becomes (a cos t - b sin t, b cos t + a sin t), t = p base^(-2i/n).
    Elements from n on stay."""
    n = rot["dims"]
    half = n // 2
    freq = torch.tensor([float(rot["base"]) ** (-2.0 * i / n) for i in range(half)], dtype=torch.float64)
    angle = torch.arange(x.shape[0], dtype=torch.float64)[:, None] * freq[None, :]
    cos, sin = angle.cos().float()[:, None, :], angle.sin().float()[:, None, :]
    a, b = x[..., :half], x[..., half:n]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., n:]], dim=-1)


def mixed_sigmoid_attention(h, w, prefix, m, eps):
    """Grouped heads; queries and keys normed over the whole projection, then rotated; the heads'
    scores of one (query, key) pair are mixed by a matrix; the weight of a visible key is
    sigmoid(mixed score + the head's bias), not normalised over the keys."""
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window = (m.get("mask") or {}).get("size", 0)
    n = h.shape[0]
    q = rms_norm(h @ w[prefix + "q"].T, w[prefix + "q.norm"], eps).view(n, heads, dim)
    k = rms_norm(h @ w[prefix + "k"].T, w[prefix + "k.norm"], eps).view(n, groups, dim)
    v = (h @ w[prefix + "v"].T).view(n, groups, vdim)
    if m.get("rot"):
        q, k = rotate_half(q, m["rot"]), rotate_half(k, m["rot"])
    per = heads // groups
    scores = torch.stack([(q[:, a] @ k[:, a // per].T) * m["scale"] for a in range(heads)])     # [heads, n, n]
    mixed = torch.einsum("hg,gij->hij", w[prefix + "talk"], scores)
    weights = torch.sigmoid(mixed + w[prefix + "pb"][:, None, None]) * visible(n, window)[None]
    outs = [weights[a] @ v[:, a // per] for a in range(heads)]
    return torch.cat(outs, dim=-1) @ w[prefix + "o"].T


def causal_conv(u, taps, bias):
    """u [T, C], taps [C, n]: y[t] = bias + sum_j taps[:, j] * u[t - (n - 1) + j], u = 0 before the start."""
    n = taps.shape[1]
    y = bias.expand_as(u).clone()
    for t in range(u.shape[0]):
        for j in range(n):
            src = t - (n - 1) + j
            if src >= 0:
                y[t] += taps[:, j] * u[src]
    return y


def block_gate(u, matrices, biases):
    """u [T, C] cut into len(matrices) equal parts; part b goes through its own square matrix."""
    blocks = matrices.shape[0]
    parts = u.view(u.shape[0], blocks, -1)
    out = torch.einsum("tbi,boi->tbo", parts, matrices) + biases[None]
    return torch.sigmoid(out).reshape(u.shape)


def gated_recurrence(h, w, prefix, m):
    """y = gelu(W_y h + b); u = conv(W_x h + b); per channel S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t
    with a_t = exp(-8 r_t softplus(lam)), S_(-1) = 0; output W_o (S * y)."""
    y = gelu_tanh(h @ w[prefix + "y"].T + w[prefix + "y.b"])
    u = causal_conv(h @ w[prefix + "x"].T + w[prefix + "x.b"], w[prefix + "conv"], w[prefix + "conv.b"])
    r = block_gate(u, w[prefix + "ra"], w[prefix + "ra.b"])
    i = block_gate(u, w[prefix + "ri"], w[prefix + "ri.b"])
    log_a = -8.0 * r * torch.nn.functional.softplus(w[prefix + "lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    state = torch.zeros(u.shape[1])
    states = []
    for t in range(u.shape[0]):
        state = a[t] * state + drive[t]
        states.append(state)
    return (torch.stack(states) * y) @ w[prefix + "o"].T


def side_by_side(h, w, prefix, m, eps):
    left = mixed_sigmoid_attention(h, w, prefix + "left.", m["left"], eps)
    right = gated_recurrence(h, w, prefix + "right.", m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def feed_forward(h, w, prefix):
    gate = h @ w[prefix + "gate"].T
    return ((gate * torch.sigmoid(gate)) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def mixer(h, w, prefix, layer, eps):
    if layer["type"] == "latent_attention":
        return latent_attention(h, w, prefix, layer["mixer"], eps)
    if layer["type"] == "parallel":
        return side_by_side(h, w, prefix, layer["mixer"], eps)
    raise ValueError(f"a layer of type {layer['type']!r}")


def norm_of(x, w, name):
    return tanh_norm(x, w[name + ".alpha"], w[name], w[name + ".b"])


def forward(config, w, tokens, streams=None):
    """Logits [T, vocab] of a whole sequence. `streams` (a list) receives x after every layer."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * (config.get("embedding") or {}).get("scale", 1.0)
    for i, layer in enumerate(config["layers"]):
        update = mixer(norm_of(x, w, f"l{i}.norm1"), w, f"l{i}.mix.", layer, eps)
        if layer.get("mlp"):
            update = update + feed_forward(norm_of(x, w, f"l{i}.norm2"), w, f"l{i}.mlp.")
        x = x + update
        if streams is not None:
            streams.append(x.clone())
    return norm_of(x, w, "final.norm") @ w["embed"].T


def greedy(config, w, prompt, n_new):
    tokens, out = list(prompt), []
    for _ in range(n_new):
        logits = forward(config, w, tokens)[-1]
        best = int((logits == logits.max()).nonzero()[0])
        out.append(best)
        tokens.append(best)
    return out
