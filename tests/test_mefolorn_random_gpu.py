"""Randomly drawn tiny Mefolorn configurations (seeded): any order of the two layer kinds, head,
value, latent and recurrence sizes that the tensor-core kernels take and sizes no tile takes, groups
of 1 to 8 heads, windows from 1 to beyond the prompts, rotated parts shorter than a head, one to
five gate blocks, one to five taps, layers without feed-forward. Each runs a batch of unequal
prompts and then decodes, shorter requests leaving earlier, in 32-bit and in bfloat16, against the
plain implementation."""
import math
import random

import pytest
import torch

import plain_mefolorn as plain
from tiny_mefolorn import random_weights, write_folder

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def draw_config(rng) -> dict:
    width = rng.choice([48, 64, 96, 128, 160, 256])

    def window():
        return rng.choice([0, 1, 2, 7, 33, 64, 65, 100, 128, 190, 1000])

    def latent():
        dim, vdim = rng.choice([8, 16, 24, 32, 64]), rng.choice([8, 16, 40, 32, 64])
        out = {"heads": rng.choice([1, 2, 3, 4, 8, 12]), "dim": dim, "vdim": vdim,
               "q_rank": rng.choice([8, 24, 40, 64, 96]), "kv_rank": rng.choice([8, 20, 32, 64, 64, 96, 128, 136]),
               "scale": rng.choice([1.0 / math.sqrt(dim), 0.2])}
        w = window()
        if w:
            out["mask"] = {"size": w}
        return out

    def pair():
        kv = rng.choice([1, 2, 2, 3, 4])
        heads = kv * rng.choice([1, 2, 4, 8]) if kv < 4 else kv * rng.choice([1, 2])
        dim, vdim = rng.choice([(32, 32), (32, 64), (64, 32), (64, 64), (96, 96), (64, 128), (128, 64), (16, 24), (40, 8), (8, 8)])
        left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 1.0 / math.sqrt(dim)}
        w = window()
        if w:
            left["mask"] = {"size": w}
        if rng.random() < 0.8:
            left["rot"] = {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": rng.choice([dim, dim // 2, 2, dim - 2 if dim > 2 else 2]) // 2 * 2 or 2}
        blocks = rng.choice([1, 2, 3, 4, 5])
        return {"left": left, "right": {"width": blocks * rng.choice([4, 16, 20, 32, 64]), "blocks": blocks, "conv": rng.choice([1, 2, 3, 4, 5])},
                "left_scale": rng.choice([0.5, 1.0, 1.5]), "right_scale": rng.choice([0.3, 1.0, 2.0])}

    layers = []
    for _ in range(rng.choice([1, 2, 3, 4])):
        kind = rng.choice(["latent_attention", "parallel"])
        ff = rng.choice([0, 32, 80, 128, 200])
        layers.append({"type": kind, "mixer": latent() if kind == "latent_attention" else pair(),
                       "mlp": {"kind": "dense", "ff": ff} if ff else None})
    return {"architecture": "Mefolorn", "vocab": rng.choice([61, 128, 300, 1000]), "width": width,
            "norm": {"eps": rng.choice([1e-5, 1e-6, 1e-3])}, "embedding": {"scale": rng.choice([1.0, 4.0, 12.0])},
            "layers": layers}


def close(got, want, dtype, scale) -> bool:
    """`scale`: the largest logit of the whole sequence (the sigmoid attention sums up to a window of weights
    that are not normalised, so a row's rounding error goes with the stream's size, not with the row's own)."""
    got, want = got.float().cpu(), want.float()
    if dtype == torch.float32:
        return float((got - want).abs().max()) <= 3e-4 * max(scale, 1.0)
    error = (got - want).abs()
    return float(error.max()) <= 0.05 * scale and float(error.mean()) <= 0.01 * scale


@pytest.mark.parametrize("case", range(100, 124))
def test_random_configuration(tmp_path, case):
    from llm_b200.engine import Engine, Entry, load_model
    rng = random.Random(10300 + case)
    raw = draw_config(rng)
    drawn = random_weights(raw, 500 + case)
    for name in drawn:                      # weights that are not normalised stay small, as in a trained model: without
        if name.endswith(".pb"):            # this a window of 1,000 sums hundreds of weights near one half, and bfloat16
            drawn[name] = (drawn[name].float() - 3.0).to(drawn[name].dtype)     # rounding of the values decides the logits
    folder = write_folder(tmp_path / "model", raw, drawn)
    config, weights = plain.read_model_folder(folder)
    lengths = [rng.choice([1, 3, 17, 64, 65, 127, 128, 129, 200, 300]) for _ in range(rng.choice([1, 2, 3, 5]))]
    extra = [rng.choice([1, 2, 8, 33]) for _ in lengths]
    gen = torch.Generator().manual_seed(case)
    seqs = [torch.randint(0, raw["vocab"], (n + e,), generator=gen).tolist() for n, e in zip(lengths, extra)]
    expected = [plain.forward(config, weights, s) for s in seqs]
    scales = [float(e.abs().max()) for e in expected]
    for dtype in (torch.float32, torch.bfloat16):
        engine = Engine(load_model(folder, dtype, DEV), max_tokens=64 * 7 * len(seqs), max_slots=len(seqs))
        slots = engine.acquire(len(seqs))
        logits = engine.step([Entry(s, q[:n], list(range(n))) for s, q, n in zip(slots, seqs, lengths)])
        at = 0
        for b, n in enumerate(lengths):
            assert close(logits[at:at + n], expected[b][:n], dtype, scales[b]), (raw, dtype, "prompt", b, lengths)
            at += n
        live = list(range(len(seqs)))
        for k in range(max(extra)):
            ended = [b for b in live if k >= extra[b]]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
            if not live:
                break
            logits = engine.step([Entry(slots[b], [seqs[b][lengths[b] + k]], [0]) for b in live])
            for row, b in enumerate(live):
                assert close(logits[row], expected[b][lengths[b] + k], dtype, scales[b]), (raw, dtype, "step", k, b, lengths)
        engine.release([slots[b] for b in live])
        engine.cache.check()
        engine.check()
