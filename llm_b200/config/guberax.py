"""Configuration of the Guberax decoder, read from its own config.json keys.

A Guberax model is a list of layers, each `x += mixer(norm(x)) + feed_forward(norm(x))` with one
norm (weight stored around zero), a differential-attention mixer with a short causal convolution
behind its projections, partly rotated maps, a sliding window that keeps the first tokens, and a
dense gated feed-forward (or none). A range of layers may run several times in a row with the same
weights, every pass with a cache of its own and the embedding output added to the stream before
each pass but the first. The logits are soft-capped.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..errors import FormatError, Unsupported
from ..parts.spec import (DiffAttentionSpec, GatedMlpSpec, ModelSpec, NormSpec, ParallelBlockSpec,
                          PositionSpec, ScheduleEntry, names)
from .base import ConfigReader

# no key of the configuration bounds a sequence: the engine's context does
MAX_POSITIONS = 1 << 22


@dataclass(frozen=True)
class GuberaxConfig:
    """`raw` is the configuration as read; the typed view of it is `model_spec()`."""
    vocab: int
    width: int
    eps: float
    logit_softcap: float
    loop: tuple                       # (start, stop, times)
    layers: tuple                     # the 'layers' list, kept as JSON text per layer (hashable)

    architecture = "Guberax"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "GuberaxConfig":
        r = ConfigReader(raw, where)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise FormatError(f"{where}: 'layers' must be a non-empty list")
        norm = ConfigReader(r.mapping("norm"), f"{where}: norm")
        loop = r.mapping("loop", None)
        if loop is None:
            span = (0, 0, 1)
        else:
            l = ConfigReader(loop, f"{where}: loop")
            span = (l.integer("start", minimum=0), l.integer("stop", minimum=0), l.integer("times", 1, minimum=1))
            if not span[0] <= span[1] <= len(layers):
                raise FormatError(f"{where}: loop {span[0]} .. {span[1]} does not lie within {len(layers)} layers")
        config = cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                     eps=norm.number("eps", positive=True), logit_softcap=r.number("logit_softcap", 0.0),
                     loop=span, layers=tuple(json.dumps(layer, sort_keys=True) for layer in layers))
        config.model_spec()            # every layer is read once here, so that a bad key is reported at load
        return config

    def to_dict(self) -> dict:
        raw = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.eps}, "layers": [json.loads(text) for text in self.layers]}
        if self.logit_softcap:
            raw["logit_softcap"] = self.logit_softcap
        if self.loop != (0, 0, 1):
            raw["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return raw

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2) + "\n"

    # ------------------------------------------------------------------ the model as data

    def _mixer(self, i: int, raw: dict, where: str):
        m = ConfigReader(raw, where)
        dim = m.integer("dim", minimum=1)
        p = f"l{i}.mix."
        roles = {r: p + r for r in ("q", "k", "v", "o", "lq1", "lk1", "lq2", "lk2")}
        taps = m.integer("conv", 0, minimum=0)
        if taps:
            roles.update({f"{r}_conv": f"{p}{r}.conv" for r in ("q", "k", "v")})
        position = None
        rot = m.mapping("rot", None)
        if rot is not None:
            rr = ConfigReader(rot, f"{where}: rot")
            dims = rr.integer("dims", minimum=2)
            if dims % 2 or dims > dim:
                raise FormatError(f"{where}: rot.dims {dims} must be even and at most dim {dim}")
            scaling = rr.mapping("scaling", None)
            if scaling is not None:
                s = ConfigReader(scaling, f"{where}: rot.scaling")
                scaling = {"rope_type": "llama3", "factor": s.number("factor", positive=True),
                           "low_freq_factor": s.number("low", positive=True),
                           "high_freq_factor": s.number("high", positive=True),
                           "original_max_position_embeddings": s.number("original", positive=True)}
                if scaling["high_freq_factor"] <= scaling["low_freq_factor"]:
                    raise FormatError(f"{where}: rot.scaling.high must exceed low")
            position = PositionSpec(head_dim=dim, theta=rr.number("base", positive=True),
                                    max_positions=MAX_POSITIONS,
                                    scaling=tuple(sorted(scaling.items())) if scaling else None,
                                    pairing="interleaved", rotary_dim=dims)
        mask = m.mapping("mask", None)
        window = keep_first = 0
        if mask is not None:
            mm = ConfigReader(mask, f"{where}: mask")
            window = mm.integer("size", 0, minimum=0)
            keep_first = mm.integer("keep_first", 0, minimum=0) if window else 0
        return DiffAttentionSpec(
            hidden=self.width, n_heads=m.integer("heads", minimum=1), n_kv_heads=m.integer("kv_heads", minimum=1),
            head_dim=dim, value_dim=m.integer("vdim", minimum=1), scale=m.number("scale"), window=window,
            keep_first=keep_first, conv_taps=taps, diff=m.number("diff"), eps=self.eps, position=position,
            names=names(**roles))

    def model_spec(self) -> ModelSpec:
        blocks = []
        for i, text in enumerate(self.layers):
            layer = json.loads(text)
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, dict):
                raise FormatError(f"{where} is not an object")
            kind = layer.get("type")
            if kind != "attention":
                raise Unsupported(f"{where}: a layer of type '{kind}' (built: 'attention')")
            if not isinstance(layer.get("mixer"), dict):
                raise FormatError(f"{where}: 'mixer' must be an object")
            mixer = self._mixer(i, layer["mixer"], f"{where}.mixer")
            ffn = None
            mlp = layer.get("mlp")
            if mlp is not None:
                f = ConfigReader(mlp, f"{where}.mlp")
                if f.string("kind", "dense") != "dense":
                    raise Unsupported(f"{where}.mlp: kind '{f.string('kind')}' (built: 'dense')")
                p = f"l{i}.mlp."
                ffn = GatedMlpSpec(hidden=self.width, intermediate=f.integer("ff", minimum=1), activation="silu",
                                   names=names(gate=p + "gate", up=p + "up", down=p + "down"))
            blocks.append(ParallelBlockSpec(
                norm=NormSpec(self.width, self.eps, f"l{i}.norm1", unit_offset=True), mixer=mixer, feed_forward=ffn))
        start, stop, times = self.loop
        schedule = [ScheduleEntry(i) for i in range(start)]
        for run in range(times):
            schedule += [ScheduleEntry(i, add_embedding=(run > 0 and i == start)) for i in range(start, stop)]
        schedule += [ScheduleEntry(i) for i in range(stop, len(blocks))]
        return ModelSpec(
            architecture=self.architecture, vocab=self.vocab, hidden=self.width, max_positions=MAX_POSITIONS,
            embedding="embed", blocks=tuple(blocks), schedule=tuple(schedule),
            final_norm=NormSpec(self.width, self.eps, "final.norm", unit_offset=True), head="head",
            logit_softcap=self.logit_softcap)
