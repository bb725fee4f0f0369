"""Configuration of the Mefolorn decoder, read from its own config.json keys.

A Mefolorn model is a list of layers, each `x += mixer(norm1(x)) + feed_forward(norm2(x))` with
two tanh norms of the same x (y = tanh(alpha x) * weight + bias). A layer's `type` names its
mixer: `latent_attention` (queries and keys/values through normed latents, only the key/value
latent cached, a sliding window, a softmax with a sink term per head, a sigmoid gate per head), or
`parallel` (two mixers side by side: a grouped sigmoid attention with query/key norms over the
whole projection, partly rotated heads, mixed heads and a window, and a gated linear recurrence
behind a short convolution). The embedding is scaled, and the head is the embedding table itself.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..errors import FormatError, Unsupported
from ..parts.spec import (GatedMlpSpec, GatedRecurrenceSpec, LatentAttentionSpec, ModelSpec, ParallelBlockSpec,
                          PositionSpec, ScheduleEntry, SideBySideSpec, SigmoidAttentionSpec, TanhNormSpec, names)
from .base import ConfigReader

# no key of the configuration bounds a sequence: the engine's context does
MAX_POSITIONS = 1 << 22
# the recurrence's decay constant: log a = -8 r softplus(lam)
RECURRENCE_DECAY = 8.0


def _window(reader, where):
    mask = reader.mapping("mask", None)
    if mask is None:
        return 0
    return ConfigReader(mask, f"{where}: mask").integer("size", 0, minimum=0)


@dataclass(frozen=True)
class MefolornConfig:
    """`raw` is the configuration as read; the typed view of it is `model_spec()`."""
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple                     # the 'layers' list, kept as JSON text per layer (hashable)

    architecture = "Mefolorn"

    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "MefolornConfig":
        r = ConfigReader(raw, where)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise FormatError(f"{where}: 'layers' must be a non-empty list")
        norm = ConfigReader(r.mapping("norm"), f"{where}: norm")
        embedding = r.mapping("embedding", None)
        scale = ConfigReader(embedding, f"{where}: embedding").number("scale", 1.0) if embedding is not None else 1.0
        config = cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                     eps=norm.number("eps", positive=True), embedding_scale=scale,
                     layers=tuple(json.dumps(layer, sort_keys=True) for layer in layers))
        config.model_spec()            # every layer is read once here, so that a bad key is reported at load
        return config

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale},
                "layers": [json.loads(text) for text in self.layers]}

    def to_json(self) -> str:
        return json.dumps(self.to_dict(), indent=2) + "\n"

    # ------------------------------------------------------------------ the model as data

    def _latent(self, p: str, raw: dict, where: str):
        m = ConfigReader(raw, where)
        roles = {"dq": p + "dq", "dq_norm": p + "dq.norm", "uq": p + "uq", "dkv": p + "dkv",
                 "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv", "o": p + "o",
                 "sink": p + "sink", "gate": p + "g"}
        return LatentAttentionSpec(
            hidden=self.width, n_heads=m.integer("heads", minimum=1), head_dim=m.integer("dim", minimum=1),
            value_dim=m.integer("vdim", minimum=1), q_rank=m.integer("q_rank", minimum=1),
            kv_rank=m.integer("kv_rank", minimum=1), scale=m.number("scale"), window=_window(m, where),
            eps=self.eps, sink=True, gate=True, names=names(**roles))

    def _sigmoid(self, p: str, raw: dict, where: str, out_scale: float):
        m = ConfigReader(raw, where)
        dim = m.integer("dim", minimum=1)
        position = None
        rot = m.mapping("rot", None)
        if rot is not None:
            rr = ConfigReader(rot, f"{where}: rot")
            dims = rr.integer("dims", minimum=2)
            if dims % 2 or dims > dim:
                raise FormatError(f"{where}: rot.dims {dims} must be even and at most dim {dim}")
            position = PositionSpec(head_dim=dim, theta=rr.number("base", positive=True), max_positions=MAX_POSITIONS,
                                    pairing="half", rotary_dim=dims)
        roles = {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "q_norm": p + "q.norm",
                 "k_norm": p + "k.norm", "talk": p + "talk", "head_bias": p + "pb"}
        heads, kv_heads = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
        if heads % kv_heads:
            raise FormatError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
        return SigmoidAttentionSpec(
            hidden=self.width, n_heads=heads, n_kv_heads=kv_heads, head_dim=dim, value_dim=m.integer("vdim", minimum=1),
            scale=m.number("scale"), window=_window(m, where), qk_norm=True, eps=self.eps, talk=True, head_bias=True,
            position=position, names=names(**roles), out_scale=out_scale)

    def _recurrence(self, p: str, raw: dict, where: str, out_scale: float):
        m = ConfigReader(raw, where)
        width, blocks = m.integer("width", minimum=1), m.integer("blocks", minimum=1)
        if width % blocks:
            raise FormatError(f"{where}: width {width} cannot be cut into {blocks} equal blocks")
        roles = {"y": p + "y", "y_bias": p + "y.b", "x": p + "x", "x_bias": p + "x.b", "conv": p + "conv",
                 "conv_bias": p + "conv.b", "ra": p + "ra", "ra_bias": p + "ra.b", "ri": p + "ri",
                 "ri_bias": p + "ri.b", "lam": p + "lam", "o": p + "o"}
        return GatedRecurrenceSpec(hidden=self.width, width=width, blocks=blocks, conv_taps=m.integer("conv", minimum=1),
                                   decay=RECURRENCE_DECAY, names=names(**roles), out_scale=out_scale)

    def _mixer(self, i: int, kind, raw: dict, where: str):
        p = f"l{i}.mix."
        if kind == "latent_attention":
            return self._latent(p, raw, where)
        if kind == "parallel":
            m = ConfigReader(raw, where)
            return SideBySideSpec(
                left=self._sigmoid(p + "left.", m.mapping("left"), f"{where}.left", m.number("left_scale", 1.0)),
                right=self._recurrence(p + "right.", m.mapping("right"), f"{where}.right", m.number("right_scale", 1.0)))
        raise Unsupported(f"{where}: a layer of type '{kind}' (built: 'latent_attention', 'parallel')")

    def _norm(self, name: str):
        return TanhNormSpec(self.width, name, name + ".b", name + ".alpha")

    def model_spec(self) -> ModelSpec:
        blocks = []
        for i, text in enumerate(self.layers):
            layer = json.loads(text)
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, dict):
                raise FormatError(f"{where} is not an object")
            if not isinstance(layer.get("mixer"), dict):
                raise FormatError(f"{where}: 'mixer' must be an object")
            mixer = self._mixer(i, layer.get("type"), layer["mixer"], f"{where}.mixer")
            ffn = None
            mlp = layer.get("mlp")
            if mlp is not None:
                f = ConfigReader(mlp, f"{where}.mlp")
                if f.string("kind", "dense") != "dense":
                    raise Unsupported(f"{where}.mlp: kind '{f.string('kind')}' (built: 'dense')")
                p = f"l{i}.mlp."
                ffn = GatedMlpSpec(hidden=self.width, intermediate=f.integer("ff", minimum=1), activation="silu",
                                   names=names(gate=p + "gate", up=p + "up", down=p + "down"))
            blocks.append(ParallelBlockSpec(norm=self._norm(f"l{i}.norm1"), mixer=mixer, feed_forward=ffn,
                                            ffn_norm=self._norm(f"l{i}.norm2") if ffn is not None else None))
        return ModelSpec(
            architecture=self.architecture, vocab=self.vocab, hidden=self.width, max_positions=MAX_POSITIONS,
            embedding="embed", blocks=tuple(blocks), schedule=tuple(ScheduleEntry(i) for i in range(len(blocks))),
            final_norm=self._norm("final.norm"), head=None, embedding_scale=self.embedding_scale)
