"""Descriptions of a model as data.

A configuration class turns config.json into a `ModelSpec`: one `BlockSpec`
for every layer (its norms, its mixer, its feed-forward, each with all
sizes and constants), a schedule that says in which order layers run and
whose cache each reads, and the names of the tensors that every part
binds. Parts are built from these records through the registries in
`llm_b200.parts`; nothing here knows an architecture.

Any object with a `kind` attribute can stand as a spec: a part registered
under that kind receives it unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    weight: str                      # tensor name
    kind: str = "rmsnorm"
    unit_offset: bool = False        # the stored weight lies around zero: the gain is 1 + weight


@dataclass(frozen=True)
class PositionSpec:
    """Rotary encoding: angle = position * inv_freq[pair]."""
    head_dim: int
    theta: float
    max_positions: int
    scaling: Optional[tuple] = None  # sorted (key, value) pairs of rope_scaling, or None
    pairing: str = "half"            # 'half': (p, p + n/2); 'interleaved': (2p, 2p + 1)
    kind: str = "rope"
    rotary_dim: Optional[int] = None # n: how many leading elements of a head rotate (None: all)

    @property
    def scaling_dict(self):
        return dict(self.scaling) if self.scaling is not None else None


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    scale: float                     # multiplies q.k
    bias: bool
    window: int                      # 0: every earlier key; w > 0: the last w keys
    position: Optional[PositionSpec]
    names: tuple                     # sorted (role, tensor name): q, k, v, o (+ q_bias, ...)
    kind: str = "attention"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Differential attention: every query head has two maps, each a softmax attention of its own
    over the same values; a head's result is map 1 minus lambda times map 2, divided by its root
    mean square and multiplied by 1 - diff. lambda = e^<lq1, lk1> - e^<lq2, lk2> + diff."""
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int                    # query / key size of ONE map
    value_dim: int
    scale: float                     # multiplies q.k
    window: int                      # 0: every earlier key; w > 0: keys less than w positions back ...
    keep_first: int                  # ... and the sequence's first keep_first keys
    conv_taps: int                   # taps of the causal convolution behind q, k, v (0: none)
    diff: float                      # lambda's constant term; the result is scaled by 1 - diff
    eps: float                       # of the head's norm
    position: Optional[PositionSpec]
    names: tuple                     # sorted (role, tensor name): q, k, v, o, lq1, lk1, lq2, lk2 (+ q_conv, k_conv, v_conv)
    kind: str = "diff_attention"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class GatedMlpSpec:
    hidden: int
    intermediate: int
    activation: str                  # 'silu'
    names: tuple                     # sorted (role, tensor name): gate, up, down
    kind: str = "gated_mlp"

    @property
    def tensor(self):
        return dict(self.names)


@dataclass(frozen=True)
class BlockSpec:
    """x += mixer(mixer_norm(x)); x += feed_forward(ffn_norm(x))  ('pre_norm')."""
    mixer_norm: object
    mixer: object
    ffn_norm: object
    feed_forward: object
    kind: str = "pre_norm"


@dataclass(frozen=True)
class ParallelBlockSpec:
    """x += mixer(norm(x)) + feed_forward(norm(x)): one norm, both parts read its output.
    `feed_forward` may be None (a layer that only mixes)."""
    norm: object
    mixer: object
    feed_forward: object
    kind: str = "parallel"


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. `cache_of` names an earlier schedule entry whose
    keys and values this run reads instead of writing its own. With `add_embedding` the
    embedding output (the stream as it was before the first run) is added to the stream
    right before this run."""
    layer: int
    cache_of: Optional[int] = None
    add_embedding: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab: int
    hidden: int
    max_positions: int
    embedding: str                   # tensor name of the [vocab, hidden] table
    blocks: tuple                    # BlockSpec per layer
    schedule: tuple                  # ScheduleEntry, in running order
    final_norm: object
    head: Optional[str]              # tensor name of the [vocab, hidden] head; None: tied to the embedding
    stop_tokens: tuple = field(default_factory=tuple)
    embedding_scale: float = 1.0     # multiplies the embedded tokens
    logit_scale: float = 1.0         # multiplies the logits
    logit_softcap: float = 0.0       # c > 0: logits <- c * tanh(logits / c), after the scale


def names(**roles) -> tuple:
    return tuple(sorted(roles.items()))
