"""Two mixers that read one input."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import Unsupported
from .base import Mixer, build_mixer, register_mixer
from .projected import ProjectedMixer


class SideBySideMixer(ProjectedMixer):
    """left(h) + right(h), each already times its own `out_scale`. Both sides are ProjectedMixers,
    so the pair is one: the rows of both first matrices are stacked (one product of h), each side
    mixes its own columns of the projection into its own columns of one buffer, and the columns
    of both output matrices are laid side by side (one product into the stream, which sums the
    two results in its 32-bit accumulator). At most one side may keep keys and values, and at
    most one a fixed-size state: a schedule entry owns one of each."""

    def __init__(self, spec):
        self.spec = spec
        self.left, self.right = build_mixer(spec.left), build_mixer(spec.right)
        for side in (self.left, self.right):
            if not isinstance(side, ProjectedMixer):
                raise Unsupported(f"a {type(side).__name__} cannot stand side by side with another mixer")
        if sum(m.kv_request() is not None for m in self.sides) > 1 or \
                sum(m.state_request() is not None for m in self.sides) > 1:
            raise Unsupported("two mixers side by side that both keep keys and values, or both a state")
        self.split_in = self.split_out = 0

    @property
    def sides(self):
        return (self.left, self.right)

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.sides)

    @property
    def libraries(self):
        return tuple(lib for m in self.sides for lib in m.libraries)

    @property
    def hidden(self):
        return self.left.hidden

    @property
    def in_width(self):
        return self.left.in_width + self.right.in_width

    @property
    def out_width(self):
        return self.left.out_width + self.right.out_width

    def parameters(self):
        return {**self.left.parameters(), **self.right.parameters()}

    def bind(self, tensors, dtype, device):
        for m in self.sides:
            m.bind(tensors, dtype, device)
        self.split_in, self.split_out = self.left.in_width, self.left.out_width
        self.w_in = torch.cat([self.left.w_in, self.right.w_in]).contiguous()
        if self.left.b_in is not None or self.right.b_in is not None:
            zeros = lambda m: torch.zeros(m.in_width, dtype=torch.float32, device=self.w_in.device)
            self.b_in = torch.cat([m.b_in if m.b_in is not None else zeros(m) for m in self.sides]).contiguous()
        self.w_out = torch.cat([self.left.w_out, self.right.w_out], dim=1).contiguous()
        for m in self.sides:                      # the stacked copies are the ones that run
            m.w_in = m.w_out = m.b_in = None

    def prepare(self, max_positions, device):
        for m in self.sides:
            m.prepare(max_positions, device)

    def kv_request(self):
        return next((r for r in (m.kv_request() for m in self.sides) if r is not None), None)

    def state_request(self):
        return next((r for r in (m.state_request() for m in self.sides) if r is not None), None)

    def mix_weights(self):
        return [w for m in self.sides for w in m.mix_weights()]

    def mix_scratch(self, n_tokens, dtype):
        left = [r.shifted(0, "left.") for r in self.left.mix_scratch(n_tokens, dtype)]
        start = 1 + max([r.last_use for r in left] + [-1])
        return left + [r.shifted(start, "right.") for r in self.right.mix_scratch(n_tokens, dtype)]

    def mix_replay_key(self, step):
        keys = [m.mix_replay_key(step) for m in self.sides]
        return None if any(k is None for k in keys) else tuple(keys)

    def mix_shapes(self, dtype, token_counts):
        return [shape for m in self.sides for shape in m.mix_shapes(dtype, token_counts)]

    def mix(self, proj, ctx, entry, cache_entry, out, scratch):
        def tagged(tag):
            return lambda name, shape=None, dtype=None: scratch(tag + name, shape, dtype)
        self.left.mix(proj[:, :self.split_in], ctx, entry, cache_entry, out[:, :self.split_out], tagged("left."))
        self.right.mix(proj[:, self.split_in:], ctx, entry, cache_entry, out[:, self.split_out:], tagged("right."))


register_mixer("side_by_side", SideBySideMixer)
