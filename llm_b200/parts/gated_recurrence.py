"""A recurrent block with a real-gated linear recurrent unit."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import StateRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import register_mixer, to_float32, to_run_dtype
from .projected import ProjectedMixer


class GatedRecurrenceMixer(ProjectedMixer):
    """Two branches of `width` channels from one product: y = gelu(W_y h + b_y) (tanh form) and
    u = conv(W_x h + b_x), a causal convolution per channel with a bias. The channels are cut into
    `blocks` equal parts; in part b, r = sigmoid(A_b u_b + a_b) and i = sigmoid(I_b u_b + i_b) with
    square matrices A_b, I_b. Per channel a = exp(-decay r softplus(lam)) and
    S_t = a S_(t-1) + sqrt(1 - a^2) i u, S = 0 before a sequence's first token (which is not
    treated specially); the block's result is W_o (S * y) (De et al., "Griffin").

    Per sequence the cache holds one float32 state [taps, width]: the convolution's last taps - 1
    inputs (rows 0 .. taps - 2, oldest first) and S (the last row). The gates, the decay, the
    recurrence and S are 32-bit in every run; the projections and the convolution's inputs are in
    the run's dtype. Launches: convolution + gates (a and the driving term of every token), then
    the scan over each sequence's tokens with y's activation, the product S * y and the update of
    the state (ops.gated_recurrence)."""
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "gated_recurrence")

    def __init__(self, spec):
        s = spec
        if s.width < 1 or s.blocks < 1 or s.width % s.blocks or s.conv_taps < 1:
            raise FormatError(f"a gated recurrence of {s.width} channels cannot be cut into {s.blocks} equal parts "
                              f"(or has no taps: {s.conv_taps})")
        self.spec = spec
        self.conv = self.conv_bias = self.gate_a = self.gate_a_bias = self.gate_i = self.gate_i_bias = self.rate = None

    @property
    def in_width(self):
        return 2 * self.spec.width

    @property
    def out_width(self):
        return self.spec.width

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        part = s.width // s.blocks
        return {t["y"]: ParamSpec((s.width, s.hidden)), t["y_bias"]: ParamSpec((s.width,), "bias"),
                t["x"]: ParamSpec((s.width, s.hidden)), t["x_bias"]: ParamSpec((s.width,), "bias"),
                t["conv"]: ParamSpec((s.width, s.conv_taps), "taps"), t["conv_bias"]: ParamSpec((s.width,), "bias"),
                t["ra"]: ParamSpec((s.blocks, part, part)), t["ra_bias"]: ParamSpec((s.blocks, part), "bias"),
                t["ri"]: ParamSpec((s.blocks, part, part)), t["ri_bias"]: ParamSpec((s.blocks, part), "bias"),
                t["lam"]: ParamSpec((s.width,), "vector"), t["o"]: ParamSpec((s.hidden, s.width))}

    def bind(self, tensors, dtype, device):
        s, t = self.spec, self.spec.tensor
        self.w_in = torch.cat([to_run_dtype(tensors[t[r]], dtype, device) for r in ("y", "x")]).contiguous()
        self.b_in = torch.cat([to_float32(tensors[t[r]], device) for r in ("y_bias", "x_bias")]).contiguous()
        self.w_out = to_run_dtype(tensors[t["o"]], dtype, device)
        self.conv = to_float32(tensors[t["conv"]], device)
        self.conv_bias = to_float32(tensors[t["conv_bias"]], device)
        # the gates are 32-bit in every run: their matrices are held so
        self.gate_a, self.gate_i = to_float32(tensors[t["ra"]], device), to_float32(tensors[t["ri"]], device)
        self.gate_a_bias = to_float32(tensors[t["ra_bias"]], device).reshape(-1).contiguous()
        self.gate_i_bias = to_float32(tensors[t["ri_bias"]], device).reshape(-1).contiguous()
        # log a = rate * r with rate = -decay * softplus(lam), once, in 32-bit
        lam = to_float32(tensors[t["lam"]], device)
        self.rate = (torch.nn.functional.softplus(lam) * torch.tensor(-s.decay, dtype=torch.float32)).contiguous()

    def mix_weights(self):
        return [self.gate_a, self.gate_i]

    def state_request(self):
        return StateRequest((self.spec.conv_taps, self.spec.width), torch.float32)

    def mix_replay_key(self, step):
        return (bool(step.decode),)

    def mix_scratch(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        # phase 0: all kernels (the scan reads what the gates wrote)
        return [BufferRequest("decay_drive", (3, n_tokens, self.spec.width), torch.float32, 0, 0)]

    def mix(self, proj, ctx, entry, cache_entry, out, scratch):
        s = self.spec
        n = proj.shape[0]
        work = scratch("decay_drive", (3, n, s.width), torch.float32)
        if work is None:
            work = torch.empty((3, n, s.width), dtype=torch.float32, device=proj.device)
        ops.gated_recurrence(proj[:, :s.width], proj[:, s.width:], self.conv, self.conv_bias, self.gate_a,
                             self.gate_a_bias, self.gate_i, self.gate_i_bias, self.rate, ctx.cache.state_view(entry),
                             ctx.tok_seq, ctx.cu_seqlens, ctx.slot_ids, out, s.out_scale, work,
                             single_tokens=ctx.decode)


register_mixer("gated_recurrence", GatedRecurrenceMixer)
