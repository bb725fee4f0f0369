"""Grouped-query attention with sigmoid weights and mixed heads."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KvRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import build_position, register_mixer, to_float32, to_run_dtype
from .projected import ProjectedMixer


class SigmoidAttentionMixer(ProjectedMixer):
    """q, k, v as one product; optionally an RMS norm over the whole query projection and one over
    the whole key projection (all heads at once, gains of that size); rotation of the first
    `rotary_dim` elements of every head; then, for query i and every key j it sees,
    s_a = scale q_a . k_g(a), optionally mixed over the heads (s_a <- sum_b T[a, b] s_b), and
    o_a = sum_j sigmoid(s_a + bias_a) v_g(a),j: no softmax, no normalisation over the keys.

    Launches: norm + rotation + cache write (ops.norm_rope_cache_write), the attention
    (ops.sigmoid_attention)."""
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "projection_norm", "sigmoid_attention")

    def __init__(self, spec):
        s = spec
        if s.n_heads < 1 or s.n_kv_heads < 1 or s.n_heads % s.n_kv_heads:
            raise FormatError(f"{s.n_heads} query heads are no multiple of {s.n_kv_heads} key/value heads")
        if s.window < 0 or s.head_dim < 1 or s.value_dim < 1:
            raise FormatError("a sigmoid attention needs positive head sizes and a window that is not negative")
        self.spec = spec
        self.position = build_position(spec.position)
        self.q_gain = self.k_gain = self.talk = self.head_bias = None

    @property
    def q_width(self):
        return self.spec.n_heads * self.spec.head_dim

    @property
    def k_width(self):
        return self.spec.n_kv_heads * self.spec.head_dim

    @property
    def v_width(self):
        return self.spec.n_kv_heads * self.spec.value_dim

    @property
    def in_width(self):
        return self.q_width + self.k_width + self.v_width

    @property
    def out_width(self):
        return self.spec.n_heads * self.spec.value_dim

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        out = {t["q"]: ParamSpec((self.q_width, s.hidden)), t["k"]: ParamSpec((self.k_width, s.hidden)),
               t["v"]: ParamSpec((self.v_width, s.hidden)), t["o"]: ParamSpec((s.hidden, self.out_width))}
        if s.qk_norm:
            out[t["q_norm"]] = ParamSpec((self.q_width,), "gain")
            out[t["k_norm"]] = ParamSpec((self.k_width,), "gain")
        if s.talk:
            out[t["talk"]] = ParamSpec((s.n_heads, s.n_heads), "vector")
        if s.head_bias:
            out[t["head_bias"]] = ParamSpec((s.n_heads,), "vector")
        return out

    def bind(self, tensors, dtype, device):
        s, t = self.spec, self.spec.tensor
        self.w_in = torch.cat([to_run_dtype(tensors[t[r]], dtype, device) for r in ("q", "k", "v")]).contiguous()
        self.w_out = to_run_dtype(tensors[t["o"]], dtype, device)
        if s.qk_norm:
            self.q_gain = to_float32(tensors[t["q_norm"]], device)
            self.k_gain = to_float32(tensors[t["k_norm"]], device)
        self.talk = to_float32(tensors[t["talk"]], device) if s.talk else None
        self.head_bias = to_float32(tensors[t["head_bias"]], device) if s.head_bias else None

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def kv_request(self):
        s = self.spec
        return KvRequest(s.n_kv_heads, s.head_dim, 0, value_dim=s.value_dim)

    def mix_scratch(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        # phases: 0 norm + rotation + cache write, 1 attention
        return [BufferRequest("queries", (n_tokens, self.q_width), dtype, 0, 1)]

    def mix_replay_key(self, step):
        return ops.sigmoid_attention_replay_key(step, self.spec)

    def mix_shapes(self, dtype, token_counts):
        s = self.spec
        return [("decode sigmoid attention" if decode else "prefill sigmoid attention", "sigmoid_attention",
                 dict(decode=decode, dtype=dtype, n_heads=s.n_heads, n_kv_heads=s.n_kv_heads, head_dim=s.head_dim,
                      value_dim=s.value_dim, window=s.window, packed=True, aligned=True))
                for decode in (True, False)]

    def mix(self, proj, ctx, entry, cache_entry, out, scratch):
        s = self.spec
        group, keys, values = ctx.cache.layer_view(cache_entry)
        table, ring = ctx.block_tables[group], ctx.cache.table_width(group)
        n = proj.shape[0]
        queries = scratch("queries", (n, self.q_width), proj.dtype)
        if queries is None:
            queries = torch.empty((n, self.q_width), dtype=proj.dtype, device=proj.device)
        ops.norm_rope_cache_write(proj, self.q_width, self.k_width, self.v_width, self.q_gain, self.k_gain, s.eps,
                                  self.position.table if self.position is not None else None, s.head_dim,
                                  self.position.interleaved if self.position is not None else False,
                                  ctx.tok_pos, ctx.tok_seq, queries, table, ring, keys, values,
                                  write_cache=(entry == cache_entry))
        ops.sigmoid_attention(queries, keys, values, table, ring, ctx.tok_pos, ctx.tok_seq, s.n_heads, s.n_kv_heads,
                              s.head_dim, s.value_dim, s.scale, s.window, self.talk, self.head_bias, s.out_scale, out,
                              decode=ctx.decode, seq_lens=ctx.seq_lens, max_len=ctx.max_len, cu_seqlens=ctx.cu_seqlens,
                              max_new=max(ctx.new_counts), seq_order=ctx.seq_order)


register_mixer("sigmoid_attention", SigmoidAttentionMixer)
