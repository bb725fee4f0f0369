"""Attention over one cached latent row per position."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KvRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import register_mixer, to_float32, to_run_dtype
from .projected import ProjectedMixer


class LatentAttentionMixer(ProjectedMixer):
    """c_q = norm(W_dq h), q = W_uq c_q; c = norm(W_dkv h) is the only thing cached;
    k_a = W_uk,a c and v_a = W_uv,a c for head a; softmax over the window with an optional sink
    term in the denominator; an optional gate sigmoid(W_g h)_a on head a; output projection.

    The keys and values are never formed. With c the cached row, q_a . k_a = (W_uk,a^T q_a) . c
    and sum_j p_j v_a,j = W_uv,a (sum_j p_j c_j), so at bind W_uk goes into the query matrix
    (A_a = W_uk,a^T W_uq,a: the query of head a lives in the latent space) and W_uv into the output
    matrix (B = W_o blockdiag(W_uv,a)), both products formed in 64-bit and rounded once. The
    attention is then one of `heads` query heads over ONE key head of `kv_rank` elements whose
    values are the keys themselves: a page of the cache is read once for all heads.

    Launches: the product [dq; dkv; gate], the two latent norms with the cache write
    (ops.norm_rope_cache_write), the query product, the attention with sink, gate and scale in its
    epilogue (ops.attention), the output product."""
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "projection_norm", "attention_generic",
                 "attention_decode", "attention_decode_window", "attention_prefill")

    def __init__(self, spec):
        s = spec
        if min(s.n_heads, s.head_dim, s.value_dim, s.q_rank, s.kv_rank) < 1 or s.window < 0:
            raise FormatError("a latent attention needs positive sizes and a window that is not negative")
        self.spec = spec
        self.w_q = self.q_gain = self.c_gain = self.sinks = None

    @property
    def in_width(self):
        s = self.spec
        return s.q_rank + s.kv_rank + (s.n_heads if s.gate else 0)

    @property
    def out_width(self):
        return self.spec.n_heads * self.spec.kv_rank

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        out = {t["dq"]: ParamSpec((s.q_rank, s.hidden)), t["dq_norm"]: ParamSpec((s.q_rank,), "gain"),
               t["uq"]: ParamSpec((s.n_heads * s.head_dim, s.q_rank)),
               t["dkv"]: ParamSpec((s.kv_rank, s.hidden)), t["dkv_norm"]: ParamSpec((s.kv_rank,), "gain"),
               t["uk"]: ParamSpec((s.n_heads * s.head_dim, s.kv_rank)),
               t["uv"]: ParamSpec((s.n_heads * s.value_dim, s.kv_rank)),
               t["o"]: ParamSpec((s.hidden, s.n_heads * s.value_dim))}
        if s.sink:
            out[t["sink"]] = ParamSpec((s.n_heads,), "vector")
        if s.gate:
            out[t["gate"]] = ParamSpec((s.n_heads, s.hidden))
        return out

    def bind(self, tensors, dtype, device):
        s, t = self.spec, self.spec.tensor
        rows = [tensors[t["dq"]], tensors[t["dkv"]]] + ([tensors[t["gate"]]] if s.gate else [])
        self.w_in = torch.cat([to_run_dtype(r, dtype, device) for r in rows]).contiguous()
        wide = dict(device=device, dtype=torch.float64)
        uq = tensors[t["uq"]].to(**wide).view(s.n_heads, s.head_dim, s.q_rank)
        uk = tensors[t["uk"]].to(**wide).view(s.n_heads, s.head_dim, s.kv_rank)
        uv = tensors[t["uv"]].to(**wide).view(s.n_heads, s.value_dim, s.kv_rank)
        o = tensors[t["o"]].to(**wide).view(s.hidden, s.n_heads, s.value_dim)
        self.w_q = torch.einsum("adr,adq->arq", uk, uq).reshape(s.n_heads * s.kv_rank, s.q_rank).to(dtype).contiguous()
        self.w_out = torch.einsum("xae,aer->xar", o, uv).reshape(s.hidden, s.n_heads * s.kv_rank).to(dtype).contiguous()
        self.q_gain = to_float32(tensors[t["dq_norm"]], device)
        self.c_gain = to_float32(tensors[t["dkv_norm"]], device)
        self.sinks = to_float32(tensors[t["sink"]], device) if s.sink else None

    def mix_weights(self):
        return [self.w_q]

    def kv_request(self):
        s = self.spec
        return KvRequest(1, s.kv_rank, 0, values_are_keys=True)

    def mix_scratch(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        s = self.spec
        # phases: 0 norms + cache write, 1 query product, 2 attention
        return [BufferRequest("latent_q", (n_tokens, s.q_rank), dtype, 0, 1),
                BufferRequest("queries", (n_tokens, self.out_width), dtype, 1, 2)]

    def mix_replay_key(self, step):
        return ops.attention_replay_key(step, self.spec.n_heads, 1, self.spec.window)

    def mix_shapes(self, dtype, token_counts):
        s, out = self.spec, []
        for n in token_counts:
            out.append((f"query product, {n} tokens", "linear",
                        dict(m=n, n=self.out_width, k=s.q_rank, in_dtype=dtype, out_dtype=dtype, lda=s.q_rank, aligned=True)))
        return out

    def mix(self, proj, ctx, entry, cache_entry, out, scratch):
        s = self.spec
        group, keys, values = ctx.cache.layer_view(cache_entry)
        table, ring = ctx.block_tables[group], ctx.cache.table_width(group)
        n = proj.shape[0]
        latent_q = scratch("latent_q", (n, s.q_rank), proj.dtype)
        if latent_q is None:
            latent_q = torch.empty((n, s.q_rank), dtype=proj.dtype, device=proj.device)
        ops.norm_rope_cache_write(proj, s.q_rank, s.kv_rank, 0, self.q_gain, self.c_gain, s.eps, None, s.kv_rank,
                                  False, ctx.tok_pos, ctx.tok_seq, latent_q, table, ring, keys, None,
                                  write_cache=(entry == cache_entry))
        queries = ops.linear(latent_q, self.w_q, out=scratch("queries", (n, self.out_width), proj.dtype))
        gate = proj[:, s.q_rank + s.kv_rank:] if s.gate else None
        ops.attention(queries, keys, values, table, ring, ctx.tok_pos, ctx.tok_seq, s.n_heads, 1, s.kv_rank,
                      s.scale, s.window, out=out, decode=ctx.decode, seq_lens=ctx.seq_lens, max_len=ctx.max_len,
                      cu_seqlens=ctx.cu_seqlens, max_new=max(ctx.new_counts), seq_order=ctx.seq_order,
                      sinks=self.sinks, gate=gate, out_scale=s.out_scale)


register_mixer("latent_attention", LatentAttentionMixer)
