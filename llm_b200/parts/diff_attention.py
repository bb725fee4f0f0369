"""Differential grouped-query attention with a short convolution behind its projections."""
from __future__ import annotations

import torch

from .. import ops
from ..cache import KvRequest, StateRequest
from ..errors import FormatError
from ..weights.loader import ParamSpec
from .base import Mixer, build_position, register_mixer, to_float32, to_run_dtype


class DiffAttentionMixer(Mixer):
    """Every query head holds two maps. The q projection gives, for each of the H heads in turn, the
    query of map 1 and then the query of map 2 (dim elements each); the k projection the same for
    the G key/value heads; the v projection one value of vdim elements per key/value head. Then:

    * optionally a causal convolution over time on every channel of q, k and v: with n taps,
      y[t] = tap[0] u[t - (n - 1)] + ... + tap[n - 1] u[t], u = 0 at negative positions; the last
      n - 1 inputs of a sequence are its state;
    * rotation of the first `rotary_dim` elements of every map of q and k;
    * per map a softmax attention over the keys a position sees (causal; with a window, the keys
      less than `window` back and the first `keep_first` of the sequence), both maps over the same
      values: a1, a2;
    * o = a1 - lambda a2, lambda = e^<lq1, lk1> - e^<lq2, lk2> + diff; o is divided by the root of
      (its mean square + eps) over the head's values and multiplied by 1 - diff;
    * the output projection, added to the residual stream.

    One launch for the projection, one for convolution + rotation + cache write
    (ops.conv_rope_cache_write), one for the attention with the maps' difference and the head's
    norm in its epilogue (ops.diff_attention), one for the output projection. A key row of the
    cache holds both maps [2 * dim]; lambda is computed once at bind, in 32-bit."""
    graph_safe = True
    emits = True
    libraries = ("elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "short_conv", "diff_attention")

    def __init__(self, spec):
        s = spec
        if s.n_heads % s.n_kv_heads:
            raise FormatError(f"{s.n_heads} query heads are no multiple of {s.n_kv_heads} key/value heads")
        if s.window < 0 or s.keep_first < 0 or s.conv_taps < 0:
            raise FormatError("a window, the kept first tokens and the taps of a convolution cannot be negative")
        self.spec = spec
        self.position = build_position(spec.position)
        self.w_qkv = self.w_o = self.w_conv = self.w_conv_rows = None
        self.lam = 0.0

    @property
    def q_width(self):
        return self.spec.n_heads * 2 * self.spec.head_dim

    @property
    def k_width(self):
        return self.spec.n_kv_heads * 2 * self.spec.head_dim

    @property
    def v_width(self):
        return self.spec.n_kv_heads * self.spec.value_dim

    @property
    def channels(self):
        return self.q_width + self.k_width + self.v_width

    @property
    def out_width(self):
        return self.spec.n_heads * self.spec.value_dim

    def parameters(self):
        s, t = self.spec, self.spec.tensor
        out = {t["q"]: ParamSpec((self.q_width, s.hidden)),
               t["k"]: ParamSpec((self.k_width, s.hidden)),
               t["v"]: ParamSpec((self.v_width, s.hidden)),
               t["o"]: ParamSpec((s.hidden, self.out_width))}
        for role in ("lq1", "lk1", "lq2", "lk2"):
            out[t[role]] = ParamSpec((s.head_dim,), "vector")
        if s.conv_taps:
            out[t["q_conv"]] = ParamSpec((self.q_width, s.conv_taps), "taps")
            out[t["k_conv"]] = ParamSpec((self.k_width, s.conv_taps), "taps")
            out[t["v_conv"]] = ParamSpec((self.v_width, s.conv_taps), "taps")
        return out

    def bind(self, tensors, dtype, device):
        t, s = self.spec.tensor, self.spec
        self.w_qkv = torch.cat([to_run_dtype(tensors[t[r]], dtype, device) for r in ("q", "k", "v")])
        self.w_o = to_run_dtype(tensors[t["o"]], dtype, device)
        if s.conv_taps:
            self.w_conv = torch.cat([to_float32(tensors[t[r + "_conv"]], device) for r in ("q", "k", "v")]).contiguous()
            # bfloat16 runs: the taps once more as [taps, channels] in bfloat16 for the 16-byte kernel, where
            # that loses nothing (taps stored as bfloat16)
            rows = self.w_conv.t().contiguous().to(torch.bfloat16)
            self.w_conv_rows = rows if dtype == torch.bfloat16 and torch.equal(rows.float().t(), self.w_conv) else None
        lq1, lk1, lq2, lk2 = (tensors[t[r]].to(torch.float32).cpu() for r in ("lq1", "lk1", "lq2", "lk2"))
        first = torch.exp((lq1 * lk1).sum())               # 32-bit, as the layer's other gates
        second = torch.exp((lq2 * lk2).sum())
        self.lam = float(first - second + torch.tensor(s.diff, dtype=torch.float32))

    def fold_input_norm(self, gain):
        """bfloat16 runs: the gain goes into the columns of the q/k/v matrix (in 32-bit, rounded
        once), and the product's epilogue applies the norm's scale."""
        if self.w_qkv.dtype != torch.bfloat16 or self.spec.hidden % 8:
            return False
        self.w_qkv = (self.w_qkv.float() * gain.to(self.w_qkv.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def prepare(self, max_positions, device):
        if self.position is not None:
            self.position.prepare(max_positions, device)

    def scratch_requests(self, n_tokens, dtype):
        from ..engine.workspace import BufferRequest
        # phases: 0 projections, 1 convolution + rotation + cache write, 2 attention, 3 output projection
        return [BufferRequest("qkv", (n_tokens, self.channels), dtype, 0, 1),
                BufferRequest("queries", (n_tokens, self.q_width), dtype, 1, 2),
                BufferRequest("mixed", (n_tokens, self.out_width), dtype, 2, 3)]

    def kernel_shapes(self, dtype, token_counts):
        s, out = self.spec, []
        for n in token_counts:
            out.append((f"qkv product, {n} tokens", "linear",
                        dict(m=n, n=self.channels, k=s.hidden, in_dtype=dtype, out_dtype=dtype, lda=s.hidden, aligned=True)))
            out.append((f"output product, {n} tokens", "linear",
                        dict(m=n, n=s.hidden, k=self.out_width, in_dtype=dtype, out_dtype=torch.float32,
                             lda=self.out_width, aligned=True)))
        for decode in (True, False):
            out.append(("decode differential attention" if decode else "prefill differential attention",
                        "diff_attention",
                        dict(decode=decode, dtype=dtype, n_heads=s.n_heads, n_kv_heads=s.n_kv_heads,
                             head_dim=s.head_dim, value_dim=s.value_dim, window=s.window,
                             keep_first=s.keep_first, packed=True, aligned=True)))
        return out

    def kv_request(self):
        # every position stays: a window that keeps the sequence's first tokens cannot live in a ring
        s = self.spec
        return KvRequest(s.n_kv_heads, 2 * s.head_dim, 0, value_dim=s.value_dim)

    def state_request(self):
        if self.spec.conv_taps > 1:
            return StateRequest((self.spec.conv_taps - 1, self.channels), None)     # in the run's dtype
        return None

    def replay_key(self, step):
        return ops.diff_attention_replay_key(step, self.spec)

    def forward(self, h, ctx, entry, cache_entry, residual, emit=None):
        s = self.spec
        group, keys, values = ctx.cache.layer_view(cache_entry)
        table = ctx.block_tables[group]
        ring = ctx.cache.table_width(group)
        norm = h if isinstance(h, ops.FoldedNorm) else None
        if norm is not None:
            h = norm.rows
        n = h.shape[0]
        qkv = ops.linear(h, self.w_qkv, out=ctx.scratch("qkv", (n, self.channels), h.dtype), norm=norm)
        queries = ctx.scratch("queries", (n, self.q_width), h.dtype)
        if queries is None:
            queries = torch.empty((n, self.q_width), dtype=h.dtype, device=h.device)
        state = ctx.cache.state_view(entry) if s.conv_taps > 1 else None
        ops.conv_rope_cache_write(
            qkv, self.w_conv, state, ctx.tok_pos, ctx.tok_seq, ctx.cu_seqlens, ctx.seq_lens, ctx.slot_ids,
            self.position.table if self.position is not None else None, s.head_dim,
            self.position.interleaved if self.position is not None else False, queries, self.k_width,
            self.v_width, table, ring, keys, values, write_cache=(entry == cache_entry), single_tokens=ctx.decode,
            conv_w_rows=self.w_conv_rows)
        mixed = ops.diff_attention(
            queries, keys, values, table, ring, ctx.tok_pos, ctx.tok_seq, s.n_heads, s.n_kv_heads, s.head_dim,
            s.value_dim, s.scale, s.window, s.keep_first, self.lam, s.eps, 1.0 - s.diff, head_norm=True,
            out=ctx.scratch("mixed", (n, self.out_width), h.dtype), decode=ctx.decode, seq_lens=ctx.seq_lens,
            max_len=ctx.max_len, cu_seqlens=ctx.cu_seqlens, max_new=max(ctx.new_counts), seq_order=ctx.seq_order)
        ops.linear(mixed, self.w_o, residual=residual, emit=emit)


register_mixer("diff_attention", DiffAttentionMixer)
