"""Mefolorn on the GPU: every new kernel beside its plain statement (also with weights and inputs
made so that one key, a window's edge, a sink or a lost state shows), and the model through the
engine, the generation entry point and the trace-replay program against the plain whole-sequence
implementation, in 32-bit and in bfloat16."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_mefolorn as plain
import plain_ops
from tiny_mefolorn import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu

PAGE = 64
DEV = "cuda:0"


def _ops():
    from llm_b200 import ops
    return ops


class Batch:
    """Sequences of given lengths of which the last `new` tokens are this step's, on shuffled pages."""

    def __init__(self, lengths, new, seed=0, slack_pages=3):
        gen = torch.Generator().manual_seed(seed)
        self.lengths, self.new = list(lengths), list(new)
        per_seq = [(n + PAGE - 1) // PAGE for n in lengths]
        self.width = max(per_seq) + 1
        self.n_pages = sum(per_seq) + slack_pages
        order = torch.randperm(self.n_pages, generator=gen).tolist()
        table = torch.zeros((len(lengths), self.width), dtype=torch.int32)
        for b, count in enumerate(per_seq):
            for i in range(count):
                table[b, i] = order.pop()
        pos, seq, cu = [], [], [0]
        for b, (n, k) in enumerate(zip(lengths, new)):
            pos += list(range(n - k, n))
            seq += [b] * k
            cu.append(cu[-1] + k)
        as_int = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
        self.table = table.to(DEV)
        self.tok_pos, self.tok_seq, self.cu, self.seq_lens = as_int(pos), as_int(seq), as_int(cu), as_int(lengths)
        self.slots = as_int(list(range(len(lengths)))[::-1])          # slot ids differ from batch indices
        self.order = as_int(sorted(range(len(lengths)), key=lambda b: -lengths[b]))
        self.n_tokens = len(pos)

    def caches(self, heads, key_width, value_width, dtype, seed=1, std=1.0):
        gen = torch.Generator().manual_seed(seed)
        k = (torch.randn((self.n_pages, heads, PAGE, key_width), generator=gen) * std).to(dtype).to(DEV)
        v = torch.randn((self.n_pages, heads, PAGE, value_width), generator=gen).to(dtype).to(DEV) if value_width else None
        return k, v

    def place(self, b, position):
        return int(self.table[b, position // PAGE]), position % PAGE

    def extra(self, decode=None):
        decode = all(k == 1 for k in self.new) if decode is None else decode
        return dict(decode=decode, seq_lens=self.seq_lens, max_len=max(self.lengths), cu_seqlens=self.cu,
                    max_new=max(self.new), seq_order=self.order)


def _close(got, want, dtype, what=""):
    got, want = got.float(), want.float()
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=3e-5, rtol=3e-5), (what, float((got - want).abs().max()))
    else:
        scale = float(want.abs().max()) + 1e-6
        assert float((got - want).abs().max()) <= 0.03 * scale, (what, float((got - want).abs().max()), scale)
        assert float((got - want).abs().mean()) <= 0.004 * scale, what


BATCHES = [([70, 5, 130, 64], [70, 2, 66, 1]), ([9, 200, 65, 129], [1, 1, 1, 1]), ([3], [3]), ([300, 64, 1], [172, 64, 1])]


# ----------------------------------------------------------------------------- the tanh norm

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 97, 128, 1024, 4100])
def test_tanh_norm(dtype, width):
    ops = _ops()
    gen = torch.Generator().manual_seed(width)
    x = (3.0 * torch.randn((9, width), generator=gen)).to(DEV)
    g1, b1, g2, b2 = (torch.randn(width, generator=gen).to(DEV) for _ in range(4))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    _close(ops.tanh_norm(x, 0.37, g1, b1, dtype), plain_ops.tanh_norm(x, 0.37, g1, b1, dtype), dtype)
    _close(ops.tanh_norm(x, 1.7, g1, b1, dtype, rows=rows), plain_ops.tanh_norm(x, 1.7, g1, b1, dtype, rows=rows), dtype)
    second = torch.zeros((9, width), dtype=dtype, device=DEV)
    first = ops.tanh_norm(x, 0.37, g1, b1, dtype, second=(0.9, g2, b2, second))
    _close(first, plain_ops.tanh_norm(x, 0.37, g1, b1, dtype), dtype)
    _close(second, plain_ops.tanh_norm(x, 0.9, g2, b2, dtype), dtype)


# ----------------------------------------------------------------------------- norm + rotation + cache write

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # query heads, key heads, head size, value heads, value size, rotated, norms, interleaved, columns behind
    (4, 2, 6, 2, 10, 4, True, False, 0), (3, 3, 10, 3, 7, 10, True, False, 5), (2, 1, 16, 1, 24, 0, True, False, 48),
    (4, 2, 64, 2, 32, 32, True, False, 192), (2, 2, 8, 2, 8, 8, False, True, 0), (1, 1, 12, 0, 0, 0, True, False, 3),
    (1, 1, 9, 0, 0, 0, False, False, 0), (8, 2, 128, 2, 128, 64, True, False, 0)])
def test_norm_rope_cache_write(dtype, case):
    ops = _ops()
    heads, groups, dim, v_heads, vdim, n_rot, norms, interleaved, behind = case
    qw, kw, vw = heads * dim, groups * dim, v_heads * vdim
    gen = torch.Generator().manual_seed(5)
    for lengths, new in BATCHES:
        batch = Batch(lengths, new, seed=len(lengths))
        wide = torch.randn((batch.n_tokens, qw + kw + vw + behind), generator=gen).to(dtype).to(DEV)
        q_gain = (1.0 + 0.3 * torch.randn(qw, generator=gen)).to(DEV) if norms else None
        k_gain = (1.0 + 0.3 * torch.randn(kw, generator=gen)).to(DEV) if norms else None
        table = None
        if n_rot:
            angle = torch.arange(400, dtype=torch.float64)[:, None] * torch.rand(n_rot // 2, generator=gen, dtype=torch.float64)
            table = torch.cat([angle.cos(), angle.sin()], dim=1).float().to(DEV)
        results = []
        for fn in (ops.norm_rope_cache_write, plain_ops.norm_rope_cache_write):
            k_cache, v_cache = batch.caches(groups, dim, vdim, dtype, seed=5)
            if v_heads and v_heads != groups:
                v_cache = v_cache[:, :v_heads].contiguous()
            q_wide = torch.zeros((batch.n_tokens, qw + 8), dtype=dtype, device=DEV)
            fn(wide, qw, kw, vw, q_gain, k_gain, 1e-3, table, dim, interleaved, batch.tok_pos, batch.tok_seq,
               q_wide[:, :qw], batch.table, batch.width, k_cache, v_cache)
            results.append((q_wide, k_cache, v_cache if vw else k_cache))
        torch.cuda.synchronize()
        for got, want, what in zip(results[0], results[1], ("queries", "keys", "values")):
            _close(got, want, dtype, (case, lengths, what))
        assert float(results[0][0][:, qw:].abs().max()) == 0.0           # nothing written beside the queries


# ----------------------------------------------------------------------------- softmax attention with sink and gate

def _attention(fn, batch, heads, groups, dim, dtype, window, sinks, gated, shared, out_scale=1.0, seed=2, q=None, caches=None):
    gen = torch.Generator().manual_seed(seed)
    if q is None:
        q = torch.randn((batch.n_tokens, heads * dim), generator=gen).to(dtype).to(DEV)
    k_cache, v_cache = caches if caches is not None else batch.caches(groups, dim, dim, dtype, seed=seed + 1)
    if shared:
        v_cache = k_cache
    gate_wide = torch.randn((batch.n_tokens, heads + 3), generator=gen).to(dtype).to(DEV)
    sink = torch.randn(heads, generator=gen).to(DEV) * 2 if sinks else None
    out_wide = torch.zeros((batch.n_tokens, heads * dim + 16), dtype=dtype, device=DEV)
    fn(q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, groups, dim, dim ** -0.5,
       window, out=out_wide[:, 8:8 + heads * dim], sinks=sink, gate=gate_wide[:, 2:2 + heads] if gated else None,
       out_scale=out_scale, **batch.extra())
    return out_wide


class only_generic:
    """Inside: the tensor-core attention kernels are switched off, so the generic ones run in bfloat16 too."""
    NAMES = ("attention_prefill", "attention_decode", "sigmoid_attention_tiles", "sigmoid_attention_decode")

    def __init__(self, on=True):
        self.on = on

    def __enter__(self):
        from llm_b200.ops import tactics
        if self.on:
            for name in self.NAMES:
                tactics.disable(name)

    def __exit__(self, *error):
        from llm_b200.ops import tactics
        if self.on:
            for name in self.NAMES:
                tactics.enable(name)


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # heads, kv heads, head size, window, sink, gate, values are keys
    (4, 1, 64, 70, True, True, True), (3, 1, 9, 5, True, True, True), (8, 1, 32, 130, True, False, True),
    (2, 1, 34, 21, False, True, True), (4, 2, 16, 0, True, True, False), (2, 1, 320, 40, True, True, True),
    (16, 1, 128, 64, True, True, True), (4, 1, 96, 1, True, True, True), (4, 2, 64, 0, False, False, False),
    (2, 1, 128, 300, True, True, True), (6, 3, 32, 63, False, True, False), (32, 1, 128, 1000, True, True, True),
    (20, 2, 64, 0, True, False, False)])
def test_attention_with_sink_gate_and_shared_values(dtype, case, generic):
    ops = _ops()
    heads, groups, dim, window, sinks, gated, shared = case
    if generic and dtype == torch.float32:
        pytest.skip("the 32-bit path is the generic kernel already")
    for lengths, new in BATCHES + [([700, 64, 129], [700, 3, 129]), ([1500, 1, 64, 65, 700], [1] * 5), ([2200], [1])]:
        batch = Batch(lengths, new, seed=3 + len(lengths))
        with only_generic(generic):
            got = _attention(ops.attention, batch, heads, groups, dim, dtype, window, sinks, gated, shared, 0.8)
        want = _attention(plain_ops.attention, batch, heads, groups, dim, dtype, window, sinks, gated, shared, 0.8)
        torch.cuda.synchronize()
        _close(got, want, dtype, (case, lengths))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, "generic"])
@pytest.mark.parametrize("decode", [False, True])
def test_attention_planted_keys_sink_and_window_edges(dtype, decode):
    generic = dtype == "generic"
    dtype = torch.bfloat16 if generic else dtype
    with only_generic(generic):
        _attention_planted(dtype, decode)


def _attention_planted(dtype, decode):
    """One key is made to stand out: the result is that key's row exactly when the key is inside the window,
    also far back, at page borders and at both edges; a sink that stands out takes all the weight."""
    ops = _ops()
    heads, dim, window, length = 2, 64, 100, 331
    batch = Batch([length, 40], [1, 1] if decode else [length, 40], seed=11)
    last = 0 if decode else length - 1                      # row of the query at position length - 1
    gen = torch.Generator().manual_seed(4)
    for planted in (length - 1, length - window, length - window - 1, 256, 255, 0, length - 2):
        k_cache, _ = batch.caches(1, dim, 0, dtype, seed=6, std=0.1)
        page, row = batch.place(0, planted)
        k_cache[page, 0, row] = 0.0
        k_cache[page, 0, row, :4] = torch.tensor([3.0, -2.0, 1.0, 2.0])
        q = (0.1 * torch.randn((batch.n_tokens, heads * dim), generator=gen)).to(dtype).to(DEV)
        q[last] = 0.0
        q[last, :4] = torch.tensor([3.0, -2.0, 1.0, 2.0]) * 8.0          # head 0 asks for the planted key
        sink = torch.tensor([-3.0, 0.5], device=DEV)
        args = dict(heads=heads, groups=1, dim=dim, dtype=dtype, window=window, sinks=False, gated=False, shared=True,
                    q=q, caches=(k_cache, None))
        got = _attention(ops.attention, batch, **args)[last, 8:8 + dim].float()
        seen = length - 1 - planted < window
        if seen:
            assert abs(float(got[0]) - 3.0) < 0.05 and abs(float(got[1]) + 2.0) < 0.05, (planted, got[:4])
        else:
            assert float(got[:4].abs().max()) < 0.5, (planted, got[:4])
        _close(_attention(ops.attention, batch, **args), _attention(plain_ops.attention, batch, **args), dtype, planted)
    # a sink far above every score: nothing of the values is left; far below: as without
    k_cache, _ = batch.caches(1, dim, 0, dtype, seed=6)
    q = torch.randn((batch.n_tokens, heads * dim), generator=gen).to(dtype).to(DEV)
    common = (q, k_cache, k_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, 1, dim, 0.1, window)
    high = ops.attention(*common, sinks=torch.tensor([60.0, 60.0], device=DEV), **batch.extra())
    low = ops.attention(*common, sinks=torch.tensor([-60.0, -60.0], device=DEV), **batch.extra())
    none = ops.attention(*common, out_scale=1.0000001, **batch.extra())
    assert float(high.float().abs().max()) < 1e-6
    _close(low, none, dtype)


# ----------------------------------------------------------------------------- sigmoid attention with mixed heads

def _sigmoid(fn, batch, heads, groups, dim, vdim, dtype, window, talk, bias, seed=2, q=None, caches=None, talk_matrix=None,
             bias_vector=None):
    gen = torch.Generator().manual_seed(seed)
    if q is None:
        q = torch.randn((batch.n_tokens, heads * dim), generator=gen).to(dtype).to(DEV)
    k_cache, v_cache = caches if caches is not None else batch.caches(groups, dim, vdim, dtype, seed=seed + 1)
    if talk_matrix is None and talk:
        talk_matrix = (torch.eye(heads) + 0.5 * torch.randn((heads, heads), generator=gen)).to(DEV)
    if bias_vector is None and bias:
        bias_vector = torch.randn(heads, generator=gen).to(DEV) - 2.0
    out_wide = torch.zeros((batch.n_tokens, heads * vdim + 16), dtype=dtype, device=DEV)
    fn(q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, groups, dim, vdim, dim ** -0.5,
       window, talk_matrix, bias_vector, 0.6, out_wide[:, 8:8 + heads * vdim], **batch.extra())
    return out_wide


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # heads, kv heads, head size, value size, window, mixed, bias
    (4, 2, 6, 10, 9, True, True), (2, 2, 8, 5, 33, True, True), (4, 2, 64, 32, 40, True, True),
    (4, 1, 32, 64, 100, True, True), (2, 1, 16, 24, 0, True, True), (3, 1, 20, 20, 7, False, True),
    (4, 4, 64, 64, 64, True, False), (8, 2, 128, 128, 200, True, True), (16, 4, 96, 96, 65, True, True),
    (32, 8, 64, 64, 100, True, True), (32, 4, 32, 32, 0, False, True), (24, 8, 64, 128, 70, True, True)])
@pytest.mark.parametrize("generic", [False, True])
def test_sigmoid_attention(dtype, case, generic):
    ops = _ops()
    heads, groups, dim, vdim, window, talk, bias = case
    if generic and dtype == torch.float32:
        pytest.skip("the 32-bit path is the generic kernel already")
    for lengths, new in BATCHES + [([700, 64, 129], [700, 3, 129]), ([1500, 1, 64, 65, 700], [1] * 5), ([2200], [1])]:
        batch = Batch(lengths, new, seed=7 + len(lengths))
        with only_generic(generic):
            got = _sigmoid(ops.sigmoid_attention, batch, heads, groups, dim, vdim, dtype, window, talk, bias)
        want = _sigmoid(plain_ops.sigmoid_attention, batch, heads, groups, dim, vdim, dtype, window, talk, bias)
        torch.cuda.synchronize()
        _close(got, want, dtype, (case, lengths))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, "generic"])
@pytest.mark.parametrize("decode", [False, True])
def test_sigmoid_attention_planted_keys_and_mixing(dtype, decode):
    generic = dtype == "generic"
    dtype = torch.bfloat16 if generic else dtype
    with only_generic(generic):
        _sigmoid_planted(dtype, decode)


def _sigmoid_planted(dtype, decode):
    """With a bias far below zero no key has weight, except one whose score is made large: its value
    arrives exactly when it is inside the window. The key is seen by head 1 only; head 0 gets it
    through the mixing matrix alone."""
    ops = _ops()
    heads, groups, dim, vdim, window, length = 2, 2, 32, 16, 70, 267
    batch = Batch([length, 40], [1, 1] if decode else [length, 40], seed=12)
    last = 0 if decode else length - 1
    gen = torch.Generator().manual_seed(5)
    mix = torch.tensor([[1.0, 1.0], [0.0, 1.0]], device=DEV)
    for planted in (length - 1, length - window, length - window - 1, 192, 191, 0):
        k_cache, v_cache = batch.caches(groups, dim, vdim, dtype, seed=6, std=0.1)
        page, row = batch.place(0, planted)
        k_cache[page, 1, row] = 0.0
        k_cache[page, 1, row, :2] = torch.tensor([4.0, -4.0])
        v_cache[page, :, row] = 0.0
        v_cache[page, 0, row, 3] = 5.0                       # head 0 reads key/value head 0, head 1 reads 1
        v_cache[page, 1, row, 3] = 7.0
        q = (0.1 * torch.randn((batch.n_tokens, heads * dim), generator=gen)).to(dtype).to(DEV)
        q[last] = 0.0
        q[last, dim:dim + 2] = torch.tensor([4.0, -4.0]) * 8.0            # only head 1 asks
        args = dict(heads=heads, groups=groups, dim=dim, vdim=vdim, dtype=dtype, window=window, talk=True, bias=True,
                    q=q, caches=(k_cache, v_cache), bias_vector=torch.tensor([-20.0, -20.0], device=DEV))
        seen = length - 1 - planted < window
        for matrix, head0 in ((mix, 5.0 * 0.6 if seen else 0.0), (torch.eye(2, device=DEV), 0.0)):
            got = _sigmoid(ops.sigmoid_attention, batch, talk_matrix=matrix, **args)[last, 8:].float()
            assert abs(float(got[3]) - head0) < 0.05, (planted, "head 0", float(got[3]))
            assert abs(float(got[vdim + 3]) - (7.0 * 0.6 if seen else 0.0)) < 0.05, (planted, "head 1", float(got[vdim + 3]))
        _close(_sigmoid(ops.sigmoid_attention, batch, talk_matrix=mix, **args),
               _sigmoid(plain_ops.sigmoid_attention, batch, talk_matrix=mix, **args), dtype, planted)


# ----------------------------------------------------------------------------- gated recurrence

def _recurrence_inputs(channels, blocks, taps, n_tokens, n_slots, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    part = channels // blocks
    wide = torch.randn((n_tokens, 2 * channels + 5), generator=gen).to(dtype).to(DEV)
    params = dict(conv_w=torch.randn((channels, taps), generator=gen) / taps ** 0.5, conv_b=0.2 * torch.randn(channels, generator=gen),
                  gate_a=torch.randn((blocks, part, part), generator=gen) / part ** 0.5,
                  gate_a_bias=torch.randn(channels, generator=gen), gate_i=torch.randn((blocks, part, part), generator=gen) / part ** 0.5,
                  gate_i_bias=torch.randn(channels, generator=gen),
                  rate=-8.0 * torch.nn.functional.softplus(torch.randn(channels, generator=gen) - 2.0))
    state = torch.randn((n_slots, taps, channels), generator=gen).to(DEV)
    return wide, {k: v.to(DEV).contiguous() for k, v in params.items()}, state


def _recurrence(fn, wide, params, state, batch, channels, dtype):
    out_wide = torch.zeros((batch.n_tokens, channels + 9), dtype=dtype, device=DEV)
    work = torch.empty((3, batch.n_tokens, channels), device=DEV)
    p = params
    fn(wide[:, 2:2 + channels], wide[:, 2 + channels:2 + 2 * channels], p["conv_w"], p["conv_b"], p["gate_a"], p["gate_a_bias"],
       p["gate_i"], p["gate_i_bias"], p["rate"], state, batch.tok_seq, batch.cu, batch.slots, out_wide[:, 4:4 + channels], 0.9, work,
       single_tokens=all(k == 1 for k in batch.new))
    return out_wide


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [(24, 3, 3), (14, 1, 1), (96, 3, 4), (128, 2, 2), (160, 2, 4), (512, 4, 4), (70, 1, 8), (33, 11, 2)])
def test_gated_recurrence(dtype, case):
    ops = _ops()
    channels, blocks, taps = case
    # (steps of more than 256 tokens scan in chunks: sequences that begin and end inside and across chunks)
    for lengths, new in BATCHES + [([700, 64, 129, 5, 2], [700, 3, 129, 5, 1]), ([60, 900, 3, 131], [60, 320, 3, 131])]:
        batch = Batch(lengths, new, seed=1)
        wide, params, state = _recurrence_inputs(channels, blocks, taps, batch.n_tokens, len(lengths) + 2, dtype, seed=channels)
        states = [state.clone(), state.clone()]
        got = _recurrence(ops.gated_recurrence, wide, params, states[0], batch, channels, dtype)
        want = _recurrence(plain_ops.gated_recurrence, wide, params, states[1], batch, channels, dtype)
        torch.cuda.synchronize()
        _close(got, want, dtype, (case, lengths, "out"))
        _close(states[0], states[1], torch.float32, (case, lengths, "state"))


def test_gated_recurrence_carries_its_state_across_any_cut():
    """A sequence in one step, and the same cut at every place into two steps (the second also token by
    token): the same results to the last bit in 32-bit, and the state that the cuts leave is the same."""
    ops = _ops()
    channels, blocks, taps, n = 48, 2, 4, 21
    whole = Batch([n], [n])
    wide, params, state = _recurrence_inputs(channels, blocks, taps, n, 3, torch.float32, seed=9)
    state.zero_()
    first_state = state.clone()
    want = _recurrence(ops.gated_recurrence, wide, params, first_state, whole, channels, torch.float32)
    for cut in range(1, n):
        held = state.clone()
        head = _recurrence(ops.gated_recurrence, wide[:cut], params, held, Batch([cut], [cut]), channels, torch.float32)
        if cut % 2:
            tail = _recurrence(ops.gated_recurrence, wide[cut:], params, held, Batch([n], [n - cut]), channels, torch.float32)
        else:
            tail = torch.cat([_recurrence(ops.gated_recurrence, wide[t:t + 1], params, held, Batch([t + 1], [1]), channels,
                                          torch.float32) for t in range(cut, n)])
        assert torch.equal(torch.cat([head, tail]), want), cut
        assert torch.equal(held, first_state), cut
    # a long decay: a state that was lost (zeroed) shows hundreds of tokens later
    params["rate"].fill_(-1e-4)
    long = Batch([400], [400])
    wide, _, _ = _recurrence_inputs(channels, blocks, taps, 400, 3, torch.float32, seed=10)
    kept, lost = state.clone(), state.clone()
    kept[0, taps - 1] = 50.0
    a = _recurrence(ops.gated_recurrence, wide, params, kept, long, channels, torch.float32)
    b = _recurrence(ops.gated_recurrence, wide, params, lost, long, channels, torch.float32)
    assert float((a[399] - b[399]).abs().max()) > 1.0


# ----------------------------------------------------------------------------- the model through the engine

def _setup(tmp_path, which, dtype, change=None, weights_change=None, **engine_options):
    from llm_b200.engine import Engine, load_model
    folder = make_folder(tmp_path, which, torch.bfloat16, change, weights_change)
    config, weights = plain.read_model_folder(folder)
    engine = Engine(load_model(folder, dtype, DEV), **{"max_tokens": 4096, **engine_options})
    return config, weights, engine


def _check_logits(got, want, dtype, what=""):
    got, want = got.float().cpu(), want.float()
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=3e-4, rtol=1e-4), (what, float((got - want).abs().max()))
    else:
        span = float(want.max() - want.min())
        assert float((got - want).abs().max()) <= 0.05 * span, (what, float((got - want).abs().max()), span)
        assert float((got - want).abs().mean()) <= 0.01 * span, what


def test_every_layer_agrees_with_plain(tmp_path):
    """The residual stream after each layer in 32-bit (a model of the first k layers, for every k)."""
    from llm_b200.engine import Entry
    for which in sorted(CONFIGS):
        depth = len(CONFIGS[which][0]["layers"])
        for k in range(1, depth + 1):
            def cut(config, k=k):
                config["layers"] = config["layers"][:k]
            def plain_final(weights):
                weights["final.norm"].fill_(1.0)
                weights["final.norm.b"].fill_(0.0)
                weights["final.norm.alpha"].fill_(1e-3)                    # tanh(a x) / a ~ x: the head reads the stream
            config, weights, engine = _setup(tmp_path / f"{which}{k}", which, torch.float32, cut, plain_final)
            tokens = random_tokens(90, config["vocab"], k)
            streams = []
            want = plain.forward(config, weights, tokens, streams)
            (slot,) = engine.acquire()
            got = engine.step([Entry(slot, tokens, list(range(90)))])
            _check_logits(got, want, torch.float32, (which, k))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["P", "Q", "R"])
def test_whole_decode_pieces_and_batches_agree_with_plain(tmp_path, which, dtype):
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, which, dtype, step_tokens=48)
    lengths = [150, 1, 67, 20]
    seqs = [random_tokens(n, config["vocab"], 30 + n) for n in lengths]
    expected = [plain.forward(config, weights, s) for s in seqs]
    for again in range(2):                                       # the second time reuses slots, pages and states
        slots = engine.acquire(len(seqs))
        heads = [max(1, n - 9 - 2 * i) for i, n in enumerate(lengths)]          # unequal prompts, cut into passes of 48
        logits = engine.step([Entry(s, q[:h], list(range(h))) for s, q, h in zip(slots, seqs, heads)])
        row = 0
        for b, h in enumerate(heads):
            _check_logits(logits[row:row + h], expected[b][:h], dtype, ("prompt", b))
            row += h
        live = [b for b in range(len(seqs)) if heads[b] < lengths[b]]
        engine.release([slots[b] for b in range(len(seqs)) if b not in live])
        done = 0
        while live:                                              # decoding together; shorter sequences end earlier
            logits = engine.step([Entry(slots[b], [seqs[b][heads[b] + done]], [0]) for b in live])
            for r, b in enumerate(live):
                _check_logits(logits[r], expected[b][heads[b] + done], dtype, ("decode", b, done))
            done += 1
            ended = [b for b in live if heads[b] + done == lengths[b]]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
        engine.cache.check()
        assert engine.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_passes_the_windows_and_page_edges(tmp_path, dtype):
    """One token a step from the first on, 300 steps: windows of 40, 70, 100 and 130 slide over decoded
    tokens, pages fill and follow each other, the recurrent state is carried 300 times, and steps are
    replayed from graphs."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", dtype)
    tokens = random_tokens(300, config["vocab"], 77)
    expected = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    for p, token in enumerate(tokens):
        logits = engine.step([Entry(slot, [token], [0])])
        _check_logits(logits[0], expected[p], dtype, p)
    assert engine.graph_replays > 200


@pytest.mark.parametrize("piece", [2, 5, 64])
def test_pieces_down_to_two_tokens(tmp_path, piece):
    from llm_b200.engine import Entry
    for which in ("P", "Q"):
        config, weights, engine = _setup(tmp_path, which, torch.float32)
        tokens = random_tokens(140, config["vocab"], 8)
        expected = plain.forward(config, weights, tokens)
        (slot,) = engine.acquire()
        for start in range(0, len(tokens), piece):
            part = tokens[start:start + piece]
            logits = engine.step([Entry(slot, part, list(range(len(part))))])
            _check_logits(logits, expected[start:start + len(part)], torch.float32, (which, start))


def test_batch_and_cut_change_nothing_in_32_bit(tmp_path):
    """A position's logits alone, among neighbours, and with its prompt cut: equal to the last bit in the
    32-bit path (every reduction's order depends only on the position; states are carried exactly)."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "P", torch.float32)
    seqs = [random_tokens(n, config["vocab"], 60 + n) for n in (50, 13, 31)]
    a, b, c, d = engine.acquire(4)
    alone = engine.step([Entry(a, seqs[0], [49, 20])]).clone()
    together = engine.step([Entry(b, seqs[1], [12]), Entry(c, seqs[0], [49, 20]), Entry(d, seqs[2], [])])
    assert torch.equal(alone, together[1:3])
    engine.release([a])
    (e,) = engine.acquire()
    engine.step([Entry(e, seqs[0][:17], [])])
    engine.step([Entry(e, seqs[0][17:21], [])])
    for t in range(21, 30):
        engine.step([Entry(e, [seqs[0][t]], [])])
    cut = engine.step([Entry(e, seqs[0][30:], [49 - 30])])
    assert torch.equal(alone[0], cut[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_passes_walked_from_their_record_agree_with_plain_passes(tmp_path, dtype):
    """The same shape of step five times on other slots, pages and states: the first pass runs through the parts,
    the second is recorded, the later ones are walked natively from the record; a mixed step likewise."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", dtype)
    firsts = []
    for again in range(5):
        seqs = [random_tokens(n, config["vocab"], 100 * again + n) for n in (90, 33)]
        slots = engine.acquire(2)
        logits = engine.step([Entry(slots[0], seqs[0][:80], [0, 79]), Entry(slots[1], seqs[1][:30], [29])])
        want = [plain.forward(config, weights, s) for s in seqs]
        _check_logits(logits, torch.stack([want[0][0], want[0][79], want[1][29]]), dtype, ("prompt", again))
        mixed = engine.step([Entry(slots[0], seqs[0][80:], [9]), Entry(slots[1], [seqs[1][30]], [0])])
        _check_logits(mixed, torch.stack([want[0][89], want[1][30]]), dtype, ("mixed", again))
        engine.release(slots)
    assert engine.records_run >= 4


def test_a_far_key_a_sink_and_a_lost_state_show_in_the_logits(tmp_path):
    """Changes that a fault would make, made on purpose in the plain model: each must move the logits by far
    more than the library differs from the unchanged plain model."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", torch.float32)
    tokens = random_tokens(200, config["vocab"], 5)
    want = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, list(range(200)))]).cpu()
    error = float((got - want).abs().max())
    for change in ("window", "sink", "state", "mix"):
        other, w = json.loads(json.dumps(config)), dict(weights)
        if change == "window":
            other["layers"][0]["mixer"]["mask"]["size"] += 1
            other["layers"][1]["mixer"]["left"]["mask"]["size"] -= 1
        elif change == "sink":
            w["l0.mix.sink"] = weights["l0.mix.sink"] - 30.0
        elif change == "state":
            w["l1.mix.right.lam"] = weights["l1.mix.right.lam"] + 3.0
        else:
            w["l1.mix.left.talk"] = torch.eye(4)
        moved = float((plain.forward(other, w, tokens) - want).abs().max())
        assert moved > 50 * error, (change, moved, error)


def test_greedy_generation_through_the_entry_point(tmp_path):
    import llm_b200
    folder = make_folder(tmp_path, "Q", torch.bfloat16)
    config, weights = plain.read_model_folder(folder)
    prompts = [random_tokens(n, config["vocab"], 90 + n) for n in (5, 70, 23)]
    llm = llm_b200.LLM(str(folder), dtype="float32", device=DEV, context=256, batch=3)
    got = llm.generate(prompts, max_tokens=8, temperature=0.0, stop_tokens=[], repeat_penalty=1.0)
    for prompt, tokens in zip(prompts, got):
        assert tokens == plain.greedy(config, weights, prompt, 8)
    llm16 = llm_b200.LLM(str(folder), dtype="bfloat16", device=DEV, context=256, batch=3)
    for prompt, tokens in zip(prompts, llm16.generate(prompts, max_tokens=8, temperature=0.0, stop_tokens=[],
                                                      repeat_penalty=1.0)):
        sequence = list(prompt)
        for token in tokens:                                    # every token is a maximum of the plain logits up to rounding
            logits = plain.forward(config, weights, sequence)[-1]
            assert logits[token] >= logits.max() - 0.05 * float(logits.max() - logits.min())
            sequence.append(token)


def test_trace_replay_program(tmp_path):
    folder = make_folder(tmp_path, "P", torch.bfloat16)
    config, weights = plain.read_model_folder(folder)
    a, b = random_tokens(40, config["vocab"], 1), random_tokens(9, config["vocab"], 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:8], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[30]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a"]}]
    program = Path(__file__).resolve().parent.parent / "bin" / "trace_run"
    out = tmp_path / "out"
    result = subprocess.run([sys.executable, str(program), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                             "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-2000:]
    assert [line for line in result.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    read = lambda n: torch.frombuffer(bytearray((out / f"{n}.f32").read_bytes()), dtype=torch.float32).view(-1, config["vocab"])
    wa, wb = plain.forward(config, weights, a), plain.forward(config, weights, b)
    _check_logits(read(0), wa[[0, 29]], torch.float32)
    _check_logits(read(1), torch.stack([wa[30], wb[8]]), torch.float32)
    _check_logits(read(2), wa[39:40], torch.float32)
