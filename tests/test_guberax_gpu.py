"""Guberax on the GPU: every new kernel beside its plain statement, and the model through the
engine, the generation entry point and the trace-replay program against the plain whole-sequence
implementation, in 32-bit and in bfloat16."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_guberax as plain
import plain_ops
from tiny_guberax import CONFIGS, make_folder, random_tokens

pytestmark = pytest.mark.gpu

PAGE = 64
DEV = "cuda:0"
SHAPES = [(32, 32), (32, 64), (48, 96), (64, 64), (64, 128), (128, 128)]       # what the tensor-core kernels take


def _ops():
    from llm_b200 import ops
    return ops


# ----------------------------------------------------------------------------- a paged cache by hand

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
        v = torch.randn((self.n_pages, heads, PAGE, value_width), generator=gen).to(dtype).to(DEV)
        return k, v

    def place(self, b, position):
        return int(self.table[b, position // PAGE]), position % PAGE


def _close(got, want, dtype, what=""):
    got, want = got.float(), want.float()
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=2e-5, rtol=2e-5), (what, float((got - want).abs().max()))
    else:
        scale = float(want.abs().max()) + 1e-6
        assert float((got - want).abs().max()) <= 0.03 * scale, (what, float((got - want).abs().max()), scale)
        assert float((got - want).abs().mean()) <= 0.004 * scale, what


# ----------------------------------------------------------------------------- convolution + rotation + cache write

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [
    # heads, kv heads, map size, value size, taps, rotated, interleaved
    (4, 2, 6, 10, 3, 4, True), (3, 3, 10, 7, 2, 10, True), (2, 1, 16, 24, 4, 8, False), (4, 2, 48, 96, 3, 32, True),
    (2, 2, 8, 12, 0, 0, True), (2, 1, 16, 16, 1, 16, True), (1, 1, 5, 3, 8, 2, True),
    (2, 2, 32, 64, 3, 16, True), (2, 2, 16, 24, 0, 0, True), (4, 2, 64, 128, 8, 64, True), (2, 1, 16, 32, 2, 0, True)])
def test_conv_rope_cache_write(dtype, case):
    ops = _ops()
    heads, groups, dim, vdim, taps, n_rot, interleaved = case
    qw, kw, vw = heads * 2 * dim, groups * 2 * dim, groups * vdim
    channels = qw + kw + vw
    gen = torch.Generator().manual_seed(3)
    cases = [([70, 5, 130, 64], [70, 2, 66, 1]), ([9, 200, 65], [1, 1, 1]), ([3], [3])]
    if dim % 8 == 0 and vdim % 8 == 0:                   # long steps: blocks walk several tokens, across sequence edges
        cases.append(([1500, 7, 300, 77, 901], [1493, 7, 129, 1, 900]))
    for lengths, new in cases:
        batch = Batch(lengths, new, seed=len(lengths))
        u = torch.randn((batch.n_tokens, channels), generator=gen).to(dtype).to(DEV)
        w = torch.randn((channels, taps), generator=gen).to(DEV) if taps else None
        state = torch.randn((len(lengths) + 1, max(taps - 1, 0), channels), generator=gen).to(dtype).to(DEV) if taps > 1 else None
        if state is not None:
            for b, (n, k) in enumerate(zip(lengths, new)):               # a sequence that starts here has no past
                if n == k:
                    state[int(batch.slots[b])] = 0
        table = None
        if n_rot:
            angle = torch.arange(1600, dtype=torch.float64)[:, None] * torch.rand(n_rot // 2, generator=gen, dtype=torch.float64)
            table = torch.cat([angle.cos(), angle.sin()], dim=1).float().to(DEV)
        results = []
        rows = w.t().contiguous().to(torch.bfloat16) if (taps and dtype == torch.bfloat16) else None
        if rows is not None:                                             # the kernel may read the taps from their bfloat16 copy
            w = rows.float().t().contiguous()
        for fn in (ops.conv_rope_cache_write, plain_ops.conv_rope_cache_write, ops.conv_rope_cache_write):
            k_cache, v_cache = batch.caches(groups, 2 * dim, vdim, dtype, seed=5)
            held = state.clone() if state is not None else None
            q_out = torch.zeros((batch.n_tokens, qw), dtype=dtype, device=DEV)
            fn(u, w, held, batch.tok_pos, batch.tok_seq, batch.cu, batch.seq_lens, batch.slots, table, dim,
               interleaved, q_out, kw, vw, batch.table, batch.width, k_cache, v_cache,
               write_cache=True, single_tokens=all(k == 1 for k in new),
               conv_w_rows=rows if len(results) == 2 else None)
            results.append((q_out, k_cache, v_cache, held))
        torch.cuda.synchronize()
        for got, want, what in zip(results[0], results[1], ("queries", "keys", "values", "state")):
            if got is not None:
                _close(got, want, dtype, what)
        for got, other in zip(results[0], results[2]):                   # with and without the taps' copy: the same bits
            assert got is None or torch.equal(got, other)
        if state is not None:                                            # the state holds the last rows exactly
            assert torch.equal(results[0][3], results[1][3])


# ----------------------------------------------------------------------------- differential attention

def _attention_both(batch, heads, groups, dim, vdim, dtype, window, keep_first, q=None, caches=None, decode=False,
                    variant=None, lam=0.7):
    ops = _ops()
    from llm_b200.ops import tactics
    gen = torch.Generator().manual_seed(11)
    if q is None:
        q = torch.randn((batch.n_tokens, heads * 2 * dim), generator=gen).to(dtype).to(DEV)
    k_cache, v_cache = caches if caches is not None else batch.caches(groups, 2 * dim, vdim, dtype, seed=7)
    scale = dim ** -0.5
    args = (q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, groups, dim, vdim,
            scale, window, keep_first, lam, 1e-5, 0.6)
    extra = dict(decode=decode, seq_lens=batch.seq_lens, max_len=max(batch.lengths), cu_seqlens=batch.cu,
                 max_new=max(batch.new), seq_order=batch.order)
    switched = []
    if variant is not None:
        for name in ("diff_attention_decode", "diff_attention_prefill", "diff_attention_generic"):
            if name != variant:
                tactics.disable(name)
                switched.append(name)
    try:
        chosen = tactics.choose_diff_attention(decode, dtype, heads, groups, dim, vdim, window, keep_first, True, True)
        got = ops.diff_attention(*args, **extra)
    finally:
        for name in switched:
            tactics.enable(name)
    torch.cuda.synchronize()
    if variant is not None:
        assert chosen == variant
    return got, plain_ops.diff_attention(*args, **extra)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(4, 2, 6, 10), (3, 3, 10, 7), (2, 1, 40, 72), (8, 1, 16, 24)])
def test_diff_attention_any_sizes(dtype, sizes):
    heads, groups, dim, vdim = sizes
    for window, keep_first in [(0, 0), (9, 2), (70, 0), (64, 64), (5, 100)]:
        batch = Batch([70, 5, 131, 64], [70, 2, 66, 1], seed=window)
        got, want = _attention_both(batch, heads, groups, dim, vdim, dtype, window, keep_first)
        _close(got, want, dtype, (window, keep_first))


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("window,keep_first", [(0, 0), (70, 3), (64, 0), (33, 65), (200, 1)])
def test_diff_attention_prefill_kernel(shape, window, keep_first):
    """The tensor-core prefill kernel: whole prompts, continued prompts that start off every tile and page
    edge, a sequence that brings one token among them, windows that end inside, at and before a page."""
    dim, vdim = shape
    batch = Batch([300, 64, 131, 77, 1, 260], [300, 64, 66, 1, 1, 129], seed=window + dim)
    got, want = _attention_both(batch, 4, 2, dim, vdim, torch.bfloat16, window, keep_first, variant="diff_attention_prefill")
    _close(got, want, torch.bfloat16, (shape, window, keep_first))


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("window,keep_first", [(0, 0), (70, 3), (64, 0), (33, 65), (200, 1)])
def test_diff_attention_decode_kernel(shape, window, keep_first, monkeypatch):
    """The split-KV decode kernel at lengths on, before and behind page edges, with one and several slices
    (also more slices than pages), groups of 1, 3 and 8 heads."""
    dim, vdim = shape
    lengths = [1, 63, 64, 65, 128, 129, 300, 700]
    for heads, groups in [(4, 4), (6, 2), (8, 1)]:
        for splits in ("1", "2", "8"):
            monkeypatch.setenv("LLMB_DECODE_SPLITS", splits)
            batch = Batch(lengths, [1] * len(lengths), seed=window + dim)
            got, want = _attention_both(batch, heads, groups, dim, vdim, torch.bfloat16, window, keep_first, decode=True,
                                        variant="diff_attention_decode")
            _close(got, want, torch.bfloat16, (shape, window, keep_first, heads, splits))
    # a launch of many blocks (the kernel then takes its short ring of pages)
    monkeypatch.setenv("LLMB_DECODE_SPLITS", "2")
    many = [1 + (37 * i) % 300 for i in range(40)]
    batch = Batch(many, [1] * len(many), seed=dim)
    got, want = _attention_both(batch, 4, 4, dim, vdim, torch.bfloat16, window, keep_first, decode=True,
                                variant="diff_attention_decode")
    _close(got, want, torch.bfloat16, (shape, window, keep_first, "many blocks"))


@pytest.mark.parametrize("variant,dtype", [("diff_attention_generic", torch.float32),
                                           ("diff_attention_generic", torch.bfloat16),
                                           ("diff_attention_prefill", torch.bfloat16),
                                           ("diff_attention_decode", torch.bfloat16)])
def test_planted_keys_show_what_a_query_sees(variant, dtype):
    """One key of a long sequence gets a direction that the last query's map 1 points at (score far above
    every other) and a value of its own. Inside the window, among the kept first tokens or far back
    without a window it must dominate map 1's result; one position outside the window or behind the
    kept tokens it must not show at all. Map 2 and the other head stay ordinary."""
    ops = _ops()
    heads, groups, dim, vdim = 2, 1, 64, 128
    window, keep_first, length = 150, 5, 700
    decode = variant == "diff_attention_decode"
    for planted, w, seen in [(length - window, window, True), (length - window - 1, window, False),     # the window's edge
                             (keep_first - 1, window, True), (keep_first, window, False),              # the kept tokens' edge
                             (5, 0, True), (63, 0, True), (64, 0, True),                                # far back, page borders
                             (length - 1, window, True), (length - 64, window, True)]:
        batch = Batch([length, 90], [1 if decode else 130, 1 if decode else 90], seed=1)
        k_cache, v_cache = batch.caches(groups, 2 * dim, vdim, dtype, seed=2, std=0.3)
        gen = torch.Generator().manual_seed(4)
        q = (0.3 * torch.randn((batch.n_tokens, heads * 2 * dim), generator=gen)).to(dtype).to(DEV)
        last = (1 if decode else 130) - 1                                 # the long sequence's last query
        direction = torch.zeros(dim)
        direction[::2] = 1.0
        q[last, :dim] = (4.0 * direction).to(dtype)                        # head 0, map 1
        page, row = batch.place(0, planted)
        k_cache[page, 0, row, :dim] = (4.0 * direction).to(dtype)          # score 16 * 32 / 8 = 64 against ~0
        v_cache[page, 0, row] = 0
        v_cache[page, 0, row, 7] = 50.0
        # lambda 0, no norm, scale 1: the result of head 0 is map 1's weighted values themselves
        args = (q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, heads, groups, dim, vdim,
                dim ** -0.5, w, keep_first if w else 0, 0.0, 1e-5, 1.0)
        extra = dict(head_norm=False, decode=decode, seq_lens=batch.seq_lens, max_len=length, cu_seqlens=batch.cu,
                     max_new=max(batch.new), seq_order=batch.order)
        from llm_b200.ops import tactics
        others = [n for n in ("diff_attention_decode", "diff_attention_prefill", "diff_attention_generic") if n != variant]
        for name in others:
            tactics.disable(name)
        try:
            got = ops.diff_attention(*args, **extra)
        finally:
            for name in others:
                tactics.enable(name)
        torch.cuda.synchronize()
        value = float(got[last, 7])
        if seen:
            assert value > 45.0, (planted, w, value)
        else:
            assert abs(value) < 5.0, (planted, w, value)
        _close(got, plain_ops.diff_attention(*args, **extra), dtype, (planted, w))


def test_head_norm_difference_and_scale():
    """lambda, the head's norm and the output scale, each alone (the generic kernel in 32-bit)."""
    batch = Batch([40, 7], [40, 7])
    for lam, norm in [(0.0, False), (1.3, False), (-0.4, True), (0.9, True)]:
        ops = _ops()
        gen = torch.Generator().manual_seed(9)
        q = torch.randn((47, 2 * 2 * 8), generator=gen).to(DEV)
        k_cache, v_cache = batch.caches(1, 16, 12, torch.float32)
        args = (q, k_cache, v_cache, batch.table, batch.width, batch.tok_pos, batch.tok_seq, 2, 1, 8, 12, 0.3, 0, 0, lam,
                1e-3, 0.75)
        got = ops.diff_attention(*args, head_norm=norm)
        _close(got, plain_ops.diff_attention(*args, head_norm=norm), torch.float32, (lam, norm))


def test_small_row_kernels():
    ops = _ops()
    gen = torch.Generator().manual_seed(1)
    x = (20 * torch.randn((5, 97), generator=gen)).to(DEV)
    want = 7.5 * torch.tanh(x / 7.5)
    assert torch.allclose(ops.softcap_(x.clone(), 7.5), want, atol=1e-5)
    y = torch.randn((5, 97), generator=gen).to(DEV)
    emit = ops.Emit(torch.empty((5, 97), dtype=torch.bfloat16, device=DEV), torch.zeros((5, ops.SUMSQ_LD), device=DEV))
    total = ops.add_rows_(x.clone(), y, emit=emit)
    torch.cuda.synchronize()
    assert torch.equal(total, x + y) and torch.equal(emit.rows, (x + y).to(torch.bfloat16))
    assert torch.allclose(emit.sumsq[:, 0], ((x + y) ** 2).sum(-1), rtol=1e-5) and emit.parts == 1


# ----------------------------------------------------------------------------- the model through the engine

def _setup(tmp_path, which, dtype, **engine_options):
    from llm_b200.engine import Engine, load_model
    folder = make_folder(tmp_path, which, torch.bfloat16)
    config, weights = plain.read_model_folder(folder)
    engine = Engine(load_model(folder, dtype, DEV), **{"max_tokens": 4096, **engine_options})
    return config, weights, engine


def _check_logits(got, want, dtype, what=""):
    got, want = got.float().cpu(), want.float()
    if dtype == torch.float32:
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (what, float((got - want).abs().max()))
    else:
        span = float(want.max() - want.min())
        assert float((got - want).abs().max()) <= 0.05 * span, (what, float((got - want).abs().max()), span)
        assert float((got - want).abs().mean()) <= 0.01 * span, what


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("which", ["P", "Q", "R"])
def test_whole_decode_pieces_and_batches_agree_with_plain(tmp_path, which, dtype):
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, which, dtype, step_tokens=48)
    lengths = [150, 1, 67, 20]
    seqs = [random_tokens(n, config["vocab"], 30 + n) for n in lengths]
    expected = [plain.forward(config, weights, s) for s in seqs]
    for again in range(2):                                       # the second time reuses slots and pages
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
def test_long_decoding_passes_the_window_and_page_edges(tmp_path, dtype):
    """One token a step from the first on, 200 steps: windows of 70 and 33 slide over decoded tokens,
    the kept first tokens stay, pages fill and follow each other, and steps are replayed from graphs."""
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", dtype)
    tokens = random_tokens(200, config["vocab"], 77)
    expected = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    for p, token in enumerate(tokens):
        logits = engine.step([Entry(slot, [token], [0])])
        _check_logits(logits[0], expected[p], dtype, p)
    assert engine.graph_replays > 100


@pytest.mark.parametrize("piece", [2, 5, 64])
def test_pieces_down_to_two_tokens(tmp_path, piece):
    from llm_b200.engine import Entry
    config, weights, engine = _setup(tmp_path, "Q", torch.float32)
    tokens = random_tokens(140, config["vocab"], 8)
    expected = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    for start in range(0, len(tokens), piece):
        part = tokens[start:start + piece]
        logits = engine.step([Entry(slot, part, list(range(len(part))))])
        _check_logits(logits, expected[start:start + len(part)], torch.float32, start)


def test_batch_and_cut_change_nothing_in_32_bit(tmp_path):
    """A position's logits alone, among neighbours, and with its prompt cut: equal to the last bit in the
    32-bit path (every reduction's order depends only on the position)."""
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
    cut = engine.step([Entry(e, seqs[0][21:], [49 - 21])])
    assert torch.equal(alone[0], cut[0])


def test_folded_norm_and_unfused_agree(tmp_path, monkeypatch):
    """bfloat16 with the norm folded into both products of a block, against the norm as a kernel of its own."""
    import llm_b200.parts.block as block
    from llm_b200.engine import Engine, Entry, load_model
    folder = make_folder(tmp_path, "Q", torch.bfloat16)
    config, weights = plain.read_model_folder(folder)
    tokens = random_tokens(100, config["vocab"], 2)
    expected = plain.forward(config, weights, tokens)
    outs = []
    for fold in (True, False):
        monkeypatch.setattr(block, "FOLD_NORMS", fold)
        model = load_model(folder, torch.bfloat16, DEV)
        assert all(b.folded == fold for b in model.blocks)
        engine = Engine(model, max_tokens=512)
        (slot,) = engine.acquire()
        outs.append(engine.step([Entry(slot, tokens, list(range(100)))]))
        _check_logits(outs[-1], expected, torch.bfloat16, fold)


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


def test_a_group_no_decode_tile_holds():
    """16 query heads on one key/value head: the decode kernel's tile has 8 rows a map, so a decode step runs on
    the prefill kernel (one query a sequence); and with sizes no tile takes, on the generic kernel."""
    lengths = [1, 64, 65, 200, 333]
    batch = Batch(lengths, [1] * len(lengths), seed=5)
    got, want = _attention_both(batch, 16, 1, 32, 64, torch.bfloat16, 70, 3, decode=True, variant=None)
    _close(got, want, torch.bfloat16, "prefill kernel in a decode step")
    got, want = _attention_both(batch, 16, 1, 24, 40, torch.bfloat16, 70, 3, decode=True, variant=None)
    _close(got, want, torch.bfloat16, "generic kernel in a decode step")
