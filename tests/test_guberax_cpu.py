"""Guberax on the CPU: configuration, the plain statement's own mechanisms, and the engine's
host-side logic (packing, positions, pages, slots, convolution state, repeated passes) with the
kernels replaced by their plain statements, against the plain whole-sequence implementation."""
import copy
import math

import pytest
import torch

import plain_guberax as plain
from tiny_guberax import CONFIGS, GUB_P, GUB_Q, make_folder, random_tokens, tensor_shapes

from llm_b200.config import GuberaxConfig, config_from_dict
from llm_b200.engine import Engine, Entry, declared_parameters, load_model
from llm_b200.errors import FormatError, MissingKey, Unsupported, WeightError

TOL = dict(atol=3e-5, rtol=2e-5)


def _setup(tmp_path, which, change=None, **engine_options):
    folder = make_folder(tmp_path, which, torch.float32, change)
    config, weights = plain.read_model_folder(folder)
    engine = Engine(load_model(folder, torch.float32, "cpu"), **{"max_tokens": 2048, **engine_options})
    return config, weights, engine


# ----------------------------------------------------------------------------- configuration

def test_config_gives_the_layers_runs_and_names():
    config = config_from_dict(copy.deepcopy(GUB_P))
    assert isinstance(config, GuberaxConfig)
    spec = config.model_spec()
    runs = [(e.layer, e.add_embedding) for e in spec.schedule]
    assert runs == [(0, False), (1, False), (1, True), (1, True), (2, False)] == plain.layer_runs(GUB_P)
    assert all(e.cache_of is None for e in spec.schedule)            # every run has a cache of its own
    assert spec.logit_softcap == 12.0 and spec.head == "head" and spec.embedding == "embed"
    first, second, third = (b.mixer for b in spec.blocks)
    assert (first.n_heads, first.n_kv_heads, first.head_dim, first.value_dim) == (4, 2, 6, 10)
    assert (first.window, first.keep_first, first.conv_taps, first.diff) == (9, 2, 3, 0.25)
    assert first.position.rotary_dim == 4 and first.position.pairing == "interleaved"
    assert second.position.scaling is None and second.keep_first == 0
    assert third.position is None and third.window == 0 and third.conv_taps == 0
    assert spec.blocks[1].feed_forward is None and spec.blocks[0].feed_forward.intermediate == 52
    declared = {name: tuple(p.shape) for name, p in declared_parameters(spec).items()}
    assert declared == tensor_shapes(GUB_P)
    assert config_from_dict(config.to_dict()).model_spec() == spec


def test_config_errors_name_the_key():
    for path, value, error in [(("layers", 0, "mixer", "heads"), 3, FormatError),          # 3 heads, 2 kv heads
                               (("layers", 0, "type"), "recurrent", Unsupported),
                               (("layers", 0, "mlp", "kind"), "routed", Unsupported),
                               (("layers", 0, "mixer", "rot", "dims"), 7, FormatError),
                               (("loop", "stop"), 9, FormatError)]:
        raw = copy.deepcopy(GUB_P)
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            config = config_from_dict(raw)
            from llm_b200.engine import DecoderModel
            DecoderModel(config.model_spec())
    raw = copy.deepcopy(GUB_P)
    del raw["layers"][1]["mixer"]["vdim"]
    with pytest.raises(MissingKey, match="vdim"):
        config_from_dict(raw)


def test_a_missing_tensor_is_reported(tmp_path):
    def drop(weights):
        del weights["l1.mix.k.conv"]
    folder = make_folder(tmp_path, "P", torch.float32, weights_change=drop)
    with pytest.raises(WeightError, match="l1.mix.k.conv"):
        load_model(folder, torch.float32, "cpu")


# ----------------------------------------------------------------------------- the plain statement itself

def test_plain_mechanisms():
    # the norm's weight is an offset from one
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(plain.offset_norm(x, torch.tensor([0.0, 1.0]), 0.0), torch.tensor([[3.0, 8.0]]) / math.sqrt(12.5))
    # convolution: the last tap multiplies the present row
    u = torch.tensor([[1.0], [10.0], [100.0]])
    assert plain.short_conv(u, torch.tensor([[2.0, 3.0]])).flatten().tolist() == [3.0, 32.0, 320.0]
    # window of 3 that keeps the first 2 keys
    mask = {"size": 3, "keep_first": 2}
    assert [j for j in range(8) if plain.visible(7, j, mask)] == [0, 1, 5, 6, 7]
    assert [j for j in range(8) if plain.visible(2, j, mask)] == [0, 1, 2]
    # frequencies: short wavelengths stay, long ones slow down by the factor
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain_f = [10000.0 ** (-2.0 * i / 16) for i in range(8)]
    scaled = plain.rotation_frequencies(rot)
    assert scaled[0] == plain_f[0] and scaled[-1] == pytest.approx(plain_f[-1] / 4.0)
    assert any(f / 4.0 < s < f for f, s in zip(plain_f, scaled))
    # rotation turns pairs (2i, 2i + 1) and leaves the rest of a unit alone
    x = torch.arange(12, dtype=torch.float32).view(1, 2, 6)
    turned = plain.rotate(x, {"base": 10.0, "dims": 2}, [1])
    assert torch.equal(turned[..., 2:], x[..., 2:])
    assert turned[0, 0, 0] == pytest.approx(0 * math.cos(1.0) - 1 * math.sin(1.0))
    assert turned[0, 0, 1] == pytest.approx(1 * math.cos(1.0) + 0 * math.sin(1.0))


# ----------------------------------------------------------------------------- the engine's host logic

@pytest.mark.parametrize("which", ["P", "Q", "R"])
def test_whole_prompt_matches_plain(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(37 if which != "Q" else 90, config["vocab"], 7)
    expected = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    logits = engine.step([Entry(slot, tokens, list(range(len(tokens))))])
    assert torch.allclose(logits, expected, **TOL)
    engine.release([slot])
    engine.cache.check()


@pytest.mark.parametrize("which", ["P", "Q"])
def test_token_by_token_equals_prefill(tmp_path, plain_kernels, which):
    """From the first token on, one token a step: the convolution's state and every run's cache carry
    the sequence, past the window's edge and the kept first tokens."""
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(24 if which == "P" else 80, config["vocab"], 3)
    expected = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    for p, token in enumerate(tokens):
        logits = engine.step([Entry(slot, [token], [0])])
        assert torch.allclose(logits[0], expected[p], **TOL), p


@pytest.mark.parametrize("piece", [2, 3, 7, 16])
def test_prompts_cut_into_pieces(tmp_path, plain_kernels, piece):
    """Pieces shorter than the convolution, equal to it, and longer; as steps of the caller and as
    passes cut by the engine (step_tokens)."""
    config, weights, engine = _setup(tmp_path, "P", step_tokens=piece)
    tokens = random_tokens(29, config["vocab"], 5)
    expected = plain.forward(config, weights, tokens)
    a, b = engine.acquire(2)
    logits = engine.step([Entry(a, tokens, list(range(len(tokens))))])          # cut by the engine
    assert torch.allclose(logits, expected, **TOL)
    for start in range(0, len(tokens), piece):                                   # cut by the caller
        part = tokens[start:start + piece]
        logits = engine.step([Entry(b, part, list(range(len(part))))])
        assert torch.allclose(logits, expected[start:start + len(part)], **TOL), start


def test_unequal_batch_slot_reuse_and_early_ends(tmp_path, plain_kernels):
    config, weights, engine = _setup(tmp_path, "P", max_tokens=640, max_slots=4)
    lengths = [1, 13, 30, 66]
    seqs = [random_tokens(n + 5, config["vocab"], 20 + i) for i, n in enumerate(lengths)]
    expected = [plain.forward(config, weights, s) for s in seqs]
    for _ in range(2):                                   # the second time runs on slots and pages that were used
        slots = engine.acquire(len(seqs))
        logits = engine.step([Entry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lengths)])
        for b, n in enumerate(lengths):
            assert torch.allclose(logits[b], expected[b][n - 1], **TOL)
        live = list(range(len(seqs)))
        for k in range(5):
            if k == 3:
                engine.release([slots[0], slots[2]])
                live = [1, 3]
            logits = engine.step([Entry(slots[b], [seqs[b][lengths[b] + k]], [0]) for b in live])
            for row, b in enumerate(live):
                assert torch.allclose(logits[row], expected[b][lengths[b] + k], **TOL)
        engine.release([slots[b] for b in live])
        engine.cache.check()
        assert engine.cache.slots.n_held == 0


def test_a_mixed_step(tmp_path, plain_kernels):
    """Two sequences go on by one token while a third brings a piece of its prompt onto what it holds."""
    config, weights, engine = _setup(tmp_path, "P")
    seqs = [random_tokens(n, config["vocab"], 40 + n) for n in (12, 20, 31)]
    expected = [plain.forward(config, weights, s) for s in seqs]
    slots = engine.acquire(3)
    engine.step([Entry(slots[0], seqs[0][:11], []), Entry(slots[1], seqs[1][:19], []), Entry(slots[2], seqs[2][:10], [])])
    logits = engine.step([Entry(slots[0], seqs[0][11:], [0]), Entry(slots[1], seqs[1][19:], [0]),
                          Entry(slots[2], seqs[2][10:], [0, 20])])
    assert torch.allclose(logits[0], expected[0][11], **TOL)
    assert torch.allclose(logits[1], expected[1][19], **TOL)
    assert torch.allclose(logits[2], expected[2][10], **TOL) and torch.allclose(logits[3], expected[2][30], **TOL)


def test_random_model_writer_round_trip(tmp_path, plain_kernels):
    """`write_random_model` serves the architecture: the folder it writes loads and runs."""
    from llm_b200.weights import write_random_model
    config = config_from_dict(copy.deepcopy(GUB_Q))
    folder = write_random_model(tmp_path / "random", config, 5, torch.float32, std=0.08)
    raw, weights = plain.read_model_folder(folder)
    assert abs(float(weights["l0.norm1"].mean())) < 0.02          # the norm's weights lie around zero
    engine = Engine(load_model(folder, torch.float32, "cpu"), max_tokens=256)
    tokens = random_tokens(20, raw["vocab"], 1)
    (slot,) = engine.acquire()
    logits = engine.step([Entry(slot, tokens, [19])])
    assert torch.allclose(logits[0], plain.forward(raw, weights, tokens)[19], **TOL)


# ----------------------------------------------------------------------------- kernel choice and command line

def test_kernel_choice_for_the_differential_attention():
    from llm_b200.ops import tactics
    names = {r.name for r in tactics.rows("diff_attention")}
    assert names == {"diff_attention_decode", "diff_attention_prefill", "diff_attention_generic"}
    assert all(r.evidence for r in tactics.rows("diff_attention"))
    bf16, f32 = torch.bfloat16, torch.float32
    choose = tactics.choose_diff_attention
    assert choose(True, bf16, 32, 8, 64, 128, 4096, 4, True, True) == "diff_attention_decode"
    assert choose(False, bf16, 32, 8, 64, 128, 4096, 4, True, True) == "diff_attention_prefill"
    assert choose(True, bf16, 32, 2, 64, 128, 0, 0, True, True) == "diff_attention_prefill"        # a group of 16 heads: no decode tile
    assert choose(False, bf16, 4, 2, 40, 72, 0, 0, True, True) == "diff_attention_generic"         # sizes no tile takes
    assert choose(True, f32, 32, 8, 64, 128, 0, 0, True, True) == "diff_attention_generic"         # the 32-bit path
    text = tactics.explain("diff_attention", decode=False, dtype=bf16, n_heads=4, n_kv_heads=2, head_dim=40,
                           value_dim=72, window=0, keep_first=0, packed=True, aligned=True)
    assert "map size 40 with value size 72" in text
    tactics.disable("diff_attention_prefill")
    try:
        assert choose(False, bf16, 32, 8, 64, 128, 4096, 4, True, True) == "diff_attention_generic"
    finally:
        tactics.enable("diff_attention_prefill")


def test_inspect_and_random_commands(tmp_path, capsys):
    import json
    from llm_b200 import cli
    folder = make_folder(tmp_path, "Q", torch.bfloat16)
    assert cli.inspect(str(folder)) == 0
    out = capsys.readouterr().out
    assert "architecture  Guberax" in out and "diff_attention_prefill" in out and "runnable" in out
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(GUB_P))
    assert cli.random_folder(["--config", str(config_file), "--out", str(tmp_path / "made"), "--seed", "3"]) == 0
    raw, weights = plain.read_model_folder(tmp_path / "made")
    assert raw["architecture"] == "Guberax" and set(weights) == set(tensor_shapes(GUB_P))
