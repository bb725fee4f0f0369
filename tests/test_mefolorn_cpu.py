"""Mefolorn on the CPU: configuration, the plain statement's own mechanisms, and the engine's
host-side logic (packing, positions, pages, slots, recurrent and convolution state) with the
kernels replaced by their plain statements, against the plain whole-sequence implementation."""
import copy
import math

import pytest
import torch

import plain_mefolorn as plain
from tiny_mefolorn import CONFIGS, MEF_P, MEF_Q, MEF_R, make_folder, random_tokens, tensor_shapes

from llm_b200.config import MefolornConfig, config_from_dict
from llm_b200.engine import Engine, Entry, declared_parameters, load_model
from llm_b200.errors import FormatError, MissingKey, Unsupported, WeightError

TOL = dict(atol=5e-5, rtol=3e-5)


def _setup(tmp_path, which, change=None, **engine_options):
    folder = make_folder(tmp_path, which, torch.float32, change)
    config, weights = plain.read_model_folder(folder)
    engine = Engine(load_model(folder, torch.float32, "cpu"), **{"max_tokens": 2048, **engine_options})
    return config, weights, engine


# ----------------------------------------------------------------------------- configuration

def test_config_gives_the_layers_and_names():
    config = config_from_dict(copy.deepcopy(MEF_P))
    assert isinstance(config, MefolornConfig)
    spec = config.model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3] and spec.head is None and spec.embedding_scale == 2.5
    pair, latent = spec.blocks[0].mixer, spec.blocks[1].mixer
    assert pair.kind == "side_by_side" and latent.kind == "latent_attention"
    left, right = pair.left, pair.right
    assert (left.n_heads, left.n_kv_heads, left.head_dim, left.value_dim, left.window) == (4, 2, 6, 10, 9)
    assert left.position.rotary_dim == 4 and left.position.pairing == "half" and left.out_scale == 0.7
    assert (right.width, right.blocks, right.conv_taps, right.decay, right.out_scale) == (24, 3, 3, 8.0, 1.2)
    assert (latent.n_heads, latent.head_dim, latent.value_dim, latent.q_rank, latent.kv_rank, latent.window) == (3, 10, 7, 12, 9, 5)
    assert spec.blocks[1].feed_forward is None and spec.blocks[1].ffn_norm is None
    assert spec.blocks[0].ffn_norm.weight == "l0.norm2" and spec.blocks[0].norm.alpha == "l0.norm1.alpha"
    nothing = config_from_dict(copy.deepcopy(MEF_R)).model_spec()
    assert nothing.blocks[0].mixer.left.position is None and nothing.blocks[0].mixer.left.window == 0
    assert nothing.blocks[1].mixer.window == 0 and nothing.embedding_scale == 1.0
    for raw in (MEF_P, MEF_Q, MEF_R):
        spec = config_from_dict(copy.deepcopy(raw)).model_spec()
        declared = {name: tuple(p.shape) for name, p in declared_parameters(spec).items()}
        assert declared == tensor_shapes(raw)
    assert config_from_dict(config.to_dict()).model_spec() == config.model_spec()


def test_config_errors_name_the_key():
    for path, value, error in [(("layers", 0, "mixer", "left", "heads"), 3, FormatError),       # 3 heads, 2 kv heads
                               (("layers", 0, "type"), "attention", Unsupported),
                               (("layers", 0, "mlp", "kind"), "routed", Unsupported),
                               (("layers", 0, "mixer", "left", "rot", "dims"), 7, FormatError),
                               (("layers", 0, "mixer", "right", "blocks"), 5, FormatError),
                               (("layers", 1, "mixer", "kv_rank"), 0, FormatError)]:
        raw = copy.deepcopy(MEF_P)
        at = raw
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(error):
            config_from_dict(raw)
    raw = copy.deepcopy(MEF_P)
    del raw["layers"][1]["mixer"]["q_rank"]
    with pytest.raises(MissingKey) as info:
        config_from_dict(raw)
    assert "q_rank" in str(info.value)


def test_a_missing_tensor_is_reported(tmp_path):
    def drop(weights):
        del weights["l1.mix.sink"]
        weights["l0.mix.left.talk"] = weights["l0.mix.left.talk"][:3]
    folder = make_folder(tmp_path, "P", torch.float32, weights_change=drop)
    with pytest.raises(WeightError) as info:
        load_model(folder, torch.float32, "cpu")
    assert "l1.mix.sink" in str(info.value) and "l0.mix.left.talk" in str(info.value)


# ----------------------------------------------------------------------------- the plain statement's mechanisms

def test_plain_mechanisms():
    gen = torch.Generator().manual_seed(0)
    x = torch.randn((7, 12), generator=gen)
    # the tanh norm has no statistic: a row's result does not depend on the row's other elements
    y = plain.tanh_norm(x, torch.tensor(0.5), torch.ones(12), torch.zeros(12))
    assert torch.allclose(y[:, 3], torch.tanh(0.5 * x[:, 3]))
    # windows: itself and the size - 1 positions before it
    seen = plain.visible(6, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True] and seen[1].tolist() == [True, True] + [False] * 4
    assert plain.visible(4, 0)[3].all()
    # a sink that dominates takes all the weight; a sink far below changes nothing
    q, k, v = torch.randn((5, 8), generator=gen), torch.randn((5, 8), generator=gen), torch.randn((5, 3), generator=gen)
    assert plain.sink_softmax_attention(q, k, v, 0.3, 0, torch.tensor(40.0)).abs().max() < 1e-6
    plain_softmax = torch.softmax((q @ k.T * 0.3).masked_fill(~plain.visible(5, 0), float("-inf")), dim=-1) @ v
    assert torch.allclose(plain.sink_softmax_attention(q, k, v, 0.3, 0, torch.tensor(-40.0)), plain_softmax, atol=1e-6)
    # the convolution: the last column is the current token's tap, zeros before the start
    u = torch.randn((5, 2), generator=gen)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]])
    c = plain.causal_conv(u, taps, torch.tensor([0.0, 10.0]))
    assert torch.allclose(c[:, 0], u[:, 0]) and torch.allclose(c[2:, 1], u[:3, 1] + 10.0) and torch.allclose(c[:2, 1], torch.full((2,), 10.0))
    # rotation: position 0 stays, norms stay, elements beyond the rotated part stay
    h = torch.randn((4, 2, 6), generator=gen)
    r = plain.rotate_half(h, {"base": 50.0, "dims": 4})
    assert torch.allclose(r[0], h[0]) and torch.allclose(r[..., 4:], h[..., 4:])
    assert torch.allclose((r[..., :4] ** 2).sum(-1), (h[..., :4] ** 2).sum(-1), atol=1e-5)
    assert torch.allclose(r[1, 0, 0], h[1, 0, 0] * math.cos(1.0) - h[1, 0, 2] * math.sin(1.0), atol=1e-6)
    # block gates: part b sees only its own channels
    m = torch.randn((2, 3, 3), generator=gen)
    g = plain.block_gate(torch.tensor([[1.0, 0, 0, 0, 0, 0]]), m, torch.zeros((2, 3)))
    assert torch.allclose(g[0, 3:], torch.full((3,), 0.5)) and torch.allclose(g[0, :3], torch.sigmoid(m[0, :, 0]))


# ----------------------------------------------------------------------------- the engine with plain kernels

@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_whole_prompt_matches_plain(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(150, config["vocab"], 1)
    want = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, list(range(len(tokens))))])
    assert torch.allclose(got, want, **TOL), float((got - want).abs().max())


@pytest.mark.parametrize("which", sorted(CONFIGS))
def test_token_by_token_equals_prefill(tmp_path, plain_kernels, which):
    config, weights, engine = _setup(tmp_path, which)
    tokens = random_tokens(80, config["vocab"], 2)
    want = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    for p, token in enumerate(tokens):                      # from the very first token on
        got = engine.step([Entry(slot, [token], [0])])
        assert torch.allclose(got[0], want[p], **TOL), (p, float((got[0] - want[p]).abs().max()))


@pytest.mark.parametrize("piece", [2, 3, 7, 64])
def test_prompts_cut_into_pieces(tmp_path, plain_kernels, piece):
    config, weights, engine = _setup(tmp_path, "P")
    tokens = random_tokens(131, config["vocab"], 3)
    want = plain.forward(config, weights, tokens)
    (slot,) = engine.acquire()
    for start in range(0, len(tokens), piece):
        part = tokens[start:start + piece]
        got = engine.step([Entry(slot, part, list(range(len(part))))])
        assert torch.allclose(got, want[start:start + len(part)], **TOL), start
    # the engine's own cutting of a long prompt into passes
    config, weights, engine = _setup(tmp_path, "Q", step_tokens=piece * 8)
    tokens = random_tokens(140, config["vocab"], 4)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, [0, 70, 139])])
    assert torch.allclose(got, plain.forward(config, weights, tokens)[[0, 70, 139]], **TOL)


def test_unequal_batch_slot_reuse_and_early_ends(tmp_path, plain_kernels):
    config, weights, engine = _setup(tmp_path, "P", max_tokens=1024)
    lengths = [70, 1, 33, 12]
    for again in range(3):                                   # slots, pages and states are taken again
        seqs = [random_tokens(n, config["vocab"], 10 * again + n) for n in lengths]
        want = [plain.forward(config, weights, s) for s in seqs]
        slots = engine.acquire(len(seqs))
        heads = [max(1, n - 5 - i) for i, n in enumerate(lengths)]
        got = engine.step([Entry(s, q[:h], [h - 1]) for s, q, h in zip(slots, seqs, heads)])
        for b, h in enumerate(heads):
            assert torch.allclose(got[b], want[b][h - 1], **TOL), (again, b)
        live = [b for b in range(len(seqs)) if heads[b] < lengths[b]]
        engine.release([slots[b] for b in range(len(seqs)) if b not in live])
        done = 0
        while live:
            got = engine.step([Entry(slots[b], [seqs[b][heads[b] + done]], [0]) for b in live])
            for r, b in enumerate(live):
                assert torch.allclose(got[r], want[b][heads[b] + done], **TOL), (again, b, done)
            done += 1
            ended = [b for b in live if heads[b] + done == lengths[b]]
            engine.release([slots[b] for b in ended])
            live = [b for b in live if b not in ended]
        engine.cache.check()
        assert engine.cache.slots.n_held == 0


def test_a_mixed_step(tmp_path, plain_kernels):
    """Two sequences go on by one token while a third brings the rest of its prompt."""
    config, weights, engine = _setup(tmp_path, "Q")
    a, b, c = (random_tokens(n, config["vocab"], 40 + n) for n in (30, 9, 90))
    sa, sb, sc = engine.acquire(3)
    engine.step([Entry(sa, a[:29], []), Entry(sb, b[:8], []), Entry(sc, c[:20], [])])
    got = engine.step([Entry(sa, [a[29]], [0]), Entry(sc, c[20:], [0, 69]), Entry(sb, [b[8]], [0])])
    wa, wb, wc = (plain.forward(config, weights, s) for s in (a, b, c))
    want = torch.stack([wa[29], wc[20], wc[89], wb[8]])
    assert torch.allclose(got, want, **TOL), float((got - want).abs().max())


def test_random_model_writer_round_trip(tmp_path, plain_kernels):
    from llm_b200.weights import write_random_model
    config = config_from_dict(copy.deepcopy(MEF_P))
    folder = write_random_model(tmp_path / "random", config, seed=5, dtype=torch.float32, std=0.3)
    raw, weights = plain.read_model_folder(folder)
    assert {k: tuple(v.shape) for k, v in weights.items()} == tensor_shapes(MEF_P)
    engine = Engine(load_model(folder, torch.float32, "cpu"), max_tokens=256)
    tokens = random_tokens(40, raw["vocab"], 6)
    (slot,) = engine.acquire()
    got = engine.step([Entry(slot, tokens, list(range(40)))])
    assert torch.allclose(got, plain.forward(raw, weights, tokens), **TOL)


def test_inspect_and_random_commands(tmp_path, capsys):
    import json
    from llm_b200.cli import main
    (tmp_path / "config.json").write_text(json.dumps(MEF_Q))
    assert main(["random", "--config", str(tmp_path / "config.json"), "--out", str(tmp_path / "m"), "--seed", "3"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    text = capsys.readouterr().out
    assert "Mefolorn" in text and "sigmoid attention" in text
