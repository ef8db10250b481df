"""The Libulorn model in the engine (step function, cache and state manager, scheduler) on the CPU stand-in kernels
against the plain implementation; its parts alone against the plain functions; its configuration."""
import copy

import pytest
import torch

import plain_libulorn as plain
import replay_modes
from helpers import assert_close, make_runner, random_tokens
from libulorn_configs import CONFIGS, PAGE_SIZE, config_dict, make_libulorn_folder
from torch_kernels import TorchKernels

REL = 1e-4


def _runner(tmp_path, name, num_pages=64, sharpen=1.0, **kw):
    folder = make_libulorn_folder(tmp_path, name, sharpen=sharpen)
    runner = make_runner(folder, TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=num_pages, **kw)
    config, weights = plain.read_folder(folder)
    return runner, config, weights


# ---- configuration --------------------------------------------------------------------------------------------------
def test_config_round_trip():
    from kvcache_b200.config import config_from_dict
    for name in CONFIGS:
        c = config_from_dict(config_dict(name))
        assert config_from_dict(c.to_dict()) == c
    c = config_from_dict(config_dict("A"))
    assert [l.type for l in c.layers] == ["mlstm", "parallel", "parallel"] and c.layers[2].mlp is None
    left = c.layers[1].mixer.left
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.window) == (4, 2, 16, 24, 11) and left.rot.scaling.high == 4.0
    assert c.layers[1].mixer.right.tau == 4.0 and c.layers[0].mixer.gate_cap == 8.0 and c.bigram.buckets == 97
    assert c.layers[0].mlp.shared.ff == 40 and c.layers[0].mlp.expert.limit == 1.5
    b = config_from_dict(config_dict("B"))
    assert b.layers[0].mlp.shared is None and b.layers[2].mixer.left.window is None and b.layers[2].mixer.left.rot is None
    assert config_from_dict(config_dict("C")).bigram is None


def test_config_faults_are_all_reported():
    from kvcache_b200.config import ConfigError, config_from_dict
    bad = config_dict("A")
    bad["layers"][0]["mixer"].pop("gate_cap")
    bad["layers"][1]["mixer"]["left"]["kv_heads"] = 3
    bad["layers"][1]["mlp"]["router"]["top"] = 9
    bad["layers"][2]["type"] = "convolution"
    bad["layers"][1]["mixer"]["right"].pop("tau")
    del bad["norm"]
    with pytest.raises(ConfigError) as info:
        config_from_dict(bad)
    text = str(info.value)
    for piece in ("gate_cap", "not a multiple of kv_heads", "top 9", "convolution", "tau", "norm"):
        assert piece in text, piece


def test_model_as_data(tmp_path):
    """Cache entries: pages for the attention side of a parallel layer (a group per window), float32 states for the
    matrix-state mixers, one int32 per request for the pair embedding, after the layers' entries."""
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    model = load_model(make_libulorn_folder(tmp_path, "A"), "float32", "cpu", max_positions=64)
    entries = model.cache_entries()
    assert len(entries) == 4 and entries[0].kv is None and set(entries[0].state) == {"memory", "normalizer", "maximum"}
    assert entries[0].state["memory"].shape == (2, 24, 16) and entries[0].state["maximum"].shape == (2,)
    assert (entries[1].kv.num_kv_heads, entries[1].kv.head_dim, entries[1].kv.v_head_dim, entries[1].kv.window) == (2, 16, 24, 11)
    assert entries[2].kv.window == 16 and set(entries[1].state) == {"right.memory"} and entries[1].state["right.memory"].shape == (3, 8, 16)
    assert entries[3].kv is None and entries[3].state["previous_token"].dtype == "int32"
    cache = CacheManager(entries, page_size=8, num_pages=8, max_slots=3, max_tokens_per_request=64, dtype="float32", device="cpu")
    assert len(cache.groups) == 2 and cache.states[3]["previous_token"].shape == (3,) and cache.states[3]["previous_token"].dtype == torch.int32
    only_memory = load_model(make_libulorn_folder(tmp_path, "C"), "float32", "cpu", max_positions=64)
    assert all(e.kv is None for e in only_memory.cache_entries()) and only_memory.embedding_parts == []


def test_decay_rank_comes_from_the_checkpoint(tmp_path):
    """The inner size of the decay's two matrices is no key of the configuration: whatever the checkpoint's pair agrees on."""
    import json
    import os
    from kvcache_b200.engine.loading import load_model
    from kvcache_b200.weights import WeightError
    folder = make_libulorn_folder(tmp_path, "B")
    path = os.path.join(folder, "config.json")
    with open(path) as fh:
        data = json.load(fh)
    for layer in data["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("decay_rank")
    with open(path, "w") as fh:
        json.dump(data, fh)
    model = load_model(folder, "float32", "cpu", max_positions=32)
    assert model.blocks[0].mixer.right.w_a1.shape[0] == 3 and model.blocks[2].mixer.right.w_a1.shape[0] == 16
    data["layers"][0]["mixer"]["right"]["dim"] = 41
    with open(path, "w") as fh:
        json.dump(data, fh)
    with pytest.raises(WeightError, match="l0.mix.right"):
        load_model(folder, "float32", "cpu", max_positions=32)


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rot", [{"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}},
                                 {"base": 100.0, "dims": 6}, {"base": 300000.0, "dims": 12, "scaling": {"factor": 2.5, "low": 2.0, "high": 8.0, "original": 64}},
                                 {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}])
def test_rotation_tables(rot):
    from kvcache_b200.parts.position import RotaryHalf, WavelengthScaling
    s = rot.get("scaling")
    part = RotaryHalf(rot["dims"], rot["base"], 300, None if s is None else WavelengthScaling(s["factor"], s["low"], s["high"], s["original"]))
    part.bind({}, torch.device("cpu"))
    freq = plain.rotation_frequencies(rot)
    assert torch.allclose(torch.from_numpy(part.frequencies()), freq, rtol=1e-12, atol=0)
    if s is not None:          # all three pieces of the stretch occur, or the test shows nothing
        plain_freq = plain.rotation_frequencies({"base": rot["base"], "dims": rot["dims"]})
        ratio = freq / plain_freq
        assert bool((ratio == 1.0).any()) and bool(torch.isclose(ratio, torch.tensor(1.0 / s["factor"], dtype=torch.float64)).any())
    table = part.rotation()
    pos = torch.tensor([0, 1, 17, 255, 299])
    x = torch.randn(5, 3, rot["dims"] + 4, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    half = rot["dims"] // 2
    c, s_ = table.cos[pos].double()[:, None, :], table.sin[pos].double()[:, None, :]
    mine = torch.cat([x[..., :half] * c - x[..., half:2 * half] * s_, x[..., half:2 * half] * c + x[..., :half] * s_, x[..., 2 * half:]], dim=-1)
    assert torch.allclose(mine, plain.rotate(x, pos, rot), atol=1e-6)


def _context(batch=None, kv=None, state=None):
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import LayerContext
    return LayerContext(batch=batch, kernels=TorchKernels(wide=True), workspace=Workspace("cpu"), kv=kv, state=state)


def _weights(specs, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    return {name: (torch.randn(spec.shape, generator=g) * std + (1.0 if name.endswith("norm") else 0.0)).to(torch.bfloat16)
            for name, spec in specs.items()}


def _states(part, slots=3):
    return {name: torch.zeros((slots, *spec.shape), dtype=torch.float32) for name, spec in part.state_spec().items()}


def _scenario(segments, part, page_size=4):
    from helpers import paged_scenario
    spec = part.cache_spec() if hasattr(part, "cache_spec") else None
    batch, kv = paged_scenario(segments, num_kv_heads=spec.num_kv_heads if spec else 1, head_dim=spec.head_dim if spec else 4, page_size=page_size,
                               dtype=torch.float32, device="cpu", fill_history=False, window=spec.window if spec else None)
    if spec is not None and spec.v_head_dim != spec.head_dim:
        from kvcache_b200.parts.base import PagedKVView
        kv = PagedKVView(spec=spec, k_pages=kv.k_pages, v_pages=torch.zeros(*kv.k_pages.shape[:-1], spec.v_head_dim), block_table=kv.block_table,
                         page_size=page_size, writes=True)
    return batch, kv


@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=16, vdim=24, window=7, dims=8), dict(heads=3, kv_heads=3, dim=6, vdim=2, window=None, dims=6),
                                   dict(heads=2, kv_heads=1, dim=8, vdim=8, window=1, dims=None)])
def test_window_attention_part_alone(sizes):
    """A whole sequence, then the same cut in two, through the attention part with sharp scores against the plain function:
    per-head norms before the rotation, rotation of part of a head, the window's first and last key, the gate per head."""
    from kvcache_b200.parts.attention import GQAAttention
    from kvcache_b200.parts.position import RotaryHalf, WavelengthScaling
    T, W, eps, scale = 29, 40, 1e-5, 9.0
    rot = None if sizes["dims"] is None else {"base": 777.0, "dims": sizes["dims"], "scaling": {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 24}}
    rope = None if rot is None else RotaryHalf(rot["dims"], rot["base"], 64, WavelengthScaling(3.0, 1.0, 4.0, 24))
    part = GQAAttention(W, sizes["heads"], sizes["kv_heads"], sizes["dim"], qkv_bias=False, out_bias=False, position=rope, window=sizes["window"],
                        prefix="m.", dtype="float32", scale=scale, value_dim=sizes["vdim"], qk_norm_eps=eps, head_gate="g", names=("q", "k", "v", "o"))
    w = _weights(part.tensor_specs(), 3)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(4))
    m = dict(heads=sizes["heads"], kv_heads=sizes["kv_heads"], dim=sizes["dim"], vdim=sizes["vdim"], scale=scale)
    if sizes["window"]:
        m["mask"] = {"size": sizes["window"]}
    if rot:
        m["rot"] = rot
    want = plain.window_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", m, eps)
    if sizes["window"] and sizes["window"] > 1:   # one key more or one key less would show: the scores are sharp
        wider = plain.window_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", dict(m, mask={"size": sizes["window"] + 1}), eps)
        narrower = plain.window_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", dict(m, mask={"size": sizes["window"] - 1}), eps)
        assert (wider - want).abs().max() > 0.02 * want.abs().max() and (narrower - want).abs().max() > 0.02 * want.abs().max()
    batch, kv = _scenario([(0, T)], part)
    assert_close(part.forward(x, _context(batch, kv)), want, 1e-5)
    second, kv = _scenario([(11, T - 11)], part)           # the pages of the whole request; the first step fills part of them
    first, _ = _scenario([(0, 11)], part)
    got = [part.forward(x[:11], _context(first, kv)).clone()]
    got.append(part.forward(x[11:], _context(second, kv)))
    assert_close(torch.cat(got), want, 1e-5, "cut in two")


@pytest.mark.parametrize("sizes", [dict(heads=3, dim=8, vdim=16, rank=6, tau=4.0), dict(heads=1, dim=40, vdim=3, rank=1, tau=32.0),
                                   dict(heads=2, dim=33, vdim=70, rank=5, tau=1.0)])
def test_gated_linear_attention_part_alone(sizes):
    """Whole, and cut into pieces that carry the state in a slot, against the plain recurrence; a state left in another
    slot does not leak."""
    from kvcache_b200.parts.recurrent import GatedLinearAttention
    T, W, eps = 23, 48, 1e-5
    part = GatedLinearAttention(W, sizes["heads"], sizes["dim"], sizes["vdim"], sizes["rank"], sizes["tau"], eps=eps, prefix="m.", dtype="float32")
    w = _weights(part.tensor_specs(), 5)
    w["m.a2.b"] = (torch.randn(sizes["heads"] * sizes["dim"], generator=torch.Generator().manual_seed(6)) * 2 + 2).to(torch.bfloat16)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(7))
    want = plain.gated_linear_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", dict(sizes), eps)
    states = _states(part)
    states["memory"][0].fill_(7.0)                                    # another request's state
    batch, _ = _scenario([(0, T)], part)
    batch.seg_slot[0] = 1
    assert_close(part.forward(x, _context(batch, state=states)), want, 1e-5)
    assert bool((states["memory"][0] == 7.0).all()) and float(states["memory"][1].abs().max()) > 0
    states, got, at = _states(part), [], 0
    for n in (1, 2, 9, 1, 10):
        batch, _ = _scenario([(at, n)], part)
        batch.seg_slot[0] = 2
        got.append(part.forward(x[at:at + n], _context(batch, state=states)).clone())
        at += n
    assert_close(torch.cat(got), want, 1e-5, "in pieces")


@pytest.mark.parametrize("sizes", [dict(heads=2, dim=24, vdim=16, gate_cap=8.0), dict(heads=1, dim=5, vdim=40, gate_cap=1.0),
                                   dict(heads=5, dim=8, vdim=8, gate_cap=12.0)])
def test_matrix_memory_part_alone(sizes):
    """The running maximum starts at 0 (not at the first input gate), the denominator's floor e^{-m} acts in the first
    tokens, and strong gates (biases of several units) keep the exponentials in range; whole and in pieces."""
    from kvcache_b200.parts.recurrent import MatrixMemory
    T, W, eps = 26, 48, 1e-5
    part = MatrixMemory(W, sizes["heads"], sizes["dim"], sizes["vdim"], sizes["gate_cap"], eps=eps, prefix="m.", dtype="float32")
    w = _weights(part.tensor_specs(), 8)
    g = torch.Generator().manual_seed(9)
    w["m.i.b"] = (torch.randn(sizes["heads"], generator=g) * 3 - 2).to(torch.bfloat16)      # mostly negative: m stays 0 for a while
    w["m.f.b"] = (torch.randn(sizes["heads"], generator=g) * 3 + 2).to(torch.bfloat16)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(10)) * 2
    wd = {k: v.double() for k, v in w.items()}
    want = plain.matrix_memory(x.double(), wd, "m.", dict(sizes), eps)
    states = _states(part)
    batch, _ = _scenario([(0, T)], part)
    assert_close(part.forward(x, _context(batch, state=states)), want, 1e-5)
    states, got, at = _states(part), [], 0
    for n in (2, 1, 1, 12, 10):
        batch, _ = _scenario([(at, n)], part)
        batch.seg_slot[0] = 1
        got.append(part.forward(x[at:at + n], _context(batch, state=states)).clone())
        at += n
    assert_close(torch.cat(got), want, 1e-5, "in pieces")


def test_parallel_mixer_sums_its_sides_with_their_scales():
    from kvcache_b200.parts.attention import GQAAttention
    from kvcache_b200.parts.recurrent import GatedLinearAttention, ParallelMixer
    T, W, eps = 17, 32, 1e-6
    left = GQAAttention(W, 2, 1, 8, qkv_bias=False, out_bias=False, position=None, window=5, prefix="m.left.", dtype="float32", scale=0.5,
                        value_dim=12, qk_norm_eps=eps, head_gate="g", names=("q", "k", "v", "o"))
    right = GatedLinearAttention(W, 3, 4, 8, 2, 2.0, eps=eps, prefix="m.right.", dtype="float32")
    part = ParallelMixer(W, left, right, 1.7, 0.4, "float32")
    w = _weights(part.tensor_specs(), 11)
    part.bind(w, torch.device("cpu"))
    assert part.cache_spec().window == 5 and set(part.state_spec()) == {"right.memory"}
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(12))
    m = {"left": dict(heads=2, kv_heads=1, dim=8, vdim=12, scale=0.5, mask={"size": 5}), "right": dict(heads=3, dim=4, vdim=8, tau=2.0),
         "left_scale": 1.7, "right_scale": 0.4}
    want = plain.parallel_mixer(x.double(), {k: v.double() for k, v in w.items()}, "m.", m, eps)
    batch, kv = _scenario([(0, T)], part)
    states = {"right.memory": torch.zeros(2, 3, 4, 8)}
    assert_close(part.forward(x, _context(batch, kv, states)), want, 1e-5)


@pytest.mark.parametrize("E,top,shared", [(5, 2, (24, 0.75)), (3, 1, None), (4, 4, (8, 2.0))])
def test_routed_feed_forward_part_alone(E, top, shared):
    """Weights are the softmax over ALL experts at the chosen ones (they do not sum to 1); the clamp acts (inputs large
    enough to pass both limits); the shared expert has a size and a limit of its own."""
    from kvcache_b200.parts.feedforward import GatedMLP, RoutedMLP
    T, W, F, limit = 9, 40, 24, 0.6
    sh = None if shared is None else GatedMLP(W, shared[0], activation="clamped_swiglu", limit=shared[1], prefix="f.shared.", dtype="float32",
                                              names=("gate", "up", "down"))
    part = RoutedMLP(W, F, E, top, activation="clamped_swiglu", limit=limit, scores="all", prefix="f.", dtype="float32", shared=sh)
    w = _weights(part.tensor_specs(), 5)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(6))
    wd = {k: v.double() for k, v in w.items()}
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": F, "limit": limit}}
    if shared is not None:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    assert_close(part.forward(x, _context()), plain.feed_forward(x.double(), wd, "f.", mlp), 1e-5)
    gate = plain.linear(x.double(), wd["f.e0.gate"])
    assert bool((gate > limit).any()) and bool((plain.linear(x.double(), wd["f.e0.up"]) < -limit).any())
    if top < E:
        _, weight = plain.route(x.double(), wd, "f.", mlp)
        assert float(weight.sum(dim=-1).max()) < 0.999
    with pytest.raises(ValueError, match="limit"):
        RoutedMLP(W, F, E, top, activation="clamped_swiglu", prefix="f.", dtype="float32")


def test_pair_embedding_carries_the_previous_token_across_steps_and_slots():
    from kvcache_b200.parts.embedding import HashedBigramEmbedding
    W, V, bigram = 8, 300, {"buckets": 11, "mul_prev": 7, "mul_cur": 3}
    part = HashedBigramEmbedding(W, 11, 7, 3, V, "bigram", "float32")
    table = torch.randn(12, W, generator=torch.Generator().manual_seed(1))
    part.bind({"bigram": table}, torch.device("cpu"))
    a, b = random_tokens(V, 9, 1), random_tokens(V, 6, 2)
    state = {"previous_token": torch.tensor([5, 77, 123], dtype=torch.int32)}       # what earlier requests left in the slots

    def run(segments):   # [(slot, start, tokens)]
        batch, _ = _scenario([(s, len(t)) for _, s, t in segments], part)
        batch.token_ids.copy_(torch.tensor([x for _, _, t in segments for x in t], dtype=torch.int32))
        batch.seg_slot.copy_(torch.tensor([slot for slot, _, _ in segments], dtype=torch.int32))
        h = torch.zeros(batch.num_tokens, W)
        part.forward(h, _context(batch, state=state))
        return h

    first = run([(2, 0, a[:4]), (0, 0, b[:1])])
    second = run([(0, 1, b[1:]), (2, 4, a[4:5])])
    third = run([(2, 5, a[5:])])
    want_a, want_b = table[plain.bigram_rows(a, bigram)], table[plain.bigram_rows(b, bigram)]
    assert plain.bigram_rows(a, bigram)[0] == 11
    assert torch.equal(torch.cat([first[:4], second[5:], third]), want_a) and torch.equal(torch.cat([first[4:], second[:5]]), want_b)
    assert state["previous_token"].tolist() == [b[-1], 77, a[-1]]


def test_residual_stream_after_every_layer(tmp_path):
    """Layer by layer: a model cut after k layers (its final norm and head replaced by the identity) gives the plain
    implementation's residual stream after layer k."""
    folder = make_libulorn_folder(tmp_path, "A")
    config, weights = plain.read_folder(folder)
    tokens = random_tokens(config["vocab"], 19, 3)
    streams = plain.residual_streams(config, weights, tokens)
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    from kvcache_b200.engine.runner import ModelRunner, StepEntry
    for k in range(1, len(streams) + 1):
        model = load_model(folder, "float32", "cpu", max_positions=64)
        model.schedule = model.schedule[:k]
        model._writers = {c.cache: c.layer for c in model.schedule}
        model.final_norm.weight = torch.ones(model.width)
        model.final_norm.eps = 0.0
        model.head = torch.eye(model.width)
        model.vocab_size = model.width
        cache = CacheManager(model.cache_entries(), page_size=8, num_pages=16, max_slots=1, max_tokens_per_request=64, dtype="float32", device="cpu")
        runner = ModelRunner(model, cache, TorchKernels(wide=True), max_tokens_per_step=64)
        got = runner.step([StepEntry(cache.admit(), tokens, list(range(len(tokens))))]).double()
        want = streams[k - 1]
        want = want / torch.sqrt((want * want).mean(dim=-1, keepdim=True))
        assert_close(got, want, 1e-5, f"after layer {k}")


# ---- the model in the engine ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_its_first_tokens(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 75, 1)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.whole(runner, tokens), want, REL)
    assert runner.cache.used_pages() == 0
    for n in (1, 2, 3):                 # a sequence's first tokens alone: the pair table's last row, empty states, m = 0
        assert_close(replay_modes.whole(runner, tokens[:n]), want[:n], REL, f"first {n}")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token_decoding(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 70, 2)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], REL)
    assert_close(replay_modes.portions(runner, tokens, [1] * 70), want, REL, "every token alone")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_down_to_two_tokens(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 101, 3)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22]), want, REL)
    assert_close(replay_modes.portions(runner, tokens, [40, 2, 2, 5, 52]), want, REL)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path, name):
    """Unequal requests beside one another against each alone; a and b end and d and e take their slots, whose
    states (matrices, normalisers, maxima, previous tokens) must start from nothing."""
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, name, num_pages=replay_modes.mixed_pool_tokens() // page)
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, tokens in seqs.items():
        assert_close(got[k], plain.logits_of(config, weights, tokens), REL, k)


@pytest.mark.parametrize("name", ["A", "D"])
def test_sharp_attention_at_the_windows_edges_in_prompts_and_decoding(tmp_path, name):
    """With the score scale multiplied, the softmax of most heads rests on single keys: a window one token too wide or too
    narrow, or a key lost at a page border or at the start of a portion, changes the logits by far more than the tolerance."""
    runner, config, weights = _runner(tmp_path, name, sharpen=60.0, max_tokens_per_step=256, max_tokens_per_request=256)
    tokens = random_tokens(config["vocab"], 150, 5)
    want = plain.logits_of(config, weights, tokens)
    for delta in (-1, 1):
        other = copy.deepcopy(config)
        for layer in other["layers"]:
            if layer["type"] == "parallel":
                layer["mixer"]["left"]["mask"]["size"] += delta
        assert (plain.logits_of(other, weights, tokens) - want).abs().max() > 0.02 * want.abs().max()
    assert_close(replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 17]), want, 1e-3)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], 1e-3)
    assert_close(replay_modes.portions(runner, tokens, [100] + [1] * 50), want, 1e-3, "the window passes over decoded tokens")


def test_long_decoding_keeps_the_states_in_range(tmp_path):
    runner, config, weights = _runner(tmp_path, "A", max_tokens_per_step=512, max_tokens_per_request=512)
    tokens = random_tokens(config["vocab"], 300, 6)
    got = replay_modes.portions(runner, tokens, [20] + [1] * 280)
    assert_close(got, plain.logits_of(config, weights, tokens), REL)


# ---- generation through the entry point and the scheduler -------------------------------------------------------------
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_plain(tmp_path, name):
    from kvcache_b200 import LLM, SamplingParams
    folder = make_libulorn_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40)]
    llm = LLM(folder, kernels=TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=40, max_running=3,
              max_tokens_per_step=48, chunk_size=16, use_graphs=False)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    for prompt, out in zip(prompts, got):
        assert out == plain.greedy_generate(config, weights, prompt, 6)
    assert llm.core.cache.used_pages() == 0 and llm.last_stats.finished == len(prompts)
