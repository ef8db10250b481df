"""The Kakipel model in the engine (step function, cache, scheduler) on the CPU stand-in kernels against the plain
implementation; its parts alone against the plain functions; its configuration."""
import math

import pytest
import torch

import plain_kakipel as plain
import replay_modes
from helpers import assert_close, make_runner, random_tokens
from kakipel_configs import CONFIGS, PAGE_SIZE, config_dict, make_kakipel_folder
from torch_kernels import TorchKernels

REL = 1e-4


def _runner(tmp_path, name, num_pages=64, sharpen=1.0, **kw):
    folder = make_kakipel_folder(tmp_path, name, sharpen=sharpen)
    runner = make_runner(folder, TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=num_pages, **kw)
    config, weights = plain.read_folder(folder)
    return runner, config, weights


# ---- configuration --------------------------------------------------------------------------------------------------
def test_config_round_trip_and_layer_runs():
    from kvcache_b200.config import config_from_dict
    for name in CONFIGS:
        c = config_from_dict(config_dict(name))
        assert config_from_dict(c.to_dict()) == c
        assert [(i, t, o) for i, t, o in c.layer_runs()] == plain.layer_runs(config_dict(name))
    c = config_from_dict(config_dict("R"))
    assert [i for i, _, _ in c.layer_runs()] == [0, 1, 1, 1, 2] and [t for _, t, _ in c.layer_runs()] == [None, 0, 1, 2, None]
    assert c.layers[0].mlp.experts == 9 and c.layers[1].mlp.kind == "dense" and c.layers[0].mixer.rot.scaling.factor == 2.5


def test_config_faults_are_all_reported():
    from kvcache_b200.config import ConfigError, config_from_dict
    bad = config_dict("P")
    bad["layers"][0]["mixer"].pop("kv_rank")
    bad["layers"][1]["mlp"]["router"]["top"] = 9
    bad["layers"][2]["type"] = "convolution"
    bad["loop"] = {"start": 2, "stop": 1, "times": 2}
    del bad["norm"]
    with pytest.raises(ConfigError) as info:
        config_from_dict(bad)
    text = str(info.value)
    for piece in ("kv_rank", "top 9", "convolution", "no run of the 3 layers", "norm"):
        assert piece in text, piece


def test_model_as_data(tmp_path):
    """Every layer run has a cache entry of its own; entries of equal geometry share a group; the looped layers'
    passes open with the loop entry and its pass number."""
    from kvcache_b200.engine.loading import load_model
    model = load_model(make_kakipel_folder(tmp_path, "P"), "float32", "cpu", max_positions=64)
    assert [(c.layer, c.cache, c.before) for c in model.schedule] == [(0, 0, (0, 0)), (1, 1, None), (0, 2, (0, 1)), (1, 3, None), (2, 4, None)]
    entries = model.cache_entries()
    assert len(entries) == 5 and all(e.kv.num_kv_heads == 1 and e.kv.head_dim == 48 and e.kv.value_dim == 0 and e.state is None for e in entries)
    q = load_model(make_kakipel_folder(tmp_path, "Q"), "float32", "cpu", max_positions=64)
    assert [e.kv.head_dim for e in q.cache_entries()] == [72, 32, 16, 72] and q.stream_parts == []


def test_checkpoint_may_carry_norms_of_an_absent_feed_forward(tmp_path):
    """Tensors that the configuration gives no use - the second pair of norms of a layer without feed-forward - are left
    alone; any other extra tensor is still an error."""
    import os
    from kvcache_b200.engine.loading import load_model
    from kvcache_b200.weights import SafetensorsFile, WeightError, write_safetensors
    folder = make_kakipel_folder(tmp_path, "P")
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    tensors["l2.norm2"], tensors["l2.norm2b"] = torch.ones(64), torch.ones(64)
    write_safetensors(path, tensors)
    assert len(load_model(folder, "float32", "cpu", max_positions=32).schedule) == 5
    tensors["l2.mlp.gate"] = torch.ones(8, 64)
    write_safetensors(path, tensors)
    with pytest.raises(WeightError, match="l2.mlp.gate"):
        load_model(folder, "float32", "cpu", max_positions=32)


def test_cache_holds_one_row_per_token_and_no_values(tmp_path):
    from kvcache_b200.cache import CacheManager
    from kvcache_b200.engine.loading import load_model
    model = load_model(make_kakipel_folder(tmp_path, "Q"), "float32", "cpu", max_positions=64)
    cache = CacheManager(model.cache_entries(), page_size=16, num_pages=8, max_slots=2, max_tokens_per_request=64, dtype="float32", device="cpu")
    assert len(cache.groups) == 3 and sorted(len(g.cache_ids) for g in cache.groups) == [1, 1, 2]
    assert all(g.v_pool.numel() == 0 for g in cache.groups)
    assert cache.kv_bytes_per_token() == 4 * (72 + 32 + 16 + 72)


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("rot", [{"base": 300000.0, "dims": 28, "scaling": {"factor": 2.5, "original": 128, "fast": 24.0, "slow": 1.5}},
                                 {"base": 100.0, "dims": 6}, {"base": 3000.0, "dims": 12, "scaling": {"factor": 3.0, "original": 48, "fast": 4.0, "slow": 0.5}},
                                 {"base": 10000.0, "dims": 64, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}])
def test_rotation_tables(rot):
    from kvcache_b200.parts.position import RampScaling, RotaryHalf
    s = rot.get("scaling")
    part = RotaryHalf(rot["dims"], rot["base"], 300, None if s is None else RampScaling(s["factor"], s["original"], s["fast"], s["slow"]))
    part.bind({}, torch.device("cpu"))
    table = part.rotation()
    freq, gain = plain.rotation_frequencies(rot)
    assert torch.allclose(torch.from_numpy(part.frequencies()), freq, rtol=1e-12, atol=0)
    pos = torch.tensor([0, 1, 17, 255, 299])
    x = torch.randn(5, 3, rot["dims"] + 4, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    half = rot["dims"] // 2
    c, s_ = table.cos[pos].double()[:, None, :], table.sin[pos].double()[:, None, :]
    mine = torch.cat([x[..., :half] * c - x[..., half:2 * half] * s_, x[..., half:2 * half] * c + x[..., :half] * s_, x[..., 2 * half:]], dim=-1)
    assert torch.allclose(mine, plain.rotate(x, pos, rot), atol=1e-6)
    if s is not None:
        assert abs(float(table.cos[0, 0]) - gain) < 1e-6 and gain == pytest.approx(0.1 * math.log(s["factor"]) + 1)
        assert not torch.allclose(freq, plain.rotation_frequencies({"base": rot["base"], "dims": rot["dims"]})[0])


def _context(batch=None, kv=None, embedded=None):
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import LayerContext
    return LayerContext(batch=batch, kernels=TorchKernels(wide=True), workspace=Workspace("cpu"), kv=kv, embedded=embedded)


def _weights(specs, seed, std=0.3):
    g = torch.Generator().manual_seed(seed)
    return {name: (torch.randn(spec.shape, generator=g) * std + (1.0 if name.endswith("norm") else 0.0)).to(torch.bfloat16)
            for name, spec in specs.items()}


@pytest.mark.parametrize("sizes", [dict(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=32), dict(heads=1, dim=6, rot_dim=4, vdim=2, kv_rank=10, q_rank=3)])
def test_latent_attention_part_alone(sizes):
    """A whole sequence through the mixer (queries taken to the latent's space, one shared key row per token in the
    cache) against the plain function, which expands every token's keys and values per head."""
    from helpers import paged_scenario
    from kvcache_b200.parts.latent_attention import LatentAttention
    from kvcache_b200.parts.position import RampScaling, RotaryHalf
    T, W, eps, scale = 21, 56, 1e-5, 0.7
    rot = {"base": 777.0, "dims": sizes["rot_dim"], "scaling": {"factor": 2.5, "original": 16, "fast": 2.0, "slow": 0.5}}
    rope = RotaryHalf(rot["dims"], rot["base"], 64, RampScaling(2.5, 16, 2.0, 0.5))
    part = LatentAttention(W, sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"], sizes["q_rank"], scale=scale,
                           eps=eps, position=rope, prefix="m.", dtype="float32")
    w = _weights(part.tensor_specs(), 3)
    part.bind(w, torch.device("cpu"))
    spec = part.cache_spec()
    assert (spec.num_kv_heads, spec.head_dim, spec.value_dim) == (1, sizes["kv_rank"] + sizes["rot_dim"], 0) and part.state_spec() is None
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(4))
    batch, kv = paged_scenario([(0, T)], num_kv_heads=1, head_dim=spec.head_dim, page_size=4, dtype=torch.float32, device="cpu", fill_history=False)
    got = part.forward(x, _context(batch, kv))
    want = plain.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, "m.", dict(sizes, scale=scale, rot=rot), eps)
    assert_close(got, want, 1e-5)


@pytest.mark.parametrize("E,top", [(5, 2), (3, 1), (4, 4)])
def test_routed_feed_forward_part_alone(E, top):
    from kvcache_b200.parts.feedforward import RoutedMLP
    T, W, F = 9, 40, 24
    part = RoutedMLP(W, F, E, top, activation="relu2", prefix="f.", dtype="float32")
    w = _weights(part.tensor_specs(), 5)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(T, W, generator=torch.Generator().manual_seed(6))
    got = part.forward(x, _context())
    want = plain.routed_ff(x.double(), {k: v.double() for k, v in w.items()}, "f.", {"router": {"experts": E, "top": top}})
    assert_close(got, want, 1e-5)
    with pytest.raises(ValueError, match="activation"):
        RoutedMLP(W, F, E, top, activation="silu", prefix="f.", dtype="float32")


def test_dense_feed_forward_takes_its_names():
    from kvcache_b200.parts.feedforward import GatedMLP
    part = GatedMLP(40, 56, activation="silu", prefix="l0.mlp.", dtype="float32", names=("gate", "up", "down"))
    assert set(part.tensor_specs()) == {"l0.mlp.gate", "l0.mlp.up", "l0.mlp.down"}
    w = _weights(part.tensor_specs(), 7)
    part.bind(w, torch.device("cpu"))
    x = torch.randn(5, 40, generator=torch.Generator().manual_seed(8))
    assert_close(part.forward(x, _context()), plain.dense_ff(x.double(), {k: v.double() for k, v in w.items()}, "l0.mlp."), 1e-5)


def test_normalised_adds_and_loop_entry():
    """h += post(delta) folded into the next norm; the loop entry: h = Win [h + post(delta); x0] + step[t]."""
    from kvcache_b200.parts.base import NormedDelta
    from kvcache_b200.parts.norm import RMSNorm
    from kvcache_b200.parts.stream import LoopEntry
    g = torch.Generator().manual_seed(9)
    T, W = 6, 24
    post, pre = RMSNorm(W, 1e-5, "post"), RMSNorm(W, 1e-6, "pre")
    wn = {"post": 1 + 0.2 * torch.randn(W, generator=g), "pre": 1 + 0.2 * torch.randn(W, generator=g)}
    post.bind(wn, torch.device("cpu"))
    pre.bind(wn, torch.device("cpu"))
    h, delta = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g) * 4
    want_h = h.double() + plain.rms_norm(delta.double(), wn["post"].double(), 1e-5)
    mine, out = h.clone(), torch.zeros(T, W)
    pre.add_norm(mine, NormedDelta(delta, post), out, _context())
    assert_close(mine, want_h, 1e-6)
    assert_close(out, plain.rms_norm(want_h, wn["pre"].double(), 1e-6), 1e-6)
    rows = torch.tensor([4, 1], dtype=torch.int32)
    mine, out = h.clone(), torch.zeros(2, W)
    pre.add_norm(mine, NormedDelta(delta, post), out, _context(), rows=rows)
    assert torch.equal(mine, h)
    assert_close(out, plain.rms_norm(want_h, wn["pre"].double(), 1e-6)[rows.long()], 1e-6)

    entry = LoopEntry(W, 3, "loop.in", "loop.step", "float32")
    w = {"loop.in": torch.randn(W, 2 * W, generator=g) * 0.2, "loop.step": torch.randn(3, W, generator=g)}
    entry.bind(w, torch.device("cpu"))
    x0 = torch.randn(T, W, generator=g)
    for t in (0, 2):
        mine = h.clone()
        assert entry.forward(mine, NormedDelta(delta, post), _context(embedded=x0), t) is None
        want = plain.linear(torch.cat([want_h, x0.double()], dim=-1), w["loop.in"].double()) + w["loop.step"][t].double()
        assert_close(mine, want, 1e-6)


def test_residual_stream_after_every_layer_run(tmp_path):
    """Layer by layer: a model cut after k layer runs (its final norm and head replaced by the identity) gives the
    plain implementation's residual stream after run k."""
    folder = make_kakipel_folder(tmp_path, "P")
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
        assert_close(got, want, 1e-5, f"after layer run {k}")


# ---- the model in the engine ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 75, 1)
    assert_close(replay_modes.whole(runner, tokens), plain.logits_of(config, weights, tokens), REL)
    assert runner.cache.used_pages() == 0


@pytest.mark.parametrize("name", list(CONFIGS))
def test_decode_one_by_one(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 70, 2)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), plain.logits_of(config, weights, tokens)[-33:], REL)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_down_to_two_tokens(tmp_path, name):
    runner, config, weights = _runner(tmp_path, name)
    tokens = random_tokens(config["vocab"], 101, 3)
    got = replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22])
    assert_close(got, plain.logits_of(config, weights, tokens), REL)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path, name):
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, name, num_pages=replay_modes.mixed_pool_tokens() // page)
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, tokens in seqs.items():
        assert_close(got[k], plain.logits_of(config, weights, tokens), REL, k)


@pytest.mark.parametrize("name", ["P", "R"])
def test_sharp_attention_sees_far_keys_in_prompts_and_decoding(tmp_path, name):
    """With the score scale multiplied, the softmax of most heads rests on single keys far back: a key lost at a
    page border, in a portion's first rows or in decoding changes the logits by far more than the tolerance."""
    runner, config, weights = _runner(tmp_path, name, sharpen=40.0, max_tokens_per_step=256, max_tokens_per_request=256)
    tokens = random_tokens(config["vocab"], 150, 5)
    want = plain.logits_of(config, weights, tokens)
    blurred = plain.logits_of(dict(config, layers=[dict(l, mixer=dict(l["mixer"], scale=l["mixer"]["scale"] / 40.0)) for l in config["layers"]]),
                              weights, tokens)
    assert (want - blurred).abs().max() > 0.05 * want.abs().max()         # the sharpening matters
    # Sharp scores magnify float32 rounding as well; a lost key costs several per cent.
    assert_close(replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 17]), want, 1e-3)
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], 1e-3)


# ---- generation through the entry point and the scheduler -------------------------------------------------------------
@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_matches_plain(tmp_path, name):
    from kvcache_b200 import LLM, SamplingParams
    folder = make_kakipel_folder(tmp_path, name)
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40)]
    llm = LLM(folder, kernels=TorchKernels(), dtype="float32", device="cpu", page_size=PAGE_SIZE[name], num_pages=40, max_running=3,
              max_tokens_per_step=48, chunk_size=16, use_graphs=False)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    for prompt, out in zip(prompts, got):
        assert out == plain.greedy_generate(config, weights, prompt, 6)
    assert llm.core.cache.used_pages() == 0 and llm.last_stats.finished == len(prompts)
