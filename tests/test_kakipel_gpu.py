"""The Kakipel model through the engine on the GPU, in float32 and bfloat16, against the plain implementation: the four
ways of cutting and batching, sharp attention over many pages, long decoding, CUDA graphs, generation, trace replay."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_kakipel as plain
import replay_modes
from helpers import assert_close, make_runner, random_tokens
from kakipel_configs import CONFIGS, PAGE_SIZE, make_kakipel_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 1e-4, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


def _runner(tmp_path, kernels, name, dtype, num_pages=64, sharpen=1.0, **kw):
    folder = make_kakipel_folder(tmp_path, name, sharpen=sharpen, dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
    runner = make_runner(folder, kernels, dtype=dtype, device=DEV, page_size=PAGE_SIZE[name], num_pages=num_pages, **kw)
    config, weights = plain.read_folder(folder)
    return runner, config, weights


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_four_ways_of_cutting(tmp_path, kernels, name, dtype):
    page = PAGE_SIZE[name]
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, num_pages=max(replay_modes.mixed_pool_tokens(), 128) // page)
    tokens = random_tokens(config["vocab"], 101, 3)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.whole(runner, tokens), want, REL[dtype], "whole")
    assert_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], REL[dtype], "decode")
    assert_close(replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22]), want, REL[dtype], "portions")
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, toks in seqs.items():
        assert_close(got[k], plain.logits_of(config, weights, toks), REL[dtype], f"mixed {k}")
    kernels.check_errors()


@pytest.mark.parametrize("name", ["P", "R"])
def test_float32_rows_do_not_depend_on_the_batch_or_the_cut(tmp_path, kernels, name):
    """In float32 a position's logits are bit for bit the same alone, beside other requests, and in portions."""
    runner, config, _ = _runner(tmp_path, kernels, name, "float32")
    from kvcache_b200.engine.runner import StepEntry
    a, b = random_tokens(config["vocab"], 40, 1), random_tokens(config["vocab"], 23, 2)
    alone = replay_modes.whole(runner, a)
    sa, sb = runner.cache.admit(), runner.cache.admit()
    first = runner.step([StepEntry(sb, b[:20], []), StepEntry(sa, a[:17], list(range(17)))]).clone()
    second = runner.step([StepEntry(sa, a[17:], list(range(23))), StepEntry(sb, b[20:21], [0])]).clone()
    assert torch.equal(torch.cat([first, second[:23]]), alone)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sharp_attention_over_many_pages(tmp_path, kernels, dtype):
    """Sharpened scores make single far keys carry the softmax: keys at page borders, in a portion's first rows and far
    behind a decoded token all have to be found.  Sharp scores magnify rounding too: bfloat16, whose rounding of a score
    40 times larger would itself change which key wins, is sharpened less and held to less (single far keys in bfloat16
    are met at kernel level, where one key takes all the weight by construction)."""
    sharpen, rel = (40.0, 2e-3) if dtype == "float32" else (5.0, 0.08)
    runner, config, weights = _runner(tmp_path, kernels, "P", dtype, sharpen=sharpen, num_pages=96, max_tokens_per_step=640,
                                      max_tokens_per_request=640)
    tokens = random_tokens(config["vocab"], 600, 5)
    want = plain.logits_of(config, weights, tokens)
    got = replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 259, 8, 168, 32])
    assert_close(got, want, rel)
    got = replay_modes.last_32_one_by_one(runner, tokens)
    assert_close(got, want[-33:], rel)


def test_one_far_key_carries_a_decoded_token(tmp_path, kernels):
    """bfloat16: the cache rows are overwritten so that one head's query at the decoded position matches exactly one key
    far back; the mixer's result for that head must be that row's value expansion."""
    from helpers import batch_to, clone_kv, paged_scenario
    from kvcache_b200.engine.workspace import Workspace
    H, D, Dv, page = 5, 80, 64, 16
    batch, kv = paged_scenario([(1000, 1), (37, 1)], num_kv_heads=1, head_dim=D, page_size=page, dtype=torch.bfloat16, device="cpu", seed=2)
    q = (torch.randn(2, H * D, generator=torch.Generator().manual_seed(3)) * 0.02).to(torch.bfloat16)
    for head, far in ((0, 15), (3, 16), (4, 511)):          # last row of a page, first row of the next, the middle
        key = kv.k_pages[int(kv.block_table[0, far // page]), 0, far % page].float()
        q.view(2, H, D)[0, head] = (key * 3.0).to(torch.bfloat16)
    got = torch.zeros(2, H * Dv, dtype=torch.bfloat16, device=DEV)
    kernels.latent_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, H, Dv, 1.0, Workspace(DEV))
    for head, far in ((0, 15), (3, 16), (4, 511)):
        key = kv.k_pages[int(kv.block_table[0, far // page]), 0, far % page]
        assert_close(got.view(2, H, Dv)[0, head], key[:Dv], 2e-2, f"key {far}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_under_graphs_matches_eager_and_plain(tmp_path, kernels, dtype):
    """200 tokens decoded one by one, two requests at a time, replayed from CUDA graphs: the routed feed-forward's
    launches do not depend on the routing, so the recorded step serves every later one."""
    from kvcache_b200.engine.runner import StepEntry
    runner, config, weights = _runner(tmp_path, kernels, "R", dtype, num_pages=40, max_slots=2)
    runner.use_graphs = True
    seqs = [random_tokens(config["vocab"], 230, 7), random_tokens(config["vocab"], 215, 8)]
    slots = [runner.cache.admit(), runner.cache.admit()]
    runner.step([StepEntry(slots[0], seqs[0][:30], []), StepEntry(slots[1], seqs[1][:15], [])])
    last = None
    for i in range(200):
        entries = [StepEntry(slots[0], [seqs[0][30 + i]], [0], (0.0, 0, i)), StepEntry(slots[1], [seqs[1][15 + i]], [0], (0.0, 0, i))]
        last, tokens = runner.step(entries, sample=True)
    assert runner.graph_replays >= 190
    kernels.check_errors()
    for r in range(2):
        want = plain.logits_of(config, weights, seqs[r])[-1]
        assert_close(last[r], want, REL[dtype], f"request {r}")
        assert int(tokens[r]) == int(torch.argmax(last[r]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(tmp_path, kernels, dtype):
    from kvcache_b200 import LLM, SamplingParams
    folder = make_kakipel_folder(tmp_path, "Q", dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40, 63)]
    llm = LLM(folder, kernels=kernels, dtype=dtype, device=DEV, page_size=16, num_pages=40, max_running=3, max_tokens_per_step=48,
              chunk_size=16, use_graphs=True)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    assert llm.core.cache.used_pages() == 0
    for prompt, out in zip(prompts, got):
        # Every generated token is the plain implementation's first choice given the same tokens, wherever that choice is clear.
        logits = plain.logits_of(config, weights, list(prompt) + out)
        for i, token in enumerate(out):
            row = logits[len(prompt) - 1 + i]
            best = torch.topk(row, 2).values
            if float(best[0] - best[1]) > (1e-3 if dtype == "float32" else 0.05) * float(row.abs().max()):
                assert token == int(torch.argmax(row)), (len(prompt), i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Kakipel folder: mixed steps, requests that pause, pages used again."""
    folder = make_kakipel_folder(tmp_path, "P", dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
    config, weights = plain.read_folder(folder)
    seqs = {k: random_tokens(config["vocab"], n, 20 + i) for i, (k, n) in enumerate([("a", 70), ("b", 33), ("c", 64), ("d", 50)])}
    plan = [([("a", 40), ("b", 2)], []), ([("b", 1), ("c", 64)], ["c"]), ([("a", 1), ("b", 30)], ["b"]), ([("d", 50), ("a", 29)], ["a", "d"])]
    done = {k: 0 for k in seqs}
    lines, expected = [], []
    for step, (parts, end) in enumerate(plan):
        entries = []
        for k, n in parts:
            entries.append({"id": k, "tokens": seqs[k][done[k]:done[k] + n], "want": list(range(n))})
            expected.append((step, k, done[k], n))
            done[k] += n
        lines.append(json.dumps({"step": step, "entries": entries, "end": end}))
    out = os.path.join(str(tmp_path), "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                           "--max-tokens", "192", "--max-live", "4"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(plan))]
    want = {k: plain.logits_of(config, weights, seqs[k]) for k in seqs}
    for step in range(len(plan)):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, config["vocab"]))
        at = 0
        for s, k, lo, n in expected:
            if s == step:
                assert_close(got[at:at + n], want[k][lo:lo + n], REL[dtype], f"step {step} {k}")
                at += n
