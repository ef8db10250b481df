"""The Libulorn model through the engine on the GPU, in float32 and bfloat16, against the plain implementation, and every
CUDA operator it brought alone against the plain PyTorch statement of the same operator (tests/torch_kernels.py)."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_libulorn as plain
import replay_modes
from helpers import assert_close, batch_to, clone_kv, make_runner, paged_scenario, random_tokens
from libulorn_configs import CONFIGS, PAGE_SIZE, make_libulorn_folder
from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REL = {"float32": 1e-4, "bfloat16": 3e-2}
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _spread(config, weights, tokens, want):
    """What rounding alone does to each position's logits: the plain implementation with every product's rows and
    results rounded to bfloat16, against itself without."""
    with plain.rounding(torch.bfloat16):
        return (plain.logits_of(config, weights, tokens) - want).abs().max(dim=1).values


def assert_model_close(got, want, dtype, what="", spread=None, rel=None):
    """float32: within `rel` of the largest logit.  bfloat16: a layer of this design divides what a sublayer returns by
    its root mean square, so a position where a sublayer's sums nearly cancel magnifies rounding however it is computed,
    and which positions those are changes with the places of the roundings (the same position read 0.05, 0.26 and 0.61
    of error with three ways of rounding, and the same alone as in a batch).  The errors are therefore held, as a
    distribution, to 4 times what rounding alone does in the plain implementation (`spread`: its per-position errors
    over the whole sequence): the k-th largest error against the k-th largest of the spread (floor: 1 % of the largest
    logit) except for the largest 2 % of them (at least one), the median position within 2 %, and no position beyond
    30 % - a lost key, state or token moves many positions by as much as the logits themselves."""
    if dtype == "float32":
        return assert_close(got, want, rel or REL[dtype], what)
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    scale = float(want.abs().max())
    floor = 0.01 * scale
    err = (got - want).abs().max(dim=1).values
    assert float(err.max()) <= 0.3 * scale, f"{what}: error {float(err.max()):.3e} of {scale:.3e}"
    if len(err) < 16:
        limit = max(4.0 * float(spread.max()), 4.0 * floor)
        assert float(err.max()) <= limit, f"{what}: error {float(err.max()):.3e}, spread {float(spread.max()):.3e}"
        return
    e, sp = torch.sort(err, descending=True).values, torch.sort(spread, descending=True).values
    like = sp[(torch.arange(len(e)) * len(sp) // len(e))]
    over = e > 4.0 * torch.clamp(like, min=floor)
    over[:max(1, len(e) // 50)] = False
    assert not bool(over.any()), f"{what}: the {int(over.nonzero()[0])}-th largest error {float(e[over][0]):.3e} against {float(like[over][0]):.3e}"
    assert float(err.median()) <= 0.02 * scale, f"{what}: median error {float(err.median()):.3e} of {scale:.3e}"


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def _segments_batch(segments, slots):
    batch, _ = paged_scenario(segments, num_kv_heads=1, head_dim=4, page_size=4, dtype=torch.float32, device="cpu", fill_history=False)
    batch.seg_slot.copy_(torch.tensor(slots, dtype=torch.int32))
    return batch


# ---- operators alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,D,Dv", [(3, 8, 16), (1, 33, 3), (2, 40, 70), (4, 64, 64), (2, 128, 128), (1, 200, 256), (5, 32, 32)])
def test_gated_linear_scan(kernels, H, D, Dv):
    """Prompts, a portion that continues a state, single tokens, states of other slots untouched; then every row alone,
    which must give the same bits as the rows together."""
    segments, slots = [(0, 19), (50, 1), (7, 6), (3, 1)], [2, 0, 3, 5]
    batch = _segments_batch(segments, slots)
    T = batch.num_tokens
    P = 2 * H * D + H * Dv + 5
    proj, z = _rand(T, P, seed=1), _rand(T, H * D, seed=2, scale=2.0) + 2.0
    memory = _rand(6, H, D, Dv, seed=3)
    ref_mem, ref_out = memory.clone(), torch.zeros(T, H * Dv)
    TorchKernels(wide=True).gated_linear_scan(proj, (3, 3 + H * D, 3 + 2 * H * D), z, 7.0, 0.3, batch, ref_mem, ref_out, H, D, Dv)
    got_mem, got_out = memory.clone().to(DEV), torch.zeros(T, H * Dv, device=DEV)
    kernels.gated_linear_scan(proj.to(DEV), (3, 3 + H * D, 3 + 2 * H * D), z.to(DEV), 7.0, 0.3, batch_to(batch, DEV), got_mem, got_out, H, D, Dv)
    assert_close(got_out, ref_out, 2e-5, "read-out")
    assert_close(got_mem, ref_mem, 2e-5, "states")
    assert torch.equal(got_mem[1].cpu(), memory[1]) and torch.equal(got_mem[4].cpu(), memory[4])
    one_mem, one_out = memory.clone().to(DEV), torch.zeros(T, H * Dv, device=DEV)
    at = 0
    for (start, n), slot in zip(segments, slots):
        for i in range(n):
            single = _segments_batch([(start + i, 1)], [slot])
            kernels.gated_linear_scan(proj[at:at + 1].to(DEV).contiguous(), (3, 3 + H * D, 3 + 2 * H * D), z[at:at + 1].to(DEV).contiguous(), 7.0, 0.3,
                                      batch_to(single, DEV), one_mem, one_out[at:at + 1], H, D, Dv)
            at += 1
    assert torch.equal(one_out, got_out) and torch.equal(one_mem, got_mem)


@pytest.mark.parametrize("H,D,Dv", [(2, 24, 16), (1, 5, 40), (5, 8, 8), (4, 48, 64), (2, 128, 128), (1, 256, 96)])
def test_matrix_memory_scan(kernels, H, D, Dv):
    segments, slots = [(0, 23), (9, 1), (0, 1), (4, 8)], [1, 3, 0, 2]
    batch = _segments_batch(segments, slots)
    T = batch.num_tokens
    cols = (0, H * D, 2 * H * D, 2 * H * D + H * Dv + 2, 2 * H * D + H * Dv + 2 + H)
    P = cols[4] + H + 1
    proj = _rand(T, P, seed=4)
    proj[:, cols[3]:cols[3] + H] = proj[:, cols[3]:cols[3] + H] * 4 - 3        # input gates mostly below the maximum's start, some far above
    proj[:, cols[4]:cols[4] + H] = proj[:, cols[4]:cols[4] + H] * 4 + 2
    memory, normalizer, maximum = _rand(4, H, D, Dv, seed=5), _rand(4, H, D, seed=6), _rand(4, H, seed=7).abs()
    for t in (memory, normalizer, maximum):
        t[0].zero_(), t[1].zero_()                                            # requests that begin in this step
    ref = [memory.clone(), normalizer.clone(), maximum.clone(), torch.zeros(T, H * Dv)]
    TorchKernels(wide=True).matrix_memory_scan(proj, cols, 6.0, 0.25, 1e-6, batch, ref[0], ref[1], ref[2], ref[3], H, D, Dv)
    got = [memory.clone().to(DEV), normalizer.clone().to(DEV), maximum.clone().to(DEV), torch.zeros(T, H * Dv, device=DEV)]
    kernels.matrix_memory_scan(proj.to(DEV), cols, 6.0, 0.25, 1e-6, batch_to(batch, DEV), got[0], got[1], got[2], got[3], H, D, Dv)
    for g, r, what in zip(got, ref, ("memory", "normalizer", "maximum", "read-out")):
        assert_close(g, r, 5e-5, what)


@pytest.mark.parametrize("mode", ["channel decay", "exponential gates"])
@pytest.mark.parametrize("H,D,Dv", [(3, 24, 16), (2, 64, 128), (1, 130, 40)])
def test_scans_in_chunks_side_by_side(kernels, mode, H, D, Dv):
    """A step with a long segment is scanned in chunks of 64 tokens that run side by side: segments that end inside a
    chunk, at a chunk's edge, one token after it, a single token and a segment that continues a state, against the
    plain statement; the states left in the slots too."""
    from kvcache_b200.engine.workspace import Workspace
    segments, slots = [(0, 300), (40, 1), (7, 128), (0, 65), (3, 63)], [1, 4, 0, 2, 5]
    batch = _segments_batch(segments, slots)
    assert batch.max_q_len >= kernels.SCAN_CHUNK_MIN_ROWS
    T = batch.num_tokens
    cols = (0, H * D, 2 * H * D, 2 * H * D + H * Dv, 2 * H * D + H * Dv + H)
    proj = _rand(T, cols[4] + H, seed=4)
    proj[:, cols[3]:cols[3] + H] = proj[:, cols[3]:cols[3] + H] * 3 - 2
    proj[:, cols[4]:cols[4] + H] = proj[:, cols[4]:cols[4] + H] * 3 + 3
    z = _rand(T, H * D, seed=2, scale=2.0) + 3.0
    memory, normalizer, maximum = _rand(6, H, D, Dv, seed=5), _rand(6, H, D, seed=6), _rand(6, H, seed=7).abs()
    for t in (memory, normalizer, maximum):
        t[1].zero_(), t[2].zero_()
    ref = [memory.clone(), normalizer.clone(), maximum.clone(), torch.zeros(T, H * Dv)]
    got = [memory.clone().to(DEV), normalizer.clone().to(DEV), maximum.clone().to(DEV), torch.zeros(T, H * Dv, device=DEV)]
    if mode == "channel decay":
        TorchKernels(wide=True).gated_linear_scan(proj, cols[:3], z, 5.0, 0.3, batch, ref[0], ref[3], H, D, Dv)
        kernels.gated_linear_scan(proj.to(DEV), cols[:3], z.to(DEV), 5.0, 0.3, batch_to(batch, DEV), got[0], got[3], H, D, Dv, Workspace(DEV))
    else:
        TorchKernels(wide=True).matrix_memory_scan(proj, cols, 6.0, 0.25, 1e-6, batch, ref[0], ref[1], ref[2], ref[3], H, D, Dv)
        kernels.matrix_memory_scan(proj.to(DEV), cols, 6.0, 0.25, 1e-6, batch_to(batch, DEV), got[0], got[1], got[2], got[3], H, D, Dv, Workspace(DEV))
    for g, r, what in zip(got, ref, ("memory", "normalizer", "maximum", "read-out")):
        assert_close(g, r, 5e-5, what)
    assert torch.equal(got[0][3].cpu(), memory[3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Dv,per_head,act", [(3, 16, False, "silu"), (2, 70, True, "sigmoid"), (1, 3, True, "silu"), (16, 128, False, "sigmoid")])
def test_head_norm_gate_and_head_gate(kernels, dtype, H, Dv, per_head, act):
    T = 11
    o, proj = _rand(T, H * Dv, seed=1, scale=3.0), _rand(T, H * Dv + 9, seed=2)
    w = 1 + _rand(H * Dv if per_head else Dv, seed=3, scale=0.3)
    ref, got = torch.zeros(T, 2 * H * Dv + 4, dtype=dtype), torch.zeros(T, 2 * H * Dv + 4, dtype=dtype, device=DEV)
    TorchKernels(wide=True).head_norm_gate(o, w, 1e-5, (proj, 5), act, 0.9, ref, H * Dv + 2, H, Dv)
    kernels.head_norm_gate(o.to(DEV), w.to(DEV), 1e-5, (proj.to(DEV), 5), act, 0.9, got, H * Dv + 2, H, Dv)
    x, g = _rand(T, H * Dv, dtype=dtype, seed=4), _rand(T, H + 6, dtype=dtype, seed=5, scale=2.0)
    TorchKernels(wide=True).head_gate(x, (g, 3), H, Dv, 1.2, ref, 1)
    kernels.head_gate(x.to(DEV), (g.to(DEV), 3), H, Dv, 1.2, got, 1)
    assert_close(got, ref, TOL[dtype])
    assert float(ref[:, 0].abs().max()) == 0 and float(got[:, 0].abs().max()) == 0            # columns of neither stay as they were


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,Dv,rot", [(4, 2, 16, 24, 8), (3, 3, 6, 2, 6), (6, 3, 80, 160, 40), (5, 1, 40, 40, 0), (2, 2, 128, 64, 128)])
def test_norm_rotation_append_with_two_sizes(kernels, dtype, Hq, Hkv, D, Dv, rot):
    from kvcache_b200.parts.base import PagedKVSpec, PagedKVView
    segments = [(0, 5), (37, 1), (14, 20)]
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=8, dtype=dtype, device="cpu", seed=3)
    kv = PagedKVView(spec=PagedKVSpec(Hkv, D, None, None if Dv == D else Dv), k_pages=kv.k_pages, v_pages=_rand(*kv.k_pages.shape[:-1], Dv, dtype=dtype, seed=4),
                     block_table=kv.block_table, page_size=8, writes=True)
    T = batch.num_tokens
    qkv = _rand(T, (Hq + Hkv) * D + Hkv * Dv + Hq, dtype=dtype, seed=7, scale=2.0)
    qw, kw = 1 + _rand(D, seed=8, scale=0.3), 1 + _rand(D, seed=9, scale=0.3)
    cos = sin = None
    if rot:
        ang = torch.arange(64, dtype=torch.float64)[:, None] * torch.logspace(0, -3, rot // 2, dtype=torch.float64)[None, :]
        cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    dev = lambda t: None if t is None else t.to(DEV)
    for norms in ((qw, kw), (None, None)):
        ref_kv, ref_q = clone_kv(kv), torch.zeros(T, Hq * D, dtype=dtype)
        TorchKernels(wide=True).qkv_rope_append(qkv, None, cos, sin, batch, ref_kv, ref_q, Hq, q_norm=norms[0], k_norm=norms[1], norm_eps=1e-5)
        got_kv, got_q = clone_kv(kv, DEV), torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        kernels.qkv_rope_append(qkv.to(DEV), None, dev(cos), dev(sin), batch_to(batch, DEV), got_kv, got_q, Hq, q_norm=dev(norms[0]), k_norm=dev(norms[1]),
                                norm_eps=1e-5)
        kernels.check_errors()
        assert_close(got_q, ref_q, TOL[dtype], "queries")
        assert_close(got_kv.k_pages, ref_kv.k_pages, TOL[dtype], "key pages")
        assert_close(got_kv.v_pages, ref_kv.v_pages, TOL[dtype], "value pages")
        untouched = ref_kv.v_pages == kv.v_pages
        assert torch.equal(got_kv.v_pages.cpu()[untouched], kv.v_pages[untouched])


def _two_size_scenario(segments, Hkv, D, Dv, page, dtype, window, seed=2):
    from kvcache_b200.parts.base import PagedKVSpec, PagedKVView
    batch, kv = paged_scenario(segments, num_kv_heads=Hkv, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=seed, window=window)
    return batch, PagedKVView(spec=PagedKVSpec(Hkv, D, window, None if Dv == D else Dv), k_pages=kv.k_pages,
                              v_pages=_rand(*kv.k_pages.shape[:-1], Dv, dtype=dtype, seed=seed + 1), block_table=kv.block_table, page_size=page, writes=True)


def test_keys_stored_as_wide_as_values(kernels):
    """bfloat16, keys of 40 numbers beside values of 64: queries and keys are stored 64 wide with zeros after their
    numbers, and the attention kernels for one size give what the plain statement gives for two."""
    from kvcache_b200.engine.workspace import Workspace
    from kvcache_b200.parts.base import PagedKVSpec, PagedKVView
    Hq, Hkv, D, Dv, dtype = 6, 2, 40, 64, torch.bfloat16
    segments = [(0, 45), (130, 1), (30, 20)]
    batch, two = _two_size_scenario(segments, Hkv, D, Dv, 8, dtype, 33)
    two.k_pages.zero_(), two.v_pages.zero_()
    wide = PagedKVView(spec=PagedKVSpec(Hkv, Dv, 33), k_pages=torch.zeros(*two.k_pages.shape[:-1], Dv, dtype=dtype), v_pages=two.v_pages.clone(),
                       block_table=two.block_table, page_size=8, writes=True)
    T = batch.num_tokens
    # The cached part of every request first (as one prompt each), then the step itself; both layouts side by side.
    history = [(0, s) for s, _ in segments if s > 0]
    hist_batch, _ = _two_size_scenario(history, Hkv, D, Dv, 8, dtype, 33)
    rows = [i for i, (s, _) in enumerate(segments) if s > 0]
    hist_table = two.block_table[rows]
    qw, kw = 1 + _rand(D, seed=8, scale=0.3), 1 + _rand(D, seed=9, scale=0.3)
    ang = torch.arange(200, dtype=torch.float64)[:, None] * torch.logspace(0, -3, 8, dtype=torch.float64)[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    outs = {}
    for name, view in (("two", two), ("wide", wide)):
        for step_batch, table, seed in ((hist_batch, hist_table, 1), (batch, two.block_table, 2)):
            n = step_batch.num_tokens
            qkv = _rand(n, (Hq + Hkv) * D + Hkv * Dv + Hq, dtype=dtype, seed=seed, scale=2.0)
            kv = PagedKVView(spec=view.spec, k_pages=view.k_pages, v_pages=view.v_pages, block_table=table, page_size=8, writes=True)
            if name == "two":
                q = torch.zeros(n, Hq * D, dtype=dtype)
                TorchKernels(wide=True).qkv_rope_append(qkv, None, cos, sin, step_batch, kv, q, Hq, q_norm=qw, k_norm=kw, norm_eps=1e-5)
                out = torch.zeros(n, Hq * Dv, dtype=dtype)
                TorchKernels(wide=True).paged_attention(q, step_batch, kv, out, Hq, 0.3)
            else:
                dev_kv = PagedKVView(spec=view.spec, k_pages=view.k_pages.to(DEV), v_pages=view.v_pages.to(DEV), block_table=table.to(DEV), page_size=8, writes=True)
                q = torch.zeros(n, Hq * Dv, dtype=dtype, device=DEV)
                kernels.qkv_rope_append(qkv.to(DEV), None, cos.to(DEV), sin.to(DEV), batch_to(step_batch, DEV), dev_kv, q, Hq, q_norm=qw.to(DEV),
                                        k_norm=kw.to(DEV), norm_eps=1e-5, key_dim=D)
                assert float(q.view(n, Hq, Dv)[:, :, D:].abs().max()) == 0
                out = torch.zeros(n, Hq * Dv, dtype=dtype, device=DEV)
                kernels.paged_attention(q, batch_to(step_batch, DEV), dev_kv, out, Hq, 0.3, Workspace(DEV))
                view.k_pages.copy_(dev_kv.k_pages.cpu()), view.v_pages.copy_(dev_kv.v_pages.cpu())
            outs[name] = out
    kernels.check_errors()
    assert_close(outs["wide"], outs["two"], 2e-2)
    assert_close(wide.k_pages[..., :D], two.k_pages, 2e-2, "keys")
    assert float(wide.k_pages[..., D:].abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,Dv,window", [(4, 2, 16, 24, 11), (3, 3, 6, 2, None), (6, 3, 80, 160, 70), (5, 1, 40, 72, 16), (2, 1, 64, 32, 1)])
def test_attention_with_values_of_another_size_than_keys(kernels, dtype, Hq, Hkv, D, Dv, window):
    from kvcache_b200.engine.workspace import Workspace
    batch, kv = _two_size_scenario([(0, 45), (130, 1), (30, 20), (16, 1)], Hkv, D, Dv, 8, dtype, window)
    T = batch.num_tokens
    q = _rand(T, Hq * D, dtype=dtype, seed=5, scale=0.5)
    ref, got = torch.zeros(T, Hq * Dv, dtype=dtype), torch.zeros(T, Hq * Dv, dtype=dtype, device=DEV)
    TorchKernels(wide=True).paged_attention(q, batch, kv, ref, Hq, 0.4)
    kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 0.4, Workspace(DEV))
    kernels.check_errors()
    assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decoded", [True, False])
def test_one_key_at_the_windows_edge_takes_all_the_weight(kernels, dtype, decoded):
    """The query of one head matches the key at the window's first position (a page's first row for the decoded token, a
    page's last row for the prompt's row) and nothing else: the head's result is that key's value.  Then it matches the
    key one position further back still more strongly: that key is outside the window, and the result must not move
    towards its value."""
    from kvcache_b200.engine.workspace import Workspace
    Hq, Hkv, D, Dv, page, window = 4, 2, 32, 48, 8, 25
    segments = [(200, 1), (5, 1)] if decoded else [(190, 11), (0, 6)]
    batch, kv = _two_size_scenario(segments, Hkv, D, Dv, page, dtype, window, seed=6)
    T = batch.num_tokens
    row, pos = (0, 200) if decoded else (9, 199)
    inside, outside = pos - window + 1, pos - window
    assert inside % page == (0 if decoded else page - 1)
    key = lambda p, hk: kv.k_pages[int(kv.block_table[0, p // page]), hk, p % page]
    val = lambda p, hk: kv.v_pages[int(kv.block_table[0, p // page]), hk, p % page]
    for head, strong_outside in ((1, False), (2, True)):
        q = (_rand(T, Hq * D, seed=7) * 0.01).to(dtype)
        hk = head // (Hq // Hkv)
        q.view(T, Hq, D)[row, head] = (key(inside, hk).float() * 2.0).to(dtype)
        if strong_outside:
            key(outside, hk).copy_((key(inside, hk).float() * 1.5).to(dtype))
        got = torch.zeros(T, Hq * Dv, dtype=dtype, device=DEV)
        kernels.paged_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, Hq, 1.0, Workspace(DEV))
        assert_close(got.view(T, Hq, Dv)[row, head], val(inside, hk), 2e-2 if dtype == torch.bfloat16 else 1e-4, f"head {head}")


@pytest.mark.parametrize("E,top", [(5, 2), (16, 1), (3, 3), (70, 4)])
def test_route_top_with_scores_over_all_experts(kernels, E, top):
    T = 37
    logits = _rand(T, E, seed=1, scale=2.0)
    ref_c, ref_s = torch.zeros(T, top, dtype=torch.int32), torch.zeros(T, top)
    TorchKernels(wide=True).route_top(logits, ref_c, ref_s, scores="all")
    got_c, got_s = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV)
    kernels.route_top(logits.to(DEV), got_c, got_s, scores="all")
    assert torch.equal(got_c.cpu(), ref_c)
    assert_close(got_s, ref_s, 1e-5)
    if top < E:
        assert float(got_s.sum(dim=-1).max()) < 1.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,F,H,with_base", [(9, 5, 2, 24, 40, True), (3, 4, 4, 16, 96, False), (300, 9, 3, 40, 120, True), (1, 12, 2, 48, 192, True),
                                                   (700, 6, 2, 72, 128, True), (1100, 16, 1, 200, 64, False)])
def test_routed_experts_with_the_clamped_gated_activation(kernels, dtype, T, E, top, F, H, with_base):
    from kvcache_b200.engine.workspace import Workspace
    x = _rand(T, H, dtype=dtype, seed=1)
    w_up, w_down = _rand(E, 2 * F, H, dtype=dtype, seed=2, scale=0.3), _rand(E, H, F, dtype=dtype, seed=3, scale=0.3)
    g = torch.Generator().manual_seed(4)
    chosen = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    share = torch.rand(T, top, generator=g)
    base = _rand(T, H, dtype=dtype, seed=5) if with_base else None
    ref, got = torch.zeros(T, H, dtype=dtype), torch.zeros(T, H, dtype=dtype, device=DEV)
    TorchKernels(wide=True).routed_experts(x, w_up, w_down, chosen, share, ref, "clamped_swiglu", None, limit=0.8, base=base)
    kernels.routed_experts(x.to(DEV), w_up.to(DEV), w_down.to(DEV), chosen.to(DEV), share.to(DEV), got, "clamped_swiglu", Workspace(DEV),
                           limit=0.8, base=None if base is None else base.to(DEV))
    assert_close(got, ref, TOL[dtype] * 2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_clamped_gated_activation(kernels, dtype, interleaved):
    T, I = 13, 40
    gu = _rand(T, 2 * I, dtype=dtype, seed=1, scale=2.0)
    ref, got = torch.zeros(T, I, dtype=dtype), torch.zeros(T, I, dtype=dtype, device=DEV)
    TorchKernels(wide=True).silu_mul(gu, ref, interleaved, "clamped_swiglu", 1.25)
    kernels.silu_mul(gu.to(DEV), got, interleaved, "clamped_swiglu", 1.25)
    assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("M", [1, 8, 16, 24, 32, 200])
def test_gated_product_with_the_clamped_activation_in_its_epilogue(kernels, M):
    """bfloat16, gate and up rows interleaved in eights: up to 16 rows the register kernel, up to 32 the weight-streaming
    tcgen05 kernel, beyond that product and activation kernel - all against the plain statement."""
    from kvcache_b200.engine.workspace import Workspace
    K, I, limit = 256, 320, 0.9
    x = _rand(M, K, dtype=torch.bfloat16, seed=1)
    gate, up = _rand(I, K, dtype=torch.bfloat16, seed=2, scale=0.1), _rand(I, K, dtype=torch.bfloat16, seed=3, scale=0.1)
    w = torch.stack([gate.view(-1, 8, K), up.view(-1, 8, K)], dim=1).reshape(-1, K).contiguous()
    ref, got = torch.zeros(M, I, dtype=torch.bfloat16), torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    TorchKernels(wide=True).gate_up_act(x, w, ref, None, True, "clamped_swiglu", limit)
    before = dict(kernels.launch_counts)
    kernels.gate_up_act(x.to(DEV), w.to(DEV), got, Workspace(DEV), True, activation="clamped_swiglu", limit=limit)
    kernels.check_errors()
    launched = {k: v - before.get(k, 0) for k, v in kernels.launch_counts.items() if v != before.get(k, 0)}
    assert launched == ({"gemm_skinny": 1} if M <= 16 else {"gemm_wstream": 1} if M <= 32 else launched) and (M <= 32 or "silu_mul" in launched)
    assert_close(got, ref, 2e-2)
    g = (x.double() @ gate.double().t())
    assert bool((g > limit).any()) and bool(((x.double() @ up.double().t()) < -limit).any())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding(kernels, dtype):
    """Rows that open a portion take the slot's previous token, position 0 takes the table's last row, tokens that the
    step before left on the device are read there; afterwards the slots hold their segments' last tokens."""
    W, V, buckets = 24, 5000, 11
    batch = _segments_batch([(0, 4), (9, 1), (3, 5), (0, 1)], [2, 0, 3, 1])
    T = batch.num_tokens
    batch.token_ids.copy_(torch.tensor(random_tokens(V, T, 1), dtype=torch.int32))
    batch.token_src = torch.full((T,), -1, dtype=torch.int32)
    batch.token_src[4] = 1
    batch.last_tokens = torch.tensor([17, 4321, 5], dtype=torch.int32)
    table = _rand(buckets + 1, W, dtype=dtype, seed=2)
    previous = torch.tensor([4999, 7, 8, 1234, 9], dtype=torch.int32)
    h = _rand(T, W, seed=3)
    ref_h, ref_prev = h.clone(), previous.clone()
    TorchKernels().bigram_embed(table, batch, ref_prev, ref_h, buckets, 1000003, 31, V)
    got_h, got_prev = h.clone().to(DEV), previous.clone().to(DEV)
    kernels.bigram_embed(table.to(DEV), batch_to(batch, DEV), got_prev, got_h, buckets, 1000003, 31, V)
    assert torch.equal(got_prev.cpu(), ref_prev) and ref_prev.tolist()[0] == 4321 and ref_prev.tolist()[4] == 9
    assert_close(got_h, ref_h, 1e-6)


# ---- the model in the engine ------------------------------------------------------------------------------------------
def _runner(tmp_path, kernels, name, dtype, num_pages=64, sharpen=1.0, **kw):
    folder = make_libulorn_folder(tmp_path, name, sharpen=sharpen, dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
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
    spread = _spread(config, weights, tokens, want)
    assert_model_close(replay_modes.whole(runner, tokens), want, dtype, "whole", spread)
    assert_model_close(replay_modes.whole(runner, tokens[:1]), want[:1], dtype, "one token", spread)
    assert_model_close(replay_modes.last_32_one_by_one(runner, tokens), want[-33:], dtype, "decode", spread)
    assert_model_close(replay_modes.portions(runner, tokens, [2, 17, 3, 31, 2, 16, 8, 22]), want, dtype, "portions", spread)
    seqs = {k: random_tokens(config["vocab"], n, 10 + i) for i, (k, n) in enumerate(replay_modes.MIXED_LENGTHS)}
    got = replay_modes.mixed(runner, seqs)
    for k, toks in seqs.items():
        alone = plain.logits_of(config, weights, toks)
        assert_model_close(got[k], alone, dtype, f"mixed {k}", _spread(config, weights, toks, alone))
    kernels.check_errors()


@pytest.mark.parametrize("name", ["A", "C"])
def test_long_prompts_whose_states_are_scanned_in_chunks(tmp_path, kernels, name):
    """float32: a prompt long enough for the chunked scans, whole, in two long portions and beside another request."""
    runner, config, weights = _runner(tmp_path, kernels, name, "float32", num_pages=160, max_tokens_per_step=700, max_tokens_per_request=700)
    from kvcache_b200.engine.runner import StepEntry
    tokens, other = random_tokens(config["vocab"], 600, 11), random_tokens(config["vocab"], 90, 12)
    want = plain.logits_of(config, weights, tokens)
    assert_close(replay_modes.whole(runner, tokens), want, 2e-4, "whole")
    assert_close(replay_modes.portions(runner, tokens, [290, 310]), want, 2e-4, "two portions")
    sa, sb = runner.cache.admit(), runner.cache.admit()
    got = runner.step([StepEntry(sb, other[:60], []), StepEntry(sa, tokens[:333], list(range(333)))]).clone()
    more = runner.step([StepEntry(sa, tokens[333:], list(range(267))), StepEntry(sb, other[60:], [29])]).clone()
    assert_close(torch.cat([got, more[:267]]), want, 2e-4, "beside another request")
    assert_close(more[267:], plain.logits_of(config, weights, other)[-1:], 2e-4, "the other request")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_through_the_tensor_core_attention_with_keys_stored_wide(tmp_path, kernels, dtype):
    """Keys of 64 beside values of 128: in bfloat16 the cache entry is 128 wide and a portion of 384 rows and more runs
    on the tensor-memory attention kernel, shorter ones and decoded tokens on the other tensor-core kernels, all with
    the window; in float32 the two-size kernel.  Whole, in portions that straddle the kernels' row limit, then decoded."""
    runner, config, weights = _runner(tmp_path, kernels, "E", dtype, num_pages=48, max_tokens_per_step=640, max_tokens_per_request=640)
    spec = runner.model.blocks[0].mixer.cache_spec()
    assert (spec.head_dim, spec.v_head_dim) == ((128, 128) if dtype == "bfloat16" else (64, 128))
    tokens = random_tokens(config["vocab"], 520, 21)
    want = plain.logits_of(config, weights, tokens)
    spread = _spread(config, weights, tokens, want) if dtype == "bfloat16" else None
    assert_model_close(replay_modes.whole(runner, tokens), want, dtype, "whole", spread, 2e-4)
    assert_model_close(replay_modes.portions(runner, tokens, [400, 3, 100, 17]), want, dtype, "portions", spread, 2e-4)
    assert_model_close(replay_modes.portions(runner, tokens, [450] + [1] * 70), want, dtype, "decoded", spread, 2e-4)
    kernels.check_errors()


@pytest.mark.parametrize("name", ["A", "B"])
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
@pytest.mark.parametrize("name", ["A", "D"])
def test_sharp_attention_at_the_windows_edges(tmp_path, kernels, name, dtype):
    """Sharpened scores make single keys carry the softmax: a window one token off, or a key lost at a page border, in a
    portion's first rows or behind decoded tokens, shows.  bfloat16, whose rounding of much larger scores would itself
    change which key wins, is sharpened less (its single keys are met at kernel level)."""
    sharpen, rel = (60.0, 2e-3) if dtype == "float32" else (6.0, None)
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, sharpen=sharpen, num_pages=96, max_tokens_per_step=320, max_tokens_per_request=320)
    tokens = random_tokens(config["vocab"], 300, 5)
    want = plain.logits_of(config, weights, tokens)
    if dtype == "float32":
        other = copy.deepcopy(config)
        for layer in other["layers"]:
            if layer["type"] == "parallel":
                layer["mixer"]["left"]["mask"]["size"] -= 1
        assert (plain.logits_of(other, weights, tokens) - want).abs().max() > 10 * rel * want.abs().max()
    spread = _spread(config, weights, tokens, want) if dtype == "bfloat16" else None
    assert_model_close(replay_modes.portions(runner, tokens, [7, 2, 57, 64, 3, 135, 32]), want, dtype, "portions", spread, rel)
    assert_model_close(replay_modes.portions(runner, tokens, [230] + [1] * 70), want, dtype, "the window passes over decoded tokens", spread, rel)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_under_graphs_matches_plain(tmp_path, kernels, name, dtype):
    """200 tokens decoded one by one, two requests at a time, replayed from CUDA graphs: every state (matrices,
    normalisers, maxima, previous tokens, pages) moves exactly once a step."""
    from kvcache_b200.engine.runner import StepEntry
    runner, config, weights = _runner(tmp_path, kernels, name, dtype, num_pages=80, max_slots=2)
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
        want = plain.logits_of(config, weights, seqs[r])
        assert_model_close(last[r:r + 1], want[-1:], dtype, f"request {r}", _spread(config, weights, seqs[r], want))
        assert int(tokens[r]) == int(torch.argmax(last[r]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(tmp_path, kernels, dtype):
    """Through `LLM`, the scheduler and CUDA graphs; generated tokens feed the next step from the device, so the pair
    embedding reads its tokens there."""
    from kvcache_b200 import LLM, SamplingParams
    folder = make_libulorn_folder(tmp_path, "B", dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
    config, weights = plain.read_folder(folder)
    prompts = [random_tokens(config["vocab"], n, 40 + n) for n in (1, 9, 24, 40, 63)]
    llm = LLM(folder, kernels=kernels, dtype=dtype, device=DEV, page_size=16, num_pages=40, max_running=3, max_tokens_per_step=48,
              chunk_size=16, use_graphs=True)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True))
    assert llm.core.cache.used_pages() == 0
    for prompt, out in zip(prompts, got):
        logits = plain.logits_of(config, weights, list(prompt) + out)
        for i, token in enumerate(out):
            row = logits[len(prompt) - 1 + i]
            best = torch.topk(row, 2).values
            if float(best[0] - best[1]) > (1e-3 if dtype == "float32" else 0.05) * float(row.abs().max()):
                assert token == int(torch.argmax(row)), (len(prompt), i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(tmp_path, dtype):
    """bin/trace_run as a user runs it, on a Libulorn folder: mixed steps, requests that pause, pages and slots used again."""
    folder = make_libulorn_folder(tmp_path, "A", dtype=torch.bfloat16, all_experts=dtype == "bfloat16")
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
                           "--max-tokens", "192", "--max-live", "3"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(plan))]
    want = {k: plain.logits_of(config, weights, seqs[k]) for k in seqs}
    spread = {k: _spread(config, weights, seqs[k], want[k]) for k in seqs}
    for step in range(len(plan)):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, config["vocab"]))
        at = 0
        for s, k, lo, n in expected:
            if s == step:
                assert_model_close(got[at:at + n], want[k][lo:lo + n], dtype, f"step {step} {k}", spread[k])
                at += n
