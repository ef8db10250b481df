"""Every CUDA operator of the latent-attention, normalised-add and routed feed-forward parts alone, against the plain
PyTorch statement of the same operator (tests/torch_kernels.py, float64)."""
import numpy as np
import pytest
import torch

from helpers import assert_close, batch_to, clone_kv, paged_scenario
from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def kernels():
    from kvcache_b200.kernels.api import CudaKernels
    return CudaKernels(DEV)


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [192, 100, 1031])
@pytest.mark.parametrize("form", ["post+norm", "plain+norm", "post+cast+tail", "add only", "rows"])
def test_norm_add_rmsnorm(kernels, dtype, H, form):
    T = 7
    h = _rand(T, H, seed=1, scale=3.0)
    delta = _rand(T, H, dtype=dtype, seed=2, scale=5.0)
    dw, w = 1 + _rand(H, seed=3, scale=0.2), 1 + _rand(H, seed=4, scale=0.2)
    tail = _rand(T, H, seed=5)
    rows = torch.tensor([5, 0, 3], dtype=torch.int32)
    args = {"post+norm": (delta, dw, 1e-5, w, 1e-6, (T, H), None, None),
            "plain+norm": (delta, None, 0.0, w, 1e-6, (T, H), None, None),
            "post+cast+tail": (delta, dw, 1e-5, None, 0.0, (T, 2 * H), None, tail),
            "add only": (delta, dw, 1e-5, None, 0.0, None, None, None),
            "rows": (delta, dw, 1e-5, w, 1e-6, (3, H), rows, None)}[form]
    d, dwt, deps, wt, eps, out_shape, rws, tl = args
    ref_h, got_h = h.clone(), h.clone().to(DEV)
    ref_out = torch.zeros(out_shape, dtype=dtype) if out_shape else None
    got_out = torch.zeros(out_shape, dtype=dtype, device=DEV) if out_shape else None
    TorchKernels(wide=True).norm_add_rmsnorm(ref_h, d, dwt, deps, wt, eps, ref_out, rws, tl)
    dev = lambda t: None if t is None else t.to(DEV)
    kernels.norm_add_rmsnorm(got_h, dev(d), dev(dwt), deps, dev(wt), eps, got_out, dev(rws), dev(tl))
    kernels.check_errors()
    assert_close(got_h, ref_h, 2e-6, "h")
    if out_shape:
        assert_close(got_out, ref_out, TOL[dtype], "out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(128, 64, 32, 32), (24, 40, 16, 8), (96, 512, 64, 64)])
def test_latent_norm_rope_append(kernels, dtype, sizes):
    q_rank, kv_rank, rot_dim, rot_used = sizes
    segments = [(0, 5), (37, 1), (14, 20)]
    batch, kv = paged_scenario(segments, num_kv_heads=1, head_dim=kv_rank + rot_dim, page_size=8, dtype=dtype, device="cpu", seed=3)
    T = batch.num_tokens
    P = q_rank + kv_rank + rot_dim + 24
    proj = _rand(T, P, dtype=dtype, seed=7, scale=2.0)
    qw, kw = 1 + _rand(q_rank, seed=8, scale=0.3), 1 + _rand(kv_rank, seed=9, scale=0.3)
    ang = torch.arange(64, dtype=torch.float64)[:, None] * torch.logspace(0, -3, rot_used // 2, dtype=torch.float64)[None, :]
    cos, sin = (torch.cos(ang) * 1.07).float(), (torch.sin(ang) * 1.07).float()
    ref_kv, ref_cq = clone_kv(kv), torch.zeros(T, q_rank, dtype=dtype)
    TorchKernels(wide=True).latent_norm_rope_append(proj, q_rank, kv_rank, rot_dim, qw, kw, 1e-5, cos, sin, batch, ref_kv, ref_cq)
    got_kv, got_cq = clone_kv(kv, DEV), torch.zeros(T, q_rank, dtype=dtype, device=DEV)
    kernels.latent_norm_rope_append(proj.to(DEV), q_rank, kv_rank, rot_dim, qw.to(DEV), kw.to(DEV), 1e-5, cos.to(DEV), sin.to(DEV),
                                    batch_to(batch, DEV), got_kv, got_cq)
    kernels.check_errors()
    assert_close(got_cq, ref_cq, TOL[dtype], "query latent")
    assert_close(got_kv.k_pages, ref_kv.k_pages, TOL[dtype], "cache rows")
    # Rows of other positions were not touched.
    untouched = ref_kv.k_pages == kv.k_pages
    assert torch.equal(got_kv.k_pages.cpu()[untouched], kv.k_pages[untouched])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 9, 70])
@pytest.mark.parametrize("shape", [(8, 64, 64, 32), (3, 40, 24, 8), (5, 72, 130, 16)])    # heads, N, K, trailing columns
def test_head_linear(kernels, dtype, T, shape):
    H, N, K, R = shape
    x = _rand(T, H * (K + R), dtype=dtype, seed=1)
    w = _rand(H, N, K, dtype=dtype, seed=2, scale=K ** -0.5)
    positions = torch.arange(T, dtype=torch.int32) * 3 % 50
    ang = torch.arange(50, dtype=torch.float64)[:, None] * torch.logspace(0, -2, R // 2, dtype=torch.float64)[None, :]
    cos, sin = torch.cos(ang).float(), torch.sin(ang).float()
    gate = _rand(T, 10 + H * N, dtype=dtype, seed=3, scale=2.0)
    for form in ("rotate", "gate", "plain"):
        width = H * (N + R) if form == "rotate" else H * N
        xin = x if form == "rotate" else x.view(T, H, K + R)[:, :, :K].reshape(T, H * K).contiguous()
        ref, got = torch.zeros(T, width, dtype=dtype), torch.zeros(T, width, dtype=dtype, device=DEV)
        rot = (cos, sin, positions) if form == "rotate" else None
        g = (gate, 10) if form == "gate" else None
        TorchKernels(wide=True).head_linear(xin, w, ref, rotate=rot, gate=g)
        kernels.head_linear(xin.to(DEV), w.to(DEV), got, rotate=None if rot is None else tuple(t.to(DEV) for t in rot),
                            gate=None if g is None else (gate.to(DEV), 10))
        kernels.check_errors()
        assert_close(got, ref, TOL[dtype], form)


def _with_latent_plan(batch, segments, heads, blocks_wanted=None, kernels=None, dims=None):
    """Adds the work list of the tensor-core kernel over shared key rows to a hand-made batch: made for `blocks_wanted`
    blocks, under the name the kernel set looks it up by."""
    import dataclasses
    from kvcache_b200.kernels.latent_plan import LatentAttentionPlanner
    from kvcache_b200.parts.base import StepPlan
    wanted, tile = kernels._latent_plan_shape(*dims)
    name = LatentAttentionPlanner.plan_name(heads, wanted, tile)
    planner = LatentAttentionPlanner(heads, blocks_wanted or wanted, tile)
    planner.name = name
    arrays, counts = planner.plan(np.asarray([s for s, _ in segments]), np.asarray([n for _, n in segments]))
    plans = dict(batch.plans)
    plans[planner.name] = StepPlan({k: torch.tensor(np.array(v), dtype=torch.int32) for k, v in arrays.items()}, counts)
    return dataclasses.replace(batch, plans=plans)


FLASH_CASES = [dict(H=8, D=96, Dv=64, page=16), dict(H=3, D=40, Dv=24, page=8), dict(H=16, D=576, Dv=512, page=32),
               dict(H=5, D=88, Dv=72, page=16), dict(H=20, D=160, Dv=128, page=64), dict(H=1, D=72, Dv=56, page=16),
               dict(H=4, D=320, Dv=256, page=16)]
FLASH_SEGMENTS = {"decode": [(70, 1), (129, 1), (0, 1), (1000, 1)], "prompt": [(0, 333)], "portion": [(190, 67), (15, 2)],
                  "mixed": [(0, 33), (70, 1), (15, 2), (129, 1), (300, 130)]}


@pytest.mark.parametrize("wanted", [None, 4])
@pytest.mark.parametrize("kind", list(FLASH_SEGMENTS))
@pytest.mark.parametrize("case", FLASH_CASES)
def test_latent_attention_tensor_cores(kernels, case, kind, wanted):
    """The bfloat16 tensor-core kernel (tiles of (token, head) rows, splits over the keys added by a second kernel)
    against the plain statement, with and without splits."""
    H, D, Dv, page = case["H"], case["D"], case["Dv"], case["page"]
    segments = FLASH_SEGMENTS[kind]
    dtype = torch.bfloat16
    batch, kv = paged_scenario(segments, num_kv_heads=1, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=5)
    batch = _with_latent_plan(batch, segments, H, wanted, kernels, (D, Dv))
    T = batch.num_tokens
    q = _rand(T, H * D, dtype=dtype, seed=6)
    ref, got = torch.zeros(T, H * Dv, dtype=dtype), torch.full((T, H * Dv), 7.0, dtype=dtype, device=DEV)
    TorchKernels(wide=True).latent_attention(q, batch, kv, ref, H, Dv, D ** -0.5)
    from kvcache_b200.engine.workspace import Workspace
    before = kernels.launch_counts["latent_flash"]
    kernels.latent_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, H, Dv, D ** -0.5, Workspace(DEV))
    kernels.check_errors()
    assert kernels.launch_counts["latent_flash"] == before + 1
    assert_close(got, ref, TOL[dtype])


def test_latent_attention_tensor_cores_one_far_key(kernels):
    """One key takes all the weight of one (token, head) row: at a page border, in another split, in a prompt's portion."""
    H, D, Dv, page = 6, 96, 64, 16
    segments = [(900, 1), (0, 200)]
    dtype = torch.bfloat16
    batch, kv = paged_scenario(segments, num_kv_heads=1, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=9)
    batch = _with_latent_plan(batch, segments, H, None, kernels, (D, Dv))
    q = _rand(batch.num_tokens, H * D, dtype=dtype, seed=10, scale=0.02)
    probes = [(0, 0, 2, 15), (0, 0, 3, 16), (0, 0, 5, 640), (1, 150, 1, 63), (1, 199, 4, 64), (1, 77, 0, 77)]   # segment, token, head, key
    for seg, tok, head, key in probes:
        row = tok if seg == 1 else 0
        row += 1 if seg == 1 else 0
        k = kv.k_pages[int(kv.block_table[seg, key // page]), 0, key % page].float()
        q.view(-1, H, D)[row, head] = (k * 3.0).to(dtype)
    got = torch.zeros(batch.num_tokens, H * Dv, dtype=dtype, device=DEV)
    from kvcache_b200.engine.workspace import Workspace
    kernels.latent_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, H, Dv, 1.0, Workspace(DEV))
    for seg, tok, head, key in probes:
        row = tok + 1 if seg == 1 else 0
        k = kv.k_pages[int(kv.block_table[seg, key // page]), 0, key % page]
        assert_close(got.view(-1, H, Dv)[row, head], k[:Dv], 2e-2, f"segment {seg} token {tok} key {key}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", [dict(H=8, D=96, Dv=64, page=16), dict(H=3, D=40, Dv=24, page=8), dict(H=16, D=576, Dv=512, page=32)])
def test_latent_attention(kernels, dtype, case):
    H, D, Dv, page = case["H"], case["D"], case["Dv"], case["page"]
    segments = [(0, 33), (70, 1), (15, 2), (129, 1)]
    batch, kv = paged_scenario(segments, num_kv_heads=1, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=5)
    T = batch.num_tokens
    q = _rand(T, H * D, dtype=dtype, seed=6)
    ref, got = torch.zeros(T, H * Dv, dtype=dtype), torch.zeros(T, H * Dv, dtype=dtype, device=DEV)
    TorchKernels(wide=True).latent_attention(q, batch, kv, ref, H, Dv, D ** -0.5)
    from kvcache_b200.engine.workspace import Workspace
    kernels.latent_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, H, Dv, D ** -0.5, Workspace(DEV))
    kernels.check_errors()
    assert_close(got, ref, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_sees_one_far_key(kernels, dtype):
    """One key far back takes all the weight of one head's query: the result is that row's value."""
    H, D, Dv, page = 4, 48, 32, 8
    segments = [(600, 1), (0, 300)]
    batch, kv = paged_scenario(segments, num_kv_heads=1, head_dim=D, page_size=page, dtype=dtype, device="cpu", seed=9)
    q = _rand(batch.num_tokens, H * D, dtype=dtype, seed=10, scale=0.05)
    far_page, far_slot = int(kv.block_table[0, 3 // page]), 3 % page            # position 3 of the first request
    key = kv.k_pages[far_page, 0, far_slot].float()
    q.view(-1, H, D)[0, 2] = (key * 4.0).to(dtype)
    got = torch.zeros(batch.num_tokens, H * Dv, dtype=dtype, device=DEV)
    from kvcache_b200.engine.workspace import Workspace
    kernels.latent_attention(q.to(DEV), batch_to(batch, DEV), clone_kv(kv, DEV), got, H, Dv, 1.0, Workspace(DEV))
    assert_close(got.view(-1, H, Dv)[0, 2], key[:Dv].to(dtype), 2e-2 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("E,top", [(16, 2), (5, 1), (70, 7), (8, 8)])
def test_route_top(kernels, E, top):
    T = 37
    logits = _rand(T, E, seed=E)
    chosen, share = torch.zeros(T, top, dtype=torch.int32, device=DEV), torch.zeros(T, top, device=DEV)
    kernels.route_top(logits.to(DEV), chosen, share)
    best, which = torch.topk(logits, top, dim=-1)
    assert torch.equal(chosen.cpu().long(), which)
    assert_close(share, torch.softmax(best.double(), dim=-1), 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 200, 700])
@pytest.mark.parametrize("shape", [(16, 2, 64, 192), (5, 1, 40, 72), (6, 6, 24, 100), (7, 3, 328, 136)])      # experts, top, ff, width
def test_routed_experts(kernels, dtype, T, shape):
    """700 rows with two or more choices each reach the tensor-memory products (bfloat16, widths in steps of 8)."""
    E, top, F, H = shape
    x = _rand(T, H, dtype=dtype, seed=1)
    w_up, w_down = _rand(E, F, H, dtype=dtype, seed=2, scale=H ** -0.5), _rand(E, H, F, dtype=dtype, seed=3, scale=F ** -0.5)
    logits = _rand(T, E, seed=4)
    if E > 2:
        logits[:, 1] -= 100.0        # an expert that nobody chooses
    best, which = torch.topk(logits, top, dim=-1)
    chosen, share = which.to(torch.int32), torch.softmax(best, dim=-1)
    ref, got = torch.zeros(T, H, dtype=dtype), torch.zeros(T, H, dtype=dtype, device=DEV)
    TorchKernels(wide=True).routed_experts(x, w_up, w_down, chosen, share, ref, "relu2")
    from kvcache_b200.engine.workspace import Workspace
    kernels.routed_experts(x.to(DEV), w_up.to(DEV), w_down.to(DEV), chosen.to(DEV), share.to(DEV), got, "relu2", Workspace(DEV))
    kernels.check_errors()
    assert_close(got, ref, TOL[dtype])
