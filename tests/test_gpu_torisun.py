"""The Torisun design on the GPU against the plain implementation: single kernels, each mechanism in a model of its own,
every schedule in both precisions and with both kernel sets, constants that are one off (negative controls on the plain
implementation, then the engine with the right ones), the sink, decoding from the first token on through captured steps,
generation through the scheduler, the trace program."""
import json
import math
import os
import subprocess

import numpy as np
import pytest
import torch

from helpers import compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_portions, trace_whole
from plain_torisun import PlainTorisun, rms_norm, rotate, route, sink_softmax, visible, yarn_frequencies
from tiny_torisun import (ONLY_ATTENTION, TINY_A, TINY_B, TINY_C, WITH_DENSE, WITH_MOE, WITH_READER, layer, make_torisun_dir, mixer)
from torisun_cases import (TOL_F32, greedy_by_the_plain_model, reference_logits, replay_all_schedules, schedules, variant_dir)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


def _ops(kernels="fast"):
    from llmengine_b200.kernels.ops import CudaOps
    ops = CudaOps(torch.device(DEV))
    ops.choose_kernels(kernels)
    return ops


def _run(ops, record, batch):
    from llmengine_b200.engine.plan import Plan
    plan = Plan()
    record(plan)
    ops.compile(plan).run(batch)
    torch.cuda.synchronize()


def _bare(T):
    from llmengine_b200.engine.batch import StepBatch
    return StepBatch.bare(T, torch.device(DEV))


# ----------------------------------------------------------------------------- single kernels
@pytest.mark.parametrize("T,D", [(3, 40), (70, 256), (5, 4100)])
def test_postnorm_kernel(T, D):
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(T, D, generator=g) * 3, torch.randn(T, D, generator=g) * 5
    gain = (1 + 0.1 * torch.randn(D, generator=g))
    for gdt in (torch.float32, torch.bfloat16):
        gn = gain.to(gdt)
        want = x + rms_norm(y, gn.float(), 1e-5)
        xd, copy = x.to(DEV), torch.zeros(T + 2, D, dtype=torch.bfloat16, device=DEV)
        _run(ops, lambda p: p.postnorm(xd, y.to(DEV), gn.to(DEV), 1e-5, copy=copy), _bare(T))
        assert float((xd.cpu() - want).abs().max()) < 2e-5
        assert torch.equal(copy[:T].cpu(), xd.cpu().to(torch.bfloat16)) and float(copy[T:].abs().max()) == 0.0
    # in place, not added: x = norm(x); and the copy alone
    xd = x.to(DEV)
    _run(ops, lambda p: p.postnorm(xd, xd, gain.to(DEV), 1e-5, accumulate=False), _bare(T))
    assert float((xd.cpu() - rms_norm(x, gain, 1e-5)).abs().max()) < 2e-5
    c32 = torch.zeros(T, D, device=DEV)
    _run(ops, lambda p: p.postnorm(xd, None, None, 0.0, copy=c32), _bare(T))
    assert torch.equal(c32, xd)


def _clamped(z, inter, limit, slope=1.702):
    g, u = torch.clamp(z[:, :inter], max=limit), torch.clamp(z[:, inter:], -limit, limit)
    return g * torch.sigmoid(slope * g) * (u + 1.0)


@pytest.mark.parametrize("T,K,inter,linear", [(5, 40, 52, "auto"), (37, 40, 52, "auto"), (8, 64, 96, "auto"), (300, 64, 200, "tcgen05"),
                                              (260, 72, 40, "tcgen05")])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_clamped_gate_in_and_behind_the_product(dtype, tol, T, K, inter, linear):
    """The clamped activation as a kernel of its own, in the weight-streaming product's epilogue (a handful of tokens)
    and in the tcgen05 product's (many): the limit cuts gate and up, the slope and the + 1 are there."""
    ops = _ops()
    ops.choose("linear", linear)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, K, generator=g).to(dtype)
    w = (torch.randn(2 * inter, K, generator=g) / 3).to(dtype)
    gate_up = torch.zeros(T + 1, 2 * inter, dtype=dtype, device=DEV)
    out = torch.zeros(T + 1, inter, dtype=dtype, device=DEV)
    _run(ops, lambda p: p.linear_swiglu(x.to(DEV), w.to(DEV), gate_up, out, act="clamped_swish", params=(0.9, 1.702)), _bare(T))
    z = (x.float() @ w.float().t()).to(dtype).float()
    assert float((z.abs() > 0.9).float().mean()) > 0.1, "the limit must cut something"
    want = _clamped(z, inter, 0.9)
    assert float((out[:T].float().cpu() - want).abs().max()) < tol
    assert float(out[T:].abs().max()) == 0.0
    assert float((want - _clamped(z, inter, 1e9)).abs().max()) > 10 * tol


def _attention_case(ops, dtype, H, G, dk, dv, W, first, page, lens, cuts, sink=True, rot=None, scaling=None, seed=0):
    """Requests of `lens` tokens whose first `cuts[r]` tokens are cached by one step; the second step brings the rest.
    Returns (engine's output of the second step, the plain result for those tokens)."""
    from llmengine_b200.engine.batch import GroupView, StepBatch
    g = torch.Generator().manual_seed(seed)
    R, ps = len(lens), page
    eps, scale = 1e-5, 1.0 / math.sqrt(dk) * 1.7
    q_gain, k_gain = 1 + 0.2 * torch.randn(H * dk, generator=g), 1 + 0.2 * torch.randn(G * dk, generator=g)
    sinks = torch.randn(H, generator=g) * 2 if sink else None
    f, amp = yarn_frequencies(rot, 500.0, scaling) if rot else (None, 1.0)
    proj = [(torch.randn(n, H * dk + G * dk + G * dv, generator=g) * 1.5).to(dtype) for n in lens]
    blocks = [-(-n // ps) for n in lens]
    perm = torch.randperm(sum(blocks) + 3, generator=g).tolist()
    tables = torch.full((R, max(blocks) + 1), -1, dtype=torch.int32)
    at = 0
    for r, nb in enumerate(blocks):
        tables[r, :nb] = torch.tensor(perm[at:at + nb], dtype=torch.int32)
        at += nb
    cache = torch.full((sum(blocks) + 3, G * ps * (dk + dv)), float("nan"), dtype=dtype, device=DEV)
    outs = []
    for step in range(2):
        spans = [(0, cuts[r]) if step == 0 else (cuts[r], lens[r]) for r in range(R)]
        spans = [(r, a, b) for r, (a, b) in enumerate(spans) if b > a]
        rows = torch.cat([proj[r][a:b] for r, a, b in spans]).to(DEV)
        T = rows.shape[0]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        pos = [p for _, a, b in spans for p in range(a, b)]
        req = [r for r, a, b in spans for _ in range(a, b)]
        slots = [int(tables[r, p // ps]) * ps + p % ps for r, a, b in spans for p in range(a, b)]
        q_lens = [b - a for _, a, b in spans]
        batch = StepBatch(
            num_tokens=T, num_requests=len(spans), q_lens=q_lens, start_positions=[a for _, a, _ in spans], token_ids=i32([0] * T),
            positions=i32(pos), token_request=i32(req), cu_q_lens=i32([0] + list(np.cumsum(q_lens))), ctx_lens=i32([b for _, _, b in spans]),
            state_slots=i32([r for r, _, _ in spans]), first_portion=i32([int(a == 0) for _, a, _ in spans]), logit_rows=i32([]),
            decode_rows=i32([i for i, q in enumerate(q_lens) if q == 1]), portion_rows=i32([i for i, q in enumerate(q_lens) if q != 1]),
            groups=[GroupView(ps, W, tables.to(DEV), i32(slots), tables.shape[1])])
        q = torch.zeros(T, H * dk, dtype=dtype, device=DEV)
        out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
        qs, ks = H * dk, G * dk
        _run(ops, lambda p: p.window_attention(
            q_in=rows[:, :qs], k_in=rows[:, qs:qs + ks], v_in=rows[:, qs + ks:], q_gain=q_gain.to(DEV), k_gain=k_gain.to(DEV), eps=eps,
            inv_freq=f.to(DEV) if rot else None, rot_dims=rot or 0, amplitude=amp, q=q, out=out, cache=cache, group=0, num_heads=H,
            num_kv_heads=G, qk_dim=dk, v_dim=dv, window=W, keep_first=first, scale=scale, sink=sinks.to(DEV) if sink else None,
            scratch=torch.zeros(R * H * 8 * (dv + 2), device=DEV) if dtype == torch.bfloat16 else None), batch)
        outs.append((spans, out.float().cpu()))
    # the plain result, request by request over the whole sequence
    rt = lambda t: t.to(dtype).float()
    want = []
    for r, a, b in outs[1][0]:
        n = lens[r]
        pr = proj[r].float()
        P = torch.arange(n)
        fin = lambda x, heads, gain: rotate(rms_norm(x, gain, eps).view(n, heads, dk), P, f, amp) if rot else rms_norm(x, gain, eps).view(n, heads, dk)
        qq, kk = rt(fin(pr[:, :qs], H, q_gain)), rt(fin(pr[:, qs:qs + ks], G, k_gain))
        vv = pr[:, qs + ks:].view(n, G, dv)
        s = torch.einsum("ihd,jhd->hij", qq, kk.repeat_interleave(H // G, 1)) * scale
        p = sink_softmax(s, sinks if sink else torch.full((H,), -1e30), visible(n, W if W else n + 1, first))
        want.append(torch.einsum("hij,jhd->ihd", p, vv.repeat_interleave(H // G, 1)).reshape(n, H * dv)[a:b])
    return outs[1][1], torch.cat(want)


@pytest.mark.parametrize("kernels", ["fast", "plain"])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("H,G,dk,dv,W,first,page,rot,scaling", [
    (4, 2, 32, 16, 24, 3, 16, 16, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}),
    (8, 2, 64, 64, 70, 17, 64, 32, None),
    (3, 3, 20, 12, 17, 5, 8, 6, None),              # sizes only the plain kernel takes
    (6, 1, 16, 48, 0, 0, 16, None, None),           # no window, no rotation, six heads on one key/value head
    (2, 2, 128, 128, 33, 40, 32, 128, None),        # more kept first positions than the window is wide
    (8, 2, 64, 64, 400, 70, 16, 32, None),          # long enough that single tokens' keys are cut into ranges
    (4, 1, 32, 48, 0, 0, 64, 16, None),             # the same without a window
])
def test_window_attention_kernels(kernels, dtype, tol, H, G, dk, dv, W, first, page, rot, scaling):
    """Portions that start inside a page, a window and the kept first positions; single tokens beside them; prompts
    shorter than the window; free pages hold NaN."""
    ops = _ops(kernels)
    lens, cuts = [150, 9, 1, 200, 131, 77], [149, 0, 0, 130, 130, 70]
    if W == 400 or (W == 0 and dv == 48):
        lens, cuts = [700, 9, 1, 650, 131, 77], [699, 0, 0, 649, 130, 70]
    got, want = _attention_case(ops, dtype, H, G, dk, dv, W, first, page, lens, cuts, rot=rot, scaling=scaling, seed=dk + W)
    assert torch.isfinite(got).all()
    assert float((got - want).abs().max()) < tol
    if kernels == "fast" and dtype == torch.bfloat16:
        assert (f"attention_window_tc@DK={dk},DV={dv}" in ops._libs) == (dk % 16 == 0 and dv % 16 == 0)


@pytest.mark.parametrize("T,E,top", [(1, 5, 1), (7, 6, 2), (300, 16, 3), (40, 9, 9), (5, 130, 4)])
def test_routing_kernel(T, E, top):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    z = torch.randn(T, E, generator=g) * 2
    experts = torch.full((T + 1, top), -7, dtype=torch.int32, device=DEV)
    weights = torch.zeros(T + 1, top, device=DEV)
    offsets = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    order = torch.full(((T + 1) * top,), -1, dtype=torch.int32, device=DEV)
    for _ in range(2):                                    # twice: the scratch counts are left clean
        _run(ops, lambda p: p.moe_route(logits=z.to(DEV), top_k=top, scale=1.7, experts=experts, weights=weights, offsets=offsets,
                                        order=order, counts=counts), _bare(T))
    idx, wt = route(z, torch.eye(E), top, 1.7)
    assert torch.equal(experts[:T].cpu().long(), idx) and int(experts[T, 0]) == -7
    assert float((weights[:T].cpu() - wt).abs().max()) < 1e-6
    off, o = offsets.cpu().tolist(), order.cpu()[: T * top].tolist()
    assert off[0] == 0 and off[-1] == T * top and sorted(o) == list(range(T * top)) and int(counts.abs().sum()) == 0
    flat = idx.reshape(-1).tolist()
    for e in range(E):
        assert all(flat[pair] == e for pair in o[off[e]:off[e + 1]])


@pytest.mark.parametrize("kernels", ["fast", "plain"])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("T,E,top,D,ff", [(3, 5, 2, 48, 40), (130, 4, 2, 64, 96), (700, 6, 1, 72, 56), (9, 40, 3, 100, 33), (64, 3, 3, 256, 160)])
def test_grouped_products(kernels, dtype, tol, T, E, top, D, ff):
    """Experts with no, one, a few and hundreds of rows; tiles of both shapes; gather by token, scatter by pair, the
    activation in the epilogue; then the weighted sum."""
    ops = _ops(kernels)
    g = torch.Generator().manual_seed(4)
    h = torch.randn(T, D, generator=g).to(dtype)
    wgu = (torch.randn(E, 2 * ff, D, generator=g) / math.sqrt(D) * 2).to(dtype)
    wd = (torch.randn(E, D, ff, generator=g) / math.sqrt(ff)).to(dtype)
    z = torch.randn(T, E, generator=g) * 2
    if E > 2:
        z[:, 1] = -50.0                                   # an expert that nobody uses
    experts = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    weights, base = torch.zeros(T, top, device=DEV), torch.randn(T, D, generator=g).to(DEV)
    offsets, counts = torch.zeros(E + 1, dtype=torch.int32, device=DEV), torch.zeros(E, dtype=torch.int32, device=DEV)
    order = torch.zeros(T * top, dtype=torch.int32, device=DEV)
    act = torch.zeros(T * top, ff, dtype=dtype, device=DEV)
    mid = torch.zeros(T * top, 2 * ff, dtype=dtype, device=DEV)
    y = torch.full((T * top, D), float("nan"), device=DEV)
    out = torch.zeros(T, D, device=DEV)

    def record(p):
        p.moe_route(logits=z.to(DEV), top_k=top, scale=2.0, experts=experts, weights=weights, offsets=offsets, order=order, counts=counts)
        p.grouped_linear(x=h.to(DEV), w=wgu.to(DEV), out=act, offsets=offsets, order=order, top_k=top, gather=True, scatter=False, mid=mid, act="silu")
        p.grouped_linear(x=act, w=wd.to(DEV), out=y, offsets=offsets, order=order, top_k=top, gather=False, scatter=True)
        p.moe_combine(y=y, weights=weights, base=base, out=out)
    _run(ops, record, _bare(T))
    idx, wt = route(z, torch.eye(E), top, 2.0)
    want = base.cpu().clone()
    rd = lambda t: t.to(dtype).float()
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            gu = rd(wgu[e].float() @ h[t].float())
            a = rd(gu[:ff] * torch.sigmoid(gu[:ff]) * gu[ff:])
            want[t] += wt[t, k] * (wd[e].float() @ a)
    assert torch.isfinite(out).all() and float((out.cpu() - want).abs().max()) < tol * 4
    if dtype == torch.bfloat16:
        assert ("moe_tc" in ops._libs) == (kernels == "fast")


# ----------------------------------------------------------------------------- each mechanism in a model of its own
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("attention", ONLY_ATTENTION), ("dense", WITH_DENSE), ("moe", WITH_MOE), ("reader", WITH_READER)])
def test_each_mechanism_alone(tmp_path, name, cfg, dtype):
    d = make_torisun_dir(str(tmp_path / name), cfg, seed=9, sharpen=2.0)
    replay_all_schedules(d, cfg, dtype, [70, 5, 130, 1, 2], 16, None, DEV, only=("whole", "bulk_then_single", "portions"))


# ----------------------------------------------------------------------------- every schedule
@pytest.mark.parametrize("kernels", ["fast", "plain"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,page,lens", [
    ("A", TINY_A, 16, [70, 33, 100, 1, 19, 45, 64]),
    ("B", TINY_B, 8, [2, 5, 64, 130, 200, 48]),
    ("C", TINY_C, 64, [300, 129, 40, 520, 128, 17]),
    ("C16", TINY_C, 16, [260, 3, 141, 64]),
])
def test_replay_gpu(tmp_path, name, cfg, page, lens, dtype, kernels):
    d = make_torisun_dir(str(tmp_path / name), cfg, seed=11, sharpen=2.0)
    worst = replay_all_schedules(d, cfg, dtype, lens, page, None, DEV, kernels=kernels)
    print(f"replay {name} {dtype} {kernels}: share of the tolerance: " + ", ".join(f"{k} {v:.2f}" for k, v in worst.items()))


def test_every_layer_with_a_mask_of_its_own(tmp_path):
    """Ten layers whose windows and kept counts all differ are ten cache groups, each with block tables of its own that
    give pages back at its own pace."""
    cfg = {"architecture": "Torisun", "vocab": 70, "width": 32, "norm": {"eps": 1e-5},
           "layers": [layer(mixer(2, 1, 16, 16, 0.3, 3 + 5 * i, i % 4, base=50.0, dims=8), None) for i in range(10)]}
    d = make_torisun_dir(str(tmp_path / "m"), cfg, seed=2, sharpen=2.0)
    for dtype in ("float32", "bfloat16"):
        eng = engine_for(d, dtype, 256, page_size=8, max_requests=2, max_model_len=256)
        assert len(eng.cache.groups) == 10
        replay_all_schedules(d, cfg, dtype, [90, 17, 60, 5, 33], 8, None, DEV, only=("whole", "mixed"))


def test_the_fused_and_tensor_core_kernels_serve_bfloat16(tmp_path):
    from llmengine_b200.engine.engine import StepEntry
    d = make_torisun_dir(str(tmp_path / "C"), TINY_C, seed=4)
    for kernels, expected in (("fast", True), ("plain", False)):
        eng = engine_for(d, "bfloat16", 512, page_size=16, kernels=kernels, max_requests=2, max_model_len=512)
        before = eng.ops.launches
        eng.step([StepEntry("a", random_ids(300, 300, 1), [299])], [])
        eng.step([StepEntry("a", [7], [0])], ["a"])
        assert ("attention_window_tc@DK=64,DV=64" in eng.ops._libs) == expected
        assert ("moe_tc" in eng.ops._libs) == expected
        assert eng.ops.launches > before


# ----------------------------------------------------------------------------- constants that are one off
EDGE = {"architecture": "Torisun", "vocab": 50, "width": 64, "norm": {"eps": 1e-5},
        "layers": [layer(mixer(4, 2, 32, 32, 0.35, 21, 5, base=1000.0, dims=16, scaling={"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}), None)]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_edges_of_the_window_and_of_the_kept_first_positions(tmp_path, dtype):
    """A window one key wider or narrower, one more or one fewer kept first position, no sink, no stretching of the
    rotation: each moves the plain implementation's logits far beyond the tolerance.  The engine, with the right
    constants, stays within it for every position, in prompts and decoded, with page edges (4, 16, 64) inside and
    outside the window and the kept positions on one page and on two."""
    d = make_torisun_dir(str(tmp_path / "edge"), EDGE, seed=31, sharpen=3.0)
    reqs = {"a": random_ids(150, 50, 1), "b": random_ids(23, 50, 2), "c": random_ids(5, 50, 3)}
    ref, tol = reference_logits(d, reqs, dtype)
    changes = {
        "window + 1": lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 22),
        "window - 1": lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 20),
        "kept + 1": lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", 6),
        "kept - 1": lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("keep_first", 4),
        "not stretched": lambda c: c["layers"][0]["mixer"]["rot"].pop("scaling"),
        "all coordinates rotated": lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 32),
    }
    for what, change in changes.items():
        other = PlainTorisun(variant_dir(d, str(tmp_path / what.replace(" ", "_")), change))
        moved = float((other.logits(reqs["a"]) - ref["a"]).abs().max())
        assert moved > 3 * tol, f"{what} moves the logits by {moved:.3g} only (tolerance {tol:.3g})"
    for page in (4, 16, 64):
        for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_bulk_then_single(reqs, 60)), ("portions", trace_portions(reqs))):
            eng = engine_for(d, dtype, 320, page_size=page, max_requests=2, max_model_len=256)
            compare(replay(eng, steps, poison=True), ref, tol, f"{dtype}/page {page}/{what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_counts(tmp_path, dtype):
    """Sinks of +6 and -6: a head whose sink dominates gives almost nothing, one whose sink vanishes is a plain softmax;
    leaving the sink out, or scaling it like a score, would move the logits far beyond the tolerance."""
    def edit(t):
        t["l0.mix.sink"] = torch.tensor([6.0, -6.0, 2.0, 0.0]).to(torch.bfloat16)
    d = make_torisun_dir(str(tmp_path / "sink"), ONLY_ATTENTION, seed=8, sharpen=2.0, edit=edit)
    d0 = make_torisun_dir(str(tmp_path / "nosink"), ONLY_ATTENTION, seed=8, sharpen=2.0,
                          edit=lambda t: t.__setitem__("l0.mix.sink", torch.full((4,), -60.0).to(torch.bfloat16)))
    d1 = make_torisun_dir(str(tmp_path / "scaled"), ONLY_ATTENTION, seed=8, sharpen=2.0,
                          edit=lambda t: t.__setitem__("l0.mix.sink", (torch.tensor([6.0, -6.0, 2.0, 0.0]) * 0.3).to(torch.bfloat16)))
    reqs = {"a": random_ids(90, 61, 1), "b": random_ids(3, 61, 2)}
    ref, tol = reference_logits(d, reqs, dtype)
    for wrong in (d0, d1):
        other = PlainTorisun(wrong)
        assert max(float((other.logits(ids) - ref[r]).abs().max()) for r, ids in reqs.items()) > 4 * tol
    for what, steps in schedules(reqs, tail=20).items():
        eng = engine_for(d, dtype, 256, page_size=16, max_requests=2, max_model_len=256)
        compare(replay(eng, steps, poison=True), ref, tol, f"sink/{dtype}/{what}")


# ----------------------------------------------------------------------------- from the first token on, for long
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_the_first_token_through_captured_steps(tmp_path, dtype):
    """Three requests decoded token by token from position 0 on, far past every window and over several pages, with the
    steps captured in CUDA graphs: the same logits as whole prompts."""
    from llmengine_b200.engine.engine import StepEntry
    d = make_torisun_dir(str(tmp_path / "A"), TINY_A, seed=13, sharpen=2.0)
    n = 150
    reqs = {f"r{i}": random_ids(n, TINY_A["vocab"], 50 + i) for i in range(3)}
    ref, tol = reference_logits(d, reqs, dtype)
    eng = engine_for(d, dtype, 3 * 192, page_size=16, max_requests=4, use_cuda_graphs=True, max_model_len=192)
    rows = {r: [] for r in reqs}
    for i in range(n):
        out = eng.step([StepEntry(r, [ids[i]], [0]) for r, ids in reqs.items()], list(reqs) if i == n - 1 else [])
        for k, r in enumerate(reqs):
            rows[r].append(out[k].float().cpu().clone())
    assert eng.graphs_enabled and eng._graphs, "the parts of this design can be captured"
    compare({r: torch.stack(v) for r, v in rows.items()}, ref, tol, f"captured decode {dtype}")
    eng.cache.check_invariants()
    assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.groups)


def test_greedy_generation_through_the_scheduler(tmp_path):
    from llmengine_b200 import LLM, SamplingParams
    d = make_torisun_dir(str(tmp_path / "m"), TINY_A, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256)
    prompts = [random_ids(n, TINY_A["vocab"], i) for i, n in enumerate([1, 5, 64, 90, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=12, eos_token_id=None)
    plain = PlainTorisun(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 12)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    cfg = TINY_A
    d = make_torisun_dir(str(tmp_path / "m"), cfg, seed=17, sharpen=2.0)
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], 200 + i) for i, n in enumerate([70, 33, 100, 1, 19, 45])}
    ref, tol = reference_logits(d, reqs, dtype)
    steps = schedules(reqs)["mixed"]
    out = tmp_path / "out"
    lines = [json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in e], "end": end})
             for i, (e, end) in enumerate(steps)]
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", str(max_live_tokens(steps, 64))],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    rows = {}
    for i, (e, _) in enumerate(steps):
        arr = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        k = 0
        for r, t, w in e:
            rows.setdefault(r, []).append(arr[k:k + len(w)])
            k += len(w)
        assert k == arr.shape[0]
    compare({r: torch.cat(v) for r, v in rows.items()}, ref, tol, f"trace_run/{dtype}")
