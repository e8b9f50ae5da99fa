"""The Bepuzen design on the GPU against the plain implementation: single kernels, each mechanism in a model of its
own, every schedule in both precisions and with both kernel sets, keys that stand out at chosen places, the sink,
decoding from the first token on through captured steps, generation through the scheduler, the trace program."""
import json
import math
import os
import subprocess

import numpy as np
import pytest
import torch

from bepuzen_cases import TOL_F32, greedy_by_the_plain_model, reference_logits, replay_all_schedules, schedules
from helpers import compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_whole
from plain_bepuzen import PlainBepuzen, gelu_tanh, token_side_input, xielu
from tiny_bepuzen import (L2, ONLY_L1, ONLY_L2, TINY_P, TINY_Q, TINY_R, TINY_S, WITH_FF, WITH_SIDE, layer, make_bepuzen_dir,
                          mixer2)

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = "cuda:0"


def _ops():
    from llmengine_b200.kernels.ops import CudaOps
    return CudaOps(torch.device(DEV))


def _run(ops, record, T, token_ids=None):
    from llmengine_b200.engine.batch import StepBatch
    from llmengine_b200.engine.plan import Plan
    plan = Plan()
    record(plan)
    ops.compile(plan).run(StepBatch.bare(T, torch.device(DEV), token_ids=token_ids))
    torch.cuda.synchronize()


def _softplus(v):
    return math.log1p(math.exp(-abs(v))) + max(v, 0.0)


# ----------------------------------------------------------------------------- single kernels
# a handful of tokens, and many with the tcgen05 product chosen: the activation rides in the product's epilogue
@pytest.mark.parametrize("T,K,N,linear", [(5, 40, 52, "auto"), (37, 40, 52, "auto"), (300, 64, 200, "tcgen05"), (260, 72, 40, "tcgen05")])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
def test_pointwise_kernels(dtype, tol, T, K, N, linear):
    ops = _ops()
    ops.choose("linear", linear)
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(T, K, generator=g)).to(dtype)
    w = (torch.randn(N, K, generator=g) / 4).to(dtype)
    pq = torch.tensor([0.3, -1.1])
    mid = torch.zeros(T + 3, N, dtype=dtype, device=DEV)
    out = torch.zeros(T + 3, N, dtype=dtype, device=DEV)
    _run(ops, lambda p: p.linear_act(x.to(DEV), w.to(DEV), mid, out, "xielu", (_softplus(0.3), 0.5 + _softplus(-1.1))), T)
    z = (x.float() @ w.float().t()).to(dtype).float()
    want = xielu(z, pq)
    # the squared branch makes values of tens: the bound follows the value (a bfloat16 digit is 1/256 of it)
    assert bool(((out[:T].float().cpu() - want).abs() <= tol * 4 + (want.abs() / 128 if dtype == torch.bfloat16 else 1e-5 * want.abs())).all())
    assert float(out[T:].abs().max()) == 0.0, "rows beyond the step's tokens are not touched"
    # a * sigmoid(b) on column ranges of a wider buffer
    wide = torch.randn(T, 3 * N, generator=g).to(dtype).to(DEV)
    a, b = wide[:, :N], wide[:, 2 * N:]
    res = torch.zeros(T, N, dtype=dtype, device=DEV)
    _run(ops, lambda p: p.pointwise("sigmoid_mul", a, b, res), T)
    assert float((res.float() - a.float() * torch.sigmoid(b.float())).abs().max()) < tol
    # one small matrix per member, strided operands
    B, k, n = 5, 24, 16
    xb = torch.randn(T, B * (k + 8), generator=g).to(dtype).to(DEV)
    wb = (torch.randn(B, n, k, generator=g) / 4).to(dtype).to(DEV)
    ob = torch.zeros(T, B * (n + 8), dtype=dtype, device=DEV)
    x3, o3 = xb.view(T, B, k + 8)[:, :, :k], ob.view(T, B, n + 8)[:, :, :n]
    _run(ops, lambda p: p.batched_linear(x3, wb, o3), T)
    want = torch.einsum("tbk,bnk->tbn", x3.float(), wb.float())
    assert float((o3.float() - want).abs().max()) < tol * 4
    assert float(ob.view(T, B, n + 8)[:, :, n:].abs().max()) == 0.0
    # contributions that no norm adds
    xs = torch.randn(T, K, generator=g).to(DEV)
    u, v = torch.randn(T, K, generator=g).to(DEV), torch.randn(T, K, generator=g).to(DEV)
    want = xs + (u + v)
    _run(ops, lambda p: p.residual_add(xs, u, v), T)
    assert float((xs - want).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-5), (torch.bfloat16, 6e-2)])
@pytest.mark.parametrize("T", [3, 150])
def test_token_side_input(dtype, tol, T):
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    D, dim, V, layers, li = 72, 24, 50, 3, 1
    W = {"gate": (torch.randn(dim, D, generator=g) / 8).to(dtype), "proj": (torch.randn(D, dim, generator=g) / 4).to(dtype),
         "norm": (1 + 0.1 * torch.randn(D, generator=g)).to(dtype)}
    table = torch.randn(V, layers * dim, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g)
    x = torch.randn(T, D, generator=g) * 3
    a, b = torch.randn(T, D, generator=g), torch.randn(T, D, generator=g)
    rnd = None if dtype == torch.float32 else dtype
    want = token_side_input(x + (a + b), ids, table.float(), li, dim, {k: v.float() for k, v in W.items()}, 1e-5, rnd)
    xd = x.to(DEV)
    ws = {k: v.to(DEV) for k, v in W.items()}
    bufs = dict(xb=torch.zeros(T, D, dtype=dtype, device=DEV), g=torch.zeros(T, dim, dtype=dtype, device=DEV),
                y=torch.zeros(T, D, device=DEV))
    _run(ops, lambda p: p.token_side(x=xd, a=a.to(DEV), b=b.to(DEV), table=table.to(DEV), offset=li * dim, dim=dim,
                                     w_gate=ws["gate"], w_proj=ws["proj"], gain=ws["norm"], eps=1e-5, **bufs), T,
         token_ids=ids.to(torch.int32).to(DEV))
    assert float((xd.cpu() - want).abs().max()) < tol


# ----------------------------------------------------------------------------- each mechanism in a model of its own
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("l2", ONLY_L2), ("l1", ONLY_L1), ("ff", WITH_FF), ("side", WITH_SIDE)])
def test_each_mechanism_alone(tmp_path, name, cfg, dtype):
    d = make_bepuzen_dir(str(tmp_path / name), cfg, seed=9, sharpen=2.0)
    replay_all_schedules(d, cfg, dtype, [70, 5, 130, 1, 2], 16, None, DEV, only=("whole", "bulk_then_single", "portions"))


# ----------------------------------------------------------------------------- every schedule
@pytest.mark.parametrize("kernels", ["fast", "plain"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,page,lens", [
    ("P", TINY_P, 16, [70, 33, 100, 1, 19, 45, 64]),
    ("Q", TINY_Q, 8, [2, 5, 64, 130, 200, 48]),
    ("R", TINY_R, 64, [300, 129, 40, 520, 128, 17]),
    ("S", TINY_S, 32, [3, 77, 140, 64, 31, 9]),
])
def test_replay_gpu(tmp_path, name, cfg, page, lens, dtype, kernels):
    d = make_bepuzen_dir(str(tmp_path / name), cfg, seed=11, sharpen=2.0)
    worst = replay_all_schedules(d, cfg, dtype, lens, page, None, DEV, kernels=kernels)
    print(f"replay {name} {dtype} {kernels}: share of the tolerance: " + ", ".join(f"{k} {v:.2f}" for k, v in worst.items()))


def test_the_tensor_core_kernel_serves_bfloat16(tmp_path):
    d = make_bepuzen_dir(str(tmp_path / "R"), TINY_R, seed=4)
    for kernels, expected in (("fast", True), ("plain", False)):
        eng = engine_for(d, "bfloat16", 256, page_size=16, kernels=kernels, max_requests=2, max_model_len=256)
        from llmengine_b200.engine.engine import StepEntry
        before = eng.ops.launches
        eng.step([StepEntry("a", random_ids(40, 300, 1), [39])], [])
        eng.step([StepEntry("a", [7], [0])], ["a"])
        assert ("attention_latent_tc@RANK=128" in eng.ops._libs) == expected
        assert eng.ops.launches > before


# ----------------------------------------------------------------------------- keys that stand out
FAR = {"architecture": "Bepuzen", "vocab": 40, "width": 64, "norm": {"eps": 1e-5},
       "layers": [layer(L2, mixer2(4, 16, 16, 64, 1.0), 0)]}


def _prompt_with_a_key_that_matters(plain, cfg, n, place, seed):
    """A prompt in which ONE key carries the last position's attention in one head.  From the model's own weights, per
    head, the score of every (query token, key token) pair; a query token b, its best key token a and a set of filler
    tokens whose scores against b lie at least 9 below a's: hundreds of fillers together then weigh less than a alone.
    The prompt is fillers drawn at random, a at `place`, b last.  Returns (prompt, the prompt with a filler in a's
    place, how far that exchange moves the last position's logits)."""
    from plain_bepuzen import scalar_rms_norm, weighted_rms_norm
    w, m, eps = plain.w, cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    V, H, dn = cfg["vocab"], m["heads"], m["dim"]
    h = scalar_rms_norm(w["embed"], w["l0.norm1"], eps)
    q = (h @ w["l0.mix.q"].t()).view(V, H, dn)
    c = weighted_rms_norm(h @ w["l0.mix.dkv"].t(), w["l0.mix.dkv.norm"], eps)
    k = (c @ w["l0.mix.uk"].t()).view(V, H, dn)
    S = torch.einsum("bhd,ahd->hba", q, k) * m["scale"]
    best = None
    for hh in range(H):
        for b in range(V):
            row = S[hh, b].clone()
            row[b] = -1e9
            a = int(row.argmax())
            fill = [f for f in range(V) if f not in (a, b) and S[hh, b, f] < S[hh, b, a] - 9]
            if S[hh, b, b] < S[hh, b, a] - 9 and (best is None or len(fill) > len(best[2])):
                best = (a, b, fill)
    assert best is not None and len(best[2]) >= 5, "the weights give no pair of tokens that stands out"
    a, b, fill = best
    g = torch.Generator().manual_seed(seed)
    ids = [fill[int(i)] for i in torch.randint(0, len(fill), (n,), generator=g)]
    ids[place], ids[-1] = a, b
    other = list(ids)
    other[place] = fill[0]
    moved = float((plain.logits(ids)[-1] - plain.logits(other)[-1]).abs().max())
    return ids, other, moved


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,place", [(700, 0), (700, 15), (700, 16), (700, 63), (700, 64), (700, 383), (130, 127), (130, 128)])
def test_one_key_among_hundreds(tmp_path, dtype, n, place):
    """Pages of 16 and of 64: the key sits on the first place, on the last place of a page and on the first of the
    next, near and far; the last token is served inside a prompt portion and as a decoded token whose keys are cut
    into ranges over several blocks."""
    d = make_bepuzen_dir(str(tmp_path / "far"), FAR, seed=21, sharpen=4.0)
    plain = PlainBepuzen(d)
    ids, other, moved = _prompt_with_a_key_that_matters(plain, FAR, n, place, seed=n + place)
    reqs = {"k": ids}
    ref, tol = reference_logits(d, reqs, dtype)
    assert moved > 2 * tol, f"exchanging the key moves the logits by {moved:.3g} only (tolerance {tol:.3g})"
    for page in (16, 64):
        for what, steps in (("whole", trace_whole(reqs)), ("decoded", trace_bulk_then_single(reqs, 3))):
            eng = engine_for(d, dtype, 768, page_size=page, max_requests=2, max_model_len=768)
            got = replay(eng, steps, poison=True)
            compare(got, ref, tol, f"{dtype}/page {page}/{what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_counts(tmp_path, dtype):
    """Sinks of +6 and -6: a head whose sink dominates gives almost nothing, one whose sink vanishes is a plain softmax;
    leaving the sink out, or scaling it like a score, would move the logits far beyond the tolerance."""
    def edit(t):
        t["l0.mix.sink"] = torch.tensor([6.0, -6.0, 2.0, 0.0]).to(torch.bfloat16)
    d = make_bepuzen_dir(str(tmp_path / "sink"), ONLY_L1, seed=8, sharpen=2.0, edit=edit)
    d0 = make_bepuzen_dir(str(tmp_path / "nosink"), ONLY_L1, seed=8, sharpen=2.0,
                          edit=lambda t: t.__setitem__("l0.mix.sink", torch.full((4,), -60.0).to(torch.bfloat16)))
    reqs = {"a": random_ids(90, 61, 1), "b": random_ids(3, 61, 2)}
    ref, tol = reference_logits(d, reqs, dtype)
    without = PlainBepuzen(d0)
    assert max(float((without.logits(ids) - ref[r]).abs().max()) for r, ids in reqs.items()) > 4 * tol
    for what, steps in schedules(reqs, tail=20).items():
        eng = engine_for(d, dtype, 256, page_size=16, max_requests=2, max_model_len=256)
        compare(replay(eng, steps, poison=True), ref, tol, f"sink/{dtype}/{what}")


# ----------------------------------------------------------------------------- from the first token on, for long
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_the_first_token_through_captured_steps(tmp_path, dtype):
    """Three requests decoded token by token from position 0 on, over several pages, with the steps captured in CUDA
    graphs: the same logits as whole prompts."""
    from llmengine_b200.engine.engine import StepEntry
    d = make_bepuzen_dir(str(tmp_path / "P"), TINY_P, seed=13, sharpen=2.0)
    n = 150
    reqs = {f"r{i}": random_ids(n, TINY_P["vocab"], 50 + i) for i in range(3)}
    ref, tol = reference_logits(d, reqs, dtype)
    eng = engine_for(d, dtype, 3 * 192, page_size=16, max_requests=4, use_cuda_graphs=True, max_model_len=192)
    rows = {r: [] for r in reqs}
    for i in range(n):
        out = eng.step([StepEntry(r, [ids[i]], [0]) for r, ids in reqs.items()], list(reqs) if i == n - 1 else [])
        for k, r in enumerate(reqs):
            rows[r].append(out[k].float().cpu().clone())
    assert eng._graphs or not eng.graphs_enabled
    assert eng.graphs_enabled, "the parts of this design can be captured"
    compare({r: torch.stack(v) for r, v in rows.items()}, ref, tol, f"captured decode {dtype}")


def test_greedy_generation_through_the_scheduler(tmp_path):
    from llmengine_b200 import LLM, SamplingParams
    d = make_bepuzen_dir(str(tmp_path / "m"), TINY_P, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256)
    prompts = [random_ids(n, TINY_P["vocab"], i) for i, n in enumerate([1, 5, 64, 90, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=12, eos_token_id=None)
    plain = PlainBepuzen(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 12)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    cfg = TINY_P
    d = make_bepuzen_dir(str(tmp_path / "m"), cfg, seed=17, sharpen=2.0)
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
