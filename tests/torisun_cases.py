"""Shared equipment of the Torisun tests: the schedules a set of requests is replayed under and the comparison with the
plain implementation."""
from __future__ import annotations

import copy
import json
import os
from typing import Dict, List, Optional, Sequence

import torch

from helpers import (compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_mixed,
                     trace_portions, trace_whole)
from plain_torisun import PlainTorisun

TOL_F32 = 3e-4          # for logits of order one to ten (only the order of sums differs); it grows with larger ones


def reference_logits(model_dir: str, reqs: Dict[str, List[int]], dtype: str):
    """(reference, tolerance).  32-bit engine: the plain implementation in 32-bit.  bfloat16 engine: the plain
    implementation rounding to bfloat16 where the engine stores bfloat16 (weights, inputs of products, queries, keys,
    values, activations), all arithmetic 32-bit.  The rounded run is the reference because a mixture of experts is
    not continuous: where two experts' scores are close, rounding decides which one a token uses, and only a run that
    rounds where the engine rounds takes the same choices.  The yardstick of the tolerance is the model's own
    sensitivity to rounding, the distance between the rounded and the unrounded plain run: the engine must stay within
    one and a half yardsticks of the rounded run (it rounds the attention's probabilities too, and adds in another
    order).  What the tests are after (a key skipped or read from a wrong place, a window one token off, a sink left
    out) moves the logits by far more; the negative controls check that on the plain implementation."""
    plain = PlainTorisun(model_dir)
    rounded = PlainTorisun(model_dir, round_to=torch.bfloat16)
    keep_away_from_close_calls(rounded if dtype == "bfloat16" else plain, reqs, 0.2 if dtype == "bfloat16" else 2e-4)
    ref = {r: plain.logits(ids) for r, ids in reqs.items()}
    if dtype != "bfloat16":
        return ref, TOL_F32 * max(1.0, max(float(v.abs().max()) for v in ref.values()) / 10.0)
    ref16 = {r: rounded.logits(ids) for r, ids in reqs.items()}
    inherent = max(float((ref16[r] - ref[r]).abs().max()) for r in ref)
    return ref16, max(5e-3, 1.5 * inherent)


def keep_away_from_close_calls(model: PlainTorisun, reqs: Dict[str, List[int]], margin: float) -> None:
    """Changes the requests IN PLACE until no router of the model makes a close call on them: where the last chosen
    expert's logit lies less than `margin` above the first one not chosen, which expert a token uses is decided by
    rounding, and no comparison can rest on that.  The token at the first such position is exchanged for the next one
    of the vocabulary (positions before it are not affected: the model is causal)."""
    vocab = model.cfg["vocab"]
    for r, ids in reqs.items():
        for _ in range(40 * len(ids)):
            model.logits(ids)
            close = (model.gaps < margin).nonzero()
            if not close.numel():
                break
            p = int(close[0])
            ids[p] = (ids[p] + 1) % vocab
        else:
            raise AssertionError(f"request {r}: no way around the routers' close calls")


def schedules(reqs: Dict[str, List[int]], tail: int = 32):
    prompt = {r: max(1, len(ids) - 12) for r, ids in reqs.items()}
    return {
        "whole": trace_whole(reqs),
        "bulk_then_single": trace_bulk_then_single(reqs, tail),
        "portions": trace_portions(reqs),
        "mixed": trace_mixed(reqs, prompt, max_live=4, seed=3),
    }


def replay_all_schedules(model_dir: str, cfg: dict, dtype: str, lens: Sequence[int], page: int, ops, device: str,
                         kernels="fast", only: Optional[Sequence[str]] = None, seed: int = 100, tail: int = 32) -> Dict[str, float]:
    """Every schedule against the plain implementation, free pages poisoned before every step; in the mixed schedule
    at most four requests are live and the pool is so small that pages and slots are handed to a second request."""
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], seed + i) for i, n in enumerate(lens)}
    ref, tol = reference_logits(model_dir, reqs, dtype)
    worst = {}
    for what, steps in schedules(reqs, tail).items():
        if only is not None and what not in only:
            continue
        pool = max_live_tokens(steps, 64)
        eng = engine_for(model_dir, dtype, pool, page_size=page, ops=ops, device=device, kernels=kernels, max_requests=4,
                         max_model_len=max(len(v) for v in reqs.values()) + 64)
        pages = {} if what == "mixed" else None
        got = replay(eng, steps, poison=True, page_log=pages)
        worst[what] = compare(got, ref, tol, f"{dtype}/{what}") / tol
        eng.cache.check_invariants()
        assert not eng.cache.requests, "every request was ended, nothing may be held"
        assert all(g.pool.free_count == g.pool.num_pages for g in eng.cache.groups)
        if pages is not None and len(reqs) > 4:
            owners: Dict[int, set] = {}
            for r, held in pages.items():
                for p in held:
                    owners.setdefault(p, set()).add(r)
            assert any(len(o) > 1 for o in owners.values()), "no page was handed to a second request: the pool is too large"
    return worst


def variant_dir(model_dir: str, path: str, change) -> str:
    """The same weights under a changed config.json (`change(cfg)` edits it): what the plain implementation computes when a
    constant is off by one is the negative control of the test that uses the right one."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    cfg = copy.deepcopy(cfg)
    change(cfg)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    dst = os.path.join(path, "model.safetensors")
    if not os.path.exists(dst):
        os.symlink(os.path.abspath(os.path.join(model_dir, "model.safetensors")), dst)
    return path


def greedy_by_the_plain_model(plain: PlainTorisun, prompt: Sequence[int], n: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(plain.logits(ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
