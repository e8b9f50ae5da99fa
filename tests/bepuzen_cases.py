"""Shared equipment of the Bepuzen tests: the schedules a set of requests is replayed under and the comparison with the
plain implementation."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from helpers import (compare, engine_for, max_live_tokens, random_ids, replay, trace_bulk_then_single, trace_mixed,
                     trace_portions, trace_whole)
from plain_bepuzen import PlainBepuzen

TOL_F32 = 2e-4          # logits of these models are of order one to ten; only the order of sums differs


def reference_logits(model_dir: str, reqs: Dict[str, List[int]], dtype: str):
    """(reference, tolerance).  The reference is always the plain implementation in 32-bit.  In bfloat16 the yardstick
    is the model's own sensitivity to rounding: the distance between the plain run that rounds to bfloat16 where the
    design is defined to store values (weights, inputs of products, keys and values) and the unrounded run.  The
    engine rounds at other places too (it never forms keys and values: the query carried into the latent space and
    the weighted sum of latents are rounded instead), so its distance from the truth is of that size but not the same
    number; measured it is 0.5 to 1.5 yardsticks, and the bound is 2.5.  What the tests are after (a key skipped or read
    from a wrong place, a sink left out) moves the logits by ten and more yardsticks; the tests that plant such a key
    check that on the plain implementation first."""
    plain = PlainBepuzen(model_dir)
    ref = {r: plain.logits(ids) for r, ids in reqs.items()}
    if dtype != "bfloat16":
        return ref, TOL_F32
    rounded = PlainBepuzen(model_dir, round_to=torch.bfloat16)
    ref16 = {r: rounded.logits(ids) for r, ids in reqs.items()}
    inherent = max(float((ref16[r] - ref[r]).abs().max()) for r in ref)
    return ref, max(5e-3, 2.5 * inherent)


def schedules(reqs: Dict[str, List[int]], tail: int = 32):
    prompt = {r: max(1, len(ids) - 12) for r, ids in reqs.items()}
    return {
        "whole": trace_whole(reqs),
        "bulk_then_single": trace_bulk_then_single(reqs, tail),
        "portions": trace_portions(reqs),
        "mixed": trace_mixed(reqs, prompt, max_live=4, seed=3),
    }


def replay_all_schedules(model_dir: str, cfg: dict, dtype: str, lens: Sequence[int], page: int, ops, device: str,
                         kernels: str = "fast", only: Optional[Sequence[str]] = None, seed: int = 100) -> Dict[str, float]:
    """Every schedule against the plain implementation, free pages poisoned before every step; in the mixed schedule
    at most four requests are live and the pool is so small that pages and slots are handed to a second request."""
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], seed + i) for i, n in enumerate(lens)}
    ref, tol = reference_logits(model_dir, reqs, dtype)
    worst = {}
    for what, steps in schedules(reqs).items():
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


def greedy_by_the_plain_model(plain: PlainBepuzen, prompt: Sequence[int], n: int) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(plain.logits(ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
