"""The Torisun design on the host: configuration, tensor names, the mechanisms' host-side constants, the cache manager's
kept first positions, and the engine's own logic (batch metadata, pages, block tables, scheduling) with a CPU stand-in
for the kernels, against the plain implementation."""
import copy
import math

import pytest
import torch

from helpers import random_ids
from host_ops import HostOps
from llmengine_b200 import LLM, SamplingParams
from llmengine_b200.cache import CacheManager
from llmengine_b200.config import ConfigError, TorisunConfig, config_from_dict
from llmengine_b200.engine.model import Model
from llmengine_b200.parts import Runtime
from llmengine_b200.parts.attention import SplitKVSpec
from llmengine_b200.parts.latent import PartialRotaryEncoding
from plain_torisun import PlainTorisun, yarn_frequencies
from tiny_torisun import (ONLY_ATTENTION, TINY_A, TINY_B, TINY_C, WITH_MOE, WITH_READER, make_torisun_dir, tensor_shapes)
from torisun_cases import greedy_by_the_plain_model, replay_all_schedules


def test_every_size_and_constant_comes_from_the_file():
    c = config_from_dict(TINY_A)
    assert isinstance(c, TorisunConfig) and c.hidden_size == 64 and c.vocab_size == 97 and c.norm_eps == 1e-5
    m = c.mixers[1]
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.window, m.keep_first, m.rot_base, m.rot_dims, m.kv_from) == \
        (4, 2, 32, 16, 0.3, 9, 1, 500.0, 16, 0)
    assert (m.rot_scaling.factor, m.rot_scaling.original, m.rot_scaling.fast, m.rot_scaling.slow) == (4.0, 64.0, 16.0, 2.0)
    assert c.mixers[2].rot_scaling is None and c.mlps[2] is None
    f = c.mlps[0]
    assert (f.kind, f.experts, f.top, f.ff, f.route_scale, f.shared_ff) == ("moe", 6, 2, 40, 1.5, 24)
    assert (c.mlps[1].kind, c.mlps[1].ff, c.mlps[1].limit) == ("dense", 72, 2.0)
    assert config_from_dict(c.to_dict()) == c
    for path in (["width"], ["norm"], ["layers", 0, "mixer", "kv_heads"], ["layers", 0, "mixer", "rot", "base"],
                 ["layers", 0, "mixer", "mask", "keep_first"], ["layers", 0, "mixer", "mask", "size"], ["layers", 0, "mixer", "scale"],
                 ["layers", 0, "mixer", "vdim"], ["layers", 0, "mixer", "rot", "scaling", "fast"], ["layers", 1, "mlp", "limit"],
                 ["layers", 0, "mlp", "router", "top"], ["layers", 0, "mlp", "expert"], ["layers", 2, "type"]):
        d = copy.deepcopy(TINY_A)
        at = d
        for k in path[:-1]:
            at = at[k]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=str(path[-1])):
            config_from_dict(d)
    for edit, word in ((lambda d: d["layers"][1]["mixer"].__setitem__("kv_from", 1), "earlier"),
                       (lambda d: d["layers"][2]["mixer"].__setitem__("kv_from", 1), "of its own"),
                       (lambda d: d["layers"][1]["mixer"].__setitem__("vdim", 32), "equal"),
                       (lambda d: d["layers"][0].__setitem__("type", "something_else"), "something_else"),
                       (lambda d: d["layers"][1]["mlp"].__setitem__("kind", "sparse"), "sparse")):
        d = copy.deepcopy(TINY_A)
        edit(d)
        with pytest.raises(ConfigError, match=word):
            config_from_dict(d)


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C, ONLY_ATTENTION, WITH_READER])
def test_the_model_declares_the_design_s_tensors(cfg):
    model = Model(config_from_dict(cfg).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1))
    declared = {n: tuple(s.shape) for n, s in model.weight_specs().items()}
    assert declared == tensor_shapes(cfg)
    assert model.tied_tensors() == {"head": "embed"}


def test_a_reader_s_cache_keeps_what_every_reader_needs():
    """The owner's cache keeps the widest window and the most first positions among itself and its readers."""
    spec = config_from_dict(TINY_B).model_spec()
    owner, reader = spec.layers[0].parts["mixer"].params, spec.layers[1].parts["mixer"].params
    assert (owner["window"], owner["keep_first"], reader["window"], reader["keep_first"]) == (17, 5, 30, 2)
    assert (owner["retain_window"], owner["retain_first"]) == (reader["retain_window"], reader["retain_first"]) == (30, 5)
    assert [r.cache_from for r in spec.order] == [None, 0, None]


def test_stretched_rotary_frequencies():
    """The part's frequencies against the formulas written out once more, and their limits: factor 1 changes nothing,
    coordinates below `lo` keep their frequency, those above `hi` are slowed by the factor."""
    dims, base = 32, 10000.0
    sc = {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}
    f = PartialRotaryEncoding.build_frequencies(dims, base, (8.0, 128.0, 32.0, 1.0))
    plain = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    turns = lambda t: dims * math.log(128 / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(turns(32.0)), 0), min(math.ceil(turns(1.0)), dims - 1)
    assert 0 <= lo < hi < dims // 2
    for i in range(dims // 2):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert abs(float(f[i]) - float(plain[i]) * (r / 8.0 + 1 - r)) <= 1e-6 * float(plain[i])
    assert torch.allclose(f[: lo + 1], plain[: lo + 1], rtol=1e-6) and torch.allclose(f[hi:], plain[hi:] / 8.0, rtol=1e-6)
    g, amp = yarn_frequencies(dims, base, sc)
    assert torch.allclose(f, g, rtol=2e-7) and abs(amp - (0.1 * math.log(8.0) + 1.0)) < 1e-12
    assert torch.allclose(PartialRotaryEncoding.build_frequencies(dims, base, (1.0, 128.0, 32.0, 1.0)), plain, rtol=1e-6)
    part = PartialRotaryEncoding(Runtime(None, torch.device("cpu"), torch.float32, 1), "x", dims, base, sc)
    assert abs(part.amplitude - amp) < 1e-6


def test_pages_of_the_kept_first_positions_are_never_given_back():
    spec = SplitKVSpec(2, 16, 8, window=20, keep_first=9)
    m = CacheManager([(spec, None), (spec, 0)], page_size=8, max_cached_tokens=160, max_requests=2, max_request_len=400)
    g = m.groups[0]
    assert (g.window, g.keep_first, g.kept_blocks) == (20, 9, 2)
    m.add_request("a")
    held_most = 0
    for n in range(1, 300):
        m.reserve("a", n)
        blocks = m.requests["a"].blocks[0]
        lo = max(0, n - 1 - 20 + 1)                       # the first key the newest query's window reaches
        for j in list(range(min(9, n))) + list(range(lo, n)):
            assert blocks[j // 8] >= 0, f"position {j} has no page at length {n}"
        m.advance("a", n)
        held_most = max(held_most, sum(p >= 0 for p in m.requests["a"].blocks[0]))
        m.check_invariants()
    assert held_most <= g.peak_pages(300, 1) <= 2 + 4 + 1
    assert all(p >= 0 for p in m.requests["a"].blocks[0][:2]) and m.requests["a"].blocks[0][2] == -1
    m.free_request("a")
    assert g.pool.free_count == g.pool.num_pages
    # different kept counts are different groups; without a window nothing is given back and the count does not matter
    two = CacheManager([(SplitKVSpec(1, 8, 8, 20, 3), None), (SplitKVSpec(1, 8, 8, 20, 4), None), (SplitKVSpec(1, 8, 8, 0, 7), None),
                        (SplitKVSpec(1, 8, 8, 0, 2), None)], 8, 64, 1, 64)
    assert len(two.groups) == 3


@pytest.mark.parametrize("name,cfg,page", [("A", TINY_A, 16), ("B", TINY_B, 8), ("C", TINY_C, 32), ("R", WITH_READER, 4)])
def test_host_logic_replay_cpu(tmp_path, name, cfg, page):
    d = make_torisun_dir(str(tmp_path / name), cfg, seed=3, sharpen=2.0)
    replay_all_schedules(d, cfg, "float32", [70, 33, 100, 1, 19, 45], page, HostOps(), "cpu", tail=20)


def test_greedy_generation_through_the_scheduler(tmp_path):
    d = make_torisun_dir(str(tmp_path / "m"), TINY_A, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256, device="cpu", ops=HostOps(), use_cuda_graphs=False)
    prompts = [random_ids(n, TINY_A["vocab"], i) for i, n in enumerate([1, 5, 64, 90, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=5, eos_token_id=None)
    plain = PlainTorisun(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 5)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


def test_a_weight_file_that_does_not_fit_is_refused(tmp_path):
    from llmengine_b200.config import EngineConfig
    from llmengine_b200.engine.engine import Engine
    from llmengine_b200.weights import WeightError

    def damage(t):
        del t["l0.mix.sink"]
        t["l1.mlp.down"] = t["l1.mlp.down"][:, :-1].contiguous()
        t["l1.mix.k"] = torch.zeros(4, 4, dtype=torch.bfloat16)          # a reader has no key projection
        t["l2.norm2"] = torch.ones(64, dtype=torch.bfloat16)             # a gain for a feed-forward the layer lacks: ignored
    d = make_torisun_dir(str(tmp_path / "m"), TINY_A, seed=1, edit=damage)
    ec = EngineConfig(dtype="float32", max_cached_tokens=64, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64,
                      device="cpu")
    with pytest.raises(WeightError, match="l0.mix.sink") as e:
        Engine(d, engine_config=ec, ops=HostOps())
    assert "l1.mlp.down" in str(e.value) and "l1.mix.k" in str(e.value) and "l2.norm2" not in str(e.value)
