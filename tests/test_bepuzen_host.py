"""The Bepuzen design on the host: configuration, tensor names, and the engine's own logic (batch metadata, the latent
cache's pages and block tables, scheduling) with a CPU stand-in for the kernels, against the plain implementation."""
import copy
import json

import pytest
import torch

from bepuzen_cases import greedy_by_the_plain_model, replay_all_schedules
from host_ops import HostOps
from helpers import random_ids
from llmengine_b200 import LLM, SamplingParams
from llmengine_b200.config import BepuzenConfig, ConfigError, config_from_dict
from llmengine_b200.engine.model import Model
from llmengine_b200.parts import Runtime
from plain_bepuzen import PlainBepuzen
from tiny_bepuzen import ONLY_L1, TINY_P, TINY_Q, TINY_S, make_bepuzen_dir, tensor_shapes


def test_every_size_and_constant_comes_from_the_file():
    c = config_from_dict(TINY_P)
    assert isinstance(c, BepuzenConfig) and c.hidden_size == 64 and c.vocab_size == 97 and c.side_dim == 8
    m = c.mixers[0]
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.rot_dims, m.rot_base, m.scale) == (4, 16, 16, 24, 64, 8, 500.0, 0.21)
    assert not c.mixers[1].rotary and c.ff_sizes == (96, 0, 40)
    assert config_from_dict(c.to_dict()) == c
    assert config_from_dict(TINY_Q).side_dim == 0
    for path in (["width"], ["norm"], ["layers", 0, "mixer", "kv_rank"], ["layers", 0, "mixer", "rot", "base"],
                 ["layers", 0, "mlp", "ff"], ["layers", 2, "type"], ["token_side", "dim"], ["layers", 0, "mixer", "scale"]):
        d = copy.deepcopy(TINY_P)
        at = d
        for k in path[:-1]:
            at = at[k]
        del at[path[-1]]
        with pytest.raises(ConfigError, match=str(path[-1])):
            config_from_dict(d)
    d = copy.deepcopy(TINY_P)
    del d["layers"][1]["mlp"]                       # no key at all reads like null: no feed-forward
    assert config_from_dict(d) == c
    d = copy.deepcopy(TINY_P)
    d["layers"][1]["type"] = "something_else"
    with pytest.raises(ConfigError, match="something_else"):
        config_from_dict(d)


@pytest.mark.parametrize("cfg", [TINY_P, TINY_Q, TINY_S, ONLY_L1])
def test_the_model_declares_the_design_s_tensors(cfg):
    model = Model(config_from_dict(cfg).model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1))
    declared = {n: tuple(s.shape) for n, s in model.weight_specs().items()}
    assert declared == tensor_shapes(cfg)


@pytest.mark.parametrize("name,cfg,page", [("P", TINY_P, 16), ("Q", TINY_Q, 8), ("S", TINY_S, 32)])
def test_host_logic_replay_cpu(tmp_path, name, cfg, page):
    d = make_bepuzen_dir(str(tmp_path / name), cfg, seed=3)
    replay_all_schedules(d, cfg, "float32", [70, 33, 100, 1, 19, 45], page, HostOps(), "cpu")


def test_greedy_generation_through_the_scheduler(tmp_path):
    d = make_bepuzen_dir(str(tmp_path / "m"), TINY_P, seed=5)
    llm = LLM(d, dtype="float32", page_size=16, max_cached_tokens=512, max_num_seqs=4, max_num_batched_tokens=64,
              prefill_chunk=40, max_model_len=256, device="cpu", ops=HostOps(), use_cuda_graphs=False)
    prompts = [random_ids(n, TINY_P["vocab"], i) for i, n in enumerate([1, 5, 64, 90, 33, 7])]
    outs = llm.generate(prompts, SamplingParams(greedy=True), max_tokens=5, eos_token_id=None)
    plain = PlainBepuzen(d)
    for p, o in zip(prompts, outs):
        assert o.token_ids == greedy_by_the_plain_model(plain, p, 5)
    llm.engine.cache.check_invariants()
    assert not llm.engine.cache.requests and llm.scheduler.all_done()


def test_a_weight_file_that_does_not_fit_is_refused(tmp_path):
    from llmengine_b200.engine.engine import Engine
    from llmengine_b200.config import EngineConfig
    from llmengine_b200.weights import WeightError

    def drop_sink(t):
        del t["l0.mix.sink"]
        t["l1.mix.uv"] = t["l1.mix.uv"][:, :-1].contiguous()
    d = make_bepuzen_dir(str(tmp_path / "m"), TINY_P, seed=1, edit=drop_sink)
    ec = EngineConfig(dtype="float32", max_cached_tokens=64, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64,
                      device="cpu")
    with pytest.raises(WeightError, match="l0.mix.sink") as e:
        Engine(d, engine_config=ec, ops=HostOps())
    assert "l1.mix.uv" in str(e.value)
