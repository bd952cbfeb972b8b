"""Botuvik's configuration: keys, errors, layout, the order of runs, what the runs keep in the cache. No GPU."""
import copy

import pytest
import torch

from botuvik_helpers import CONFIGS, RAGGED, SMALL, WIDE


def cfg_of(raw):
    from llmplayer_b200.config import config_from_dict
    return config_from_dict(raw)


def test_round_trip_and_registry():
    from llmplayer_b200.config import BotuvikConfig, known_architectures
    assert "Botuvik" in known_architectures()
    for raw, _, _ in CONFIGS.values():
        cfg = cfg_of(raw)
        assert isinstance(cfg, BotuvikConfig)
        assert cfg_of(cfg.to_dict()) == cfg
        assert cfg.max_positions() >= 65536


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 26), (("layers", 0, "mixer", "rot", "dims"), 7),
    (("layers", 0, "mixer", "softcap"), 0.0), (("layers", 1, "mixer", "gate_cap"), -1.0), (("layers", 1, "type"), "lstm"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4), (("layers", 0, "mlp", "router", "groups", "keep"), 4),
    (("layers", 0, "mlp", "router", "top"), 5), (("layers", 1, "mlp", "kind"), "sparse"), (("loop", "stop"), 9),
    (("loop", "times"), 0), (("norm", "eps"), 0.0), (("width",), 0), (("layers", 1, "mlp", "ff"), None),
])
def test_bad_values_are_refused(path, value):
    from llmplayer_b200.errors import ConfigError
    raw = copy.deepcopy(SMALL)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        cfg_of(raw)


def test_order_of_runs():
    runs = cfg_of(SMALL).layout().run_order()
    assert [r.layer for r in runs] == [0, 1, 2, 1, 2, 3]
    assert [(r.add_embedding, r.add_vector, r.add_row) for r in runs] == [
        (False, None, 0), (False, "loop.step", 0), (False, None, 0), (True, "loop.step", 1), (False, None, 0),
        (False, None, 0)]
    runs = cfg_of(WIDE).layout().run_order()
    assert [r.layer for r in runs] == [0, 0, 0, 1, 2]
    assert [r.add_embedding for r in runs] == [False, True, True, False, False]
    assert [r.add_row for r in runs[:3]] == [0, 1, 2]
    runs = cfg_of(RAGGED).layout().run_order()
    assert [r.layer for r in runs] == [0, 1] and not any(r.add_embedding or r.add_vector for r in runs)


def test_tensors_and_cache_requests():
    from llmplayer_b200.cache.sequence_cache import KVRequest, StateRequest
    from llmplayer_b200.engine.model import Model
    model = Model(cfg_of(SMALL).layout())
    specs = model.tensor_specs()
    assert specs["loop.step"].shape == (2, 72)
    assert specs["l0.mix.q"].shape == (96, 72) and specs["l0.mix.v"].shape == (80, 72) and specs["l0.mix.o"].shape == (72, 160)
    assert specs["l0.mix.q.b"].shape == (96,) and specs["l0.mix.v.b"].shape == (80,) and specs["l0.mix.sink"].shape == (4,)
    assert specs["l1.mix.i"].shape == (3, 72) and specs["l1.mix.f.b"].shape == (3,) and specs["l1.mix.norm"].shape == (84,)
    assert specs["l0.mlp.e5.down"].shape == (72, 24) and specs["l0.mlp.shared.gate"].shape == (40, 72)
    assert specs["l0.mlp.router"].shape == (6, 72) and "l3.mlp.shared.up" not in specs and "l2.norm2" not in specs
    assert specs["head"].shape == (211, 72) and specs["final.norm"].shape == (72,)
    reqs = model.cache_requests()
    assert len(reqs) == 6                                        # every pass of the loop keeps a cache of its own
    assert reqs[0] == KVRequest(2, 48, None)                     # keys of 24 and values of 40 stored in heads of 48
    assert reqs[1] == reqs[3] == (StateRequest((3, 29, 10), torch.float32), StateRequest((3,), torch.float32))
    assert reqs[2] == reqs[4] == KVRequest(3, 16, None)
    assert reqs[5][0].shape == (1, 21, 36)


def test_cache_gives_every_run_its_own_state():
    from llmplayer_b200.cache.sequence_cache import SequenceCache
    from llmplayer_b200.engine.model import Model
    model = Model(cfg_of(SMALL).layout())
    cache = SequenceCache(model.cache_requests(), max_tokens=256, max_slots=3, kv_dtype=torch.float32, device="cpu")
    assert cache.view(1).blocks[0].data_ptr() != cache.view(3).blocks[0].data_ptr()
    assert cache.view(2).pages.data_ptr() != cache.view(4).pages.data_ptr()
    assert cache.view(2).group_index == cache.view(4).group_index
    a = cache.acquire()
    cache.view(1).blocks[0][a].fill_(3.0)
    cache.view(1).blocks[1][a].fill_(-2.0)
    cache.release(a)
    b = cache.acquire()
    assert b == a and float(cache.view(1).blocks[0][b].abs().max()) == 0.0 and float(cache.view(1).blocks[1][b].abs().max()) == 0.0
