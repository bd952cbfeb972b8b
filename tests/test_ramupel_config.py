"""The Ramupel configuration, its layout and what it asks of the loader and the cache (no GPU)."""
import copy
import json
import os

import pytest
import torch

from ramupel_helpers import SMALL, WIDE


def test_configuration_is_read_and_written_back():
    from llmplayer_b200.config import RamupelConfig, config_from_dict
    cfg = config_from_dict(SMALL)
    assert isinstance(cfg, RamupelConfig)
    assert cfg.to_dict() == SMALL
    assert cfg.layers[1].ff is None and cfg.layers[0].mixer.rot_dims == 8
    assert config_from_dict(cfg.to_dict()) == cfg
    assert "gla" in cfg.describe()


@pytest.mark.parametrize("change,match", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r["embedding"].pop("scale"), "embedding.'scale'"),
    (lambda r: r["layers"][0].__setitem__("type", "conv"), "unknown"),
    (lambda r: r["layers"][0]["mlp"].__setitem__("kind", "experts"), "mlp.kind"),
    (lambda r: r["layers"][0]["mixer"]["rot"].__setitem__("dims", 14), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("tau", 0.0), "tau"),
    (lambda r: r["layers"][1]["mixer"].pop("vdim"), "vdim"),
    (lambda r: r.__setitem__("layers", []), "layers"),
])
def test_bad_configurations_are_refused(change, match):
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.errors import ConfigError
    raw = copy.deepcopy(SMALL)
    change(raw)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_layout_names_every_tensor_with_its_shape():
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.engine.model import expected_tensors
    from llmplayer_b200.parts.specs import ANY
    specs = expected_tensors(config_from_dict(SMALL).layout())
    shapes = {k: v.shape for k, v in specs.items()}
    assert shapes["embed"] == (203, 88) and shapes["final.norm"] == (88,)
    assert shapes["l0.mix.q"] == (3 * 36, 88) and shapes["l0.mix.dkv"] == (52, 88) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (72, 40) and shapes["l0.mix.uv"] == (60, 40) and shapes["l0.mix.g"] == (3, 88)
    assert shapes["l0.mix.o"] == (88, 60) and shapes["l0.mlp.up"] == (136, 88) and shapes["l0.mlp.act"] == (2,)
    assert shapes["l1.mix.a1"] == (ANY, 88) and shapes["l1.mix.a2"] == (40, ANY) and shapes["l1.mix.a2.b"] == (40,)
    assert shapes["l1.mix.norm"] == (36,) and shapes["l1.mix.g"] == (72, 88)
    assert "l1.mlp.up" not in shapes and "l1.rg2" not in shapes and shapes["l1.rg1"] == (88, 88)
    assert [shapes[f"l{i}.dwa"] for i in range(4)] == [(2,), (3,), (4,), (5,)]


def test_a_size_left_to_the_file_is_accepted_and_a_mismatch_is_reported(tmp_path):
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.engine.model import expected_tensors
    from llmplayer_b200.errors import WeightError
    from llmplayer_b200.weights import write_random_model
    from llmplayer_b200.weights.loader import load_tensors
    from llmplayer_b200.weights.safetensors_io import write_safetensors
    from plain_llama import read_safetensors
    cfg = config_from_dict(SMALL)
    out = write_random_model(cfg, 1, str(tmp_path / "m"), dtype="bfloat16")
    path = os.path.join(out, "model.safetensors")
    tensors = read_safetensors(path)
    tensors["l1.mix.a1"] = torch.zeros(7, 88, dtype=torch.bfloat16)
    tensors["l1.mix.a2"] = torch.zeros(40, 7, dtype=torch.bfloat16)
    write_safetensors(path, tensors)
    loaded = load_tensors(out, expected_tensors(cfg.layout()))
    assert loaded["l1.mix.a1"].shape == (7, 88)
    tensors["l1.mix.a2"] = torch.zeros(41, 7, dtype=torch.bfloat16)
    write_safetensors(path, tensors)
    with pytest.raises(WeightError, match=r"l1.mix.a2: expected shape \[40, 'any'\]"):
        load_tensors(out, expected_tensors(cfg.layout()))
    assert json.load(open(os.path.join(out, "config.json")))["architecture"] == "Ramupel"
    # a gate for the feed-forward that layer 1 does not have is passed over, anything else unexpected is reported
    tensors["l1.mix.a2"] = torch.zeros(40, 7, dtype=torch.bfloat16)
    tensors["l1.rg2"] = torch.zeros(88, 88, dtype=torch.bfloat16)
    tensors["l1.rg2.b"] = torch.zeros(88, dtype=torch.bfloat16)
    write_safetensors(path, tensors)
    loaded = load_tensors(out, expected_tensors(cfg.layout()), ignore=cfg.ignorable_tensors())
    assert "l1.rg2" not in loaded and cfg.ignorable_tensors() == ("l1.rg2", "l1.rg2.b")
    tensors["l0.extra"] = torch.zeros(3, dtype=torch.bfloat16)
    write_safetensors(path, tensors)
    with pytest.raises(WeightError, match=r"unexpected \(1\): l0.extra"):
        load_tensors(out, expected_tensors(cfg.layout()), ignore=cfg.ignorable_tensors())


def test_cache_groups_rows_and_states():
    from llmplayer_b200.cache import RowsRequest, SequenceCache, StateRequest
    from llmplayer_b200.config import config_from_dict
    from llmplayer_b200.engine.model import Model
    model = Model(config_from_dict(WIDE).layout())
    requests = model.cache_requests()
    assert requests == [StateRequest((2, 128, 64), torch.float32), RowsRequest(192), RowsRequest(32)]
    cache = SequenceCache(requests, max_tokens=256, max_slots=3, kv_dtype=torch.bfloat16, device="cpu")
    assert [tuple(g.storage.shape) for g in cache.groups] == [(1, 4, 64, 192), (1, 4, 64, 32)]
    a = cache.acquire()
    cache.view(0).rows[a].fill_(3.0)
    cache.reserve([a], [70])
    cache.commit([a], [70])
    assert cache.page_tables([a]) == [[[0, 1]], [[0, 1]]]
    cache.release(a)
    b = cache.acquire()
    assert b == a and float(cache.view(0).rows[b].abs().sum()) == 0.0      # a slot's state starts at zero again
    assert cache.free_pages() == [4, 4]
