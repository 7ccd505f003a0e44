"""Revesun without a GPU: reading ``config.json``, the model description, the tensors it expects, the cache needs of
its mixers and what the cache manager makes of them."""

import copy

import pytest
import torch

from tesseract_b200.cache.manager import CacheManager
from tesseract_b200.config import ConfigError, load_model_description, resolve_architecture
from tesseract_b200.models.decoder import expected_tensors
from tesseract_b200.parts import PagedKeyValueNeed, StateNeed
from tesseract_b200.weights.random_init import write_random_model
from tests.revesun_models import TINY_REVESUN


def test_the_architecture_is_found_by_its_single_name():
    assert resolve_architecture({"architecture": "Revesun"}).name == "Revesun"
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"], "architecture": "Revesun"}).name == "LlamaForCausalLM"


@pytest.mark.parametrize("name", sorted(TINY_REVESUN))
def test_description_and_expected_tensors(tmp_path, name):
    config = TINY_REVESUN[name]
    folder = write_random_model(str(tmp_path / name), config, seed=3)
    architecture, typed, spec = load_model_description(folder)
    assert architecture.name == "Revesun" and spec.vocab_size == config["vocab"] and spec.hidden_size == config["width"]
    assert len(spec.layers) == len(config["layers"])
    expected = expected_tensors(spec)
    for index, layer in enumerate(config["layers"]):
        assert (spec.layers[index].feed_forward is None) == (layer["mlp"] is None)
        assert (f"l{index}.norm2" in expected) == (layer["mlp"] is not None)
        m = layer["mixer"]
        if layer["type"] == "attention":
            assert spec.layers[index].mixer.kind == "conv_attention"
            assert expected[f"l{index}.mix.q"].shape == (m["heads"] * m["dim"], config["width"])
            assert expected[f"l{index}.mix.v.conv"].shape == (m["kv_heads"] * m["vdim"], m["conv"])
            assert expected[f"l{index}.mix.o"].shape == (config["width"], m["heads"] * m["vdim"])
        else:
            assert spec.layers[index].mixer.kind == "mingru"
            assert expected[f"l{index}.mix.z.b"].shape == (m["width"],)
    assert spec.head.weights["weight"] == spec.embedding.weights["table"] == "embed"
    libraries = architecture.kernel_libraries(typed, "float32")
    assert "gemm_f32" in libraries and "attention_tcgen05" not in libraries


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "lstm"), "unknown type"),
    (lambda c: c["norm"].__setitem__("groups", 5), "groups"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 4), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "experts", "ff": 8}), "dense"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_bad_configurations_are_refused(change, message):
    from tesseract_b200.models.revesun_config import RevesunConfig

    config = copy.deepcopy(TINY_REVESUN["p"])
    change(config)
    with pytest.raises(ConfigError, match=message):
        RevesunConfig.from_dict(config)


def test_block_masked_pages_go_back_and_a_mixer_may_keep_pages_and_state():
    pages = PagedKeyValueNeed(num_kv_heads=2, key_dim=8, value_dim=4, block=40)
    assert pages.page_shape(16) == (2 * 16 * 12,)
    assert [pages.first_needed_position(p) for p in (0, 39, 40, 85)] == [0, 0, 40, 80]
    assert PagedKeyValueNeed(key_dim=8, value_dim=8, window=10, block=40).first_needed_position(45) == 40
    assert PagedKeyValueNeed(key_dim=8, value_dim=8, window=10, block=40).first_needed_position(59) == 50
    state = StateNeed((3, 24), torch.float32)
    manager = CacheManager([(pages, state), state, None], [None, None, None], num_pages=8, page_size=16,
                           max_requests=2, dtype=torch.float32, device="cpu", max_step_tokens=16)
    first, second, third = manager.bindings
    assert isinstance(first, tuple) and first[0].page_size == 16 and first[1].page_size == 0
    assert first[1].group == second.group and first[1].storage is not second.storage and third is None
    assert tuple(first[1].storage.shape) == (3, 3, 24)          # two requests and the scratch slot
    assert manager.admit("a")
    held = []
    for _ in range(12):                                          # 120 tokens, ten at a time
        manager.extend("a", 10)
        manager.commit("a", 10)
        held.append(manager.used_pages())
    assert max(held) <= 4 and held[-1] <= 3                      # never the eight pages that 120 tokens would take
    assert 0 not in manager.pages_of("a", first[0].group)        # the block that holds position 120 starts in page 7
    manager.release("a")
    manager.check()
    assert manager.used_pages() == 0
