"""Pekodra without a GPU: reading ``config.json``, the run order of a looped model, the model description, the
tensors it expects, the cache needs of its mixers and what the cache manager makes of a sliding window."""

import copy

import pytest
import torch

from tesseract_b200.cache.manager import CacheManager
from tesseract_b200.config import ConfigError, load_model_description, resolve_architecture
from tesseract_b200.models.decoder import expected_tensors
from tesseract_b200.parts import PagedKeyValueNeed
from tesseract_b200.weights.random_init import write_random_model
from tests.pekodra_models import TINY_PEKODRA, random_config
from tests.plain import pekodra as plain


def test_the_architecture_is_found_by_its_single_name():
    assert resolve_architecture({"architecture": "Pekodra"}).name == "Pekodra"


@pytest.mark.parametrize("name", sorted(TINY_PEKODRA))
def test_description_and_expected_tensors(tmp_path, name):
    config = TINY_PEKODRA[name]
    folder = write_random_model(str(tmp_path / name), config, seed=3)
    architecture, typed, spec = load_model_description(folder)
    assert architecture.name == "Pekodra" and spec.vocab_size == config["vocab"] and spec.hidden_size == config["width"]
    assert len(spec.layers) == len(config["layers"])
    expected = expected_tensors(spec)
    width = config["width"]
    for index, layer in enumerate(config["layers"]):
        assert spec.layers[index].block == "parallel" and spec.layers[index].mixer.kind == "normed_attention"
        assert (f"l{index}.norm2" in expected) == (layer["mlp"] is not None)
        m = layer["mixer"]
        assert expected[f"l{index}.mix.q"].shape == (m["heads"] * m["dim"], width)
        assert expected[f"l{index}.mix.v"].shape == (m["kv_heads"] * m["vdim"], width)
        assert expected[f"l{index}.mix.o"].shape == (width, m["heads"] * m["vdim"])
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            assert expected[f"l{index}.mlp.gate.b"].shape == (mlp["ff"],)
            assert expected[f"l{index}.mlp.down.b"].shape == (width,)
        elif mlp:
            last = mlp["router"]["experts"] - 1
            assert expected[f"l{index}.mlp.router"].shape == (mlp["router"]["experts"], width)
            assert expected[f"l{index}.mlp.e{last}.down"].shape == (width, mlp["expert"]["ff"])
            assert (f"l{index}.mlp.shared.up" in expected) == ("shared" in mlp)
    assert spec.head.weights["weight"] == "head" and spec.embedding.weights["table"] == "embed"
    assert ("loop.in" in expected) == ("loop" in config)
    # the run order of the description is the plain model's, and every walk of the loop starts with the injection
    assert [(e.layer, e.inject is not None) for e in spec.run_order] == plain.run_order(config)
    assert all(e.cache_of is None for e in spec.run_order)           # a cache of its own for every run of a layer
    libraries = architecture.kernel_libraries(typed, "float32")
    assert "gemm_f32" in libraries and "attention_tcgen05" not in libraries and "decode_linear" not in libraries


def test_the_loop_repeats_its_layers_in_a_row():
    from tesseract_b200.models.pekodra_config import PekodraConfig

    config = copy.deepcopy(TINY_PEKODRA["a"])
    config["loop"] = {"start": 2, "stop": 4, "times": 3}
    order = PekodraConfig.from_dict(config).run_order()
    assert order == ((0, False), (1, False), (2, True), (3, False), (2, True), (3, False), (2, True), (3, False))
    config["loop"] = {"start": 0, "stop": 4, "times": 2}
    assert [i for i, _ in PekodraConfig.from_dict(config).run_order()] == [0, 1, 2, 3, 0, 1, 2, 3]
    del config["loop"]
    assert PekodraConfig.from_dict(config).run_order() == ((0, False), (1, False), (2, False), (3, False))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "lstm"), "unknown type"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 2), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "experts", "ff": 8}), "unknown kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "loop"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_bad_configurations_are_refused(change, message):
    from tesseract_b200.models.pekodra_config import PekodraConfig

    config = copy.deepcopy(TINY_PEKODRA["a"])
    change(config)
    with pytest.raises(ConfigError, match=message):
        PekodraConfig.from_dict(config)


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations_describe_and_write(tmp_path, seed):
    config = random_config(seed)
    folder = write_random_model(str(tmp_path / "m"), config, seed=seed)
    _, _, spec = load_model_description(folder)
    loaded, tensors = plain.load_folder(folder)
    assert set(tensors) == set(expected_tensors(spec))
    assert len(spec.run_order) == len(plain.run_order(loaded))


def test_blended_frequencies_agree_with_the_plain_recipe():
    from tesseract_b200.parts.rotary import blended_inverse_frequencies

    for dims, base, scaling in [(64, 5e5, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
                                (8, 1000.0, {"factor": 3.0, "original": 64, "fast": 8.0, "slow": 1.0}),
                                (12, 500.0, {"factor": 16.0, "original": 8, "fast": 1.0, "slow": 0.25}),
                                (10, 30.0, None)]:
        got, amplitude = blended_inverse_frequencies(dims, base, scaling)
        want, want_amplitude = plain.blended_frequencies(dims, base, scaling)
        assert amplitude == pytest.approx(want_amplitude, rel=1e-12)
        assert list(got) == pytest.approx(want, rel=1e-12)
    # with a stretch, the fastest frequencies stay and the slowest are divided by the factor
    got, _ = blended_inverse_frequencies(64, 5e5, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0})
    assert got[0] == 1.0 and got[-1] == pytest.approx(5e5 ** (-62 / 64) / 8.0)


def test_a_window_gives_pages_back_while_the_request_lives():
    pages = PagedKeyValueNeed(num_kv_heads=2, key_dim=8, value_dim=4, window=21)
    assert [pages.first_needed_position(p) for p in (0, 20, 21, 85)] == [0, 0, 1, 65]
    # two runs of one layer: a group of two entries, each with storage of its own under the same page ids
    manager = CacheManager([pages, pages], [None, None], num_pages=6, page_size=16, max_requests=2,
                           dtype=torch.float32, device="cpu", max_step_tokens=16)
    first, second = manager.bindings
    assert first.group == second.group and first.storage is not second.storage
    assert manager.admit("a")
    held = []
    for _ in range(20):                                          # 200 tokens, ten at a time
        manager.extend("a", 10)
        manager.commit("a", 10)
        held.append(manager.used_pages())
    assert max(held) <= 4                                        # never the thirteen pages that 200 tokens would take
    manager.release("a")
    manager.check()
    assert manager.used_pages() == 0
