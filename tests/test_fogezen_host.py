"""The Fogezen design's host side: configuration, run order, parameter names, cache needs and the
plain model's own consistency.  No GPU."""
import pytest
import torch

import fogezen_util as U
import plain_fogezen as P


def _config(cfg):
    from llm_singularity_b200.config.fogezen import FogezenConfig
    return FogezenConfig.from_dict(cfg)


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_configuration_round_trip_and_registry(name, tmp_path):
    from llm_singularity_b200.registry import load_config
    cfg = U.CONFIGS[name]
    c = _config(cfg)
    assert c.to_dict() == cfg
    U.write_model(str(tmp_path), cfg, {"embed": torch.zeros(2, 2)})
    assert load_config(str(tmp_path)) == c


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_run_order_and_caches(name):
    """The spec's run order is the plain model's; every run of a layer has a cache of its own; the
    first call of every pass through the loop carries the pass's number."""
    cfg = U.CONFIGS[name]
    spec = _config(cfg).to_model_spec()
    assert [(c.block, c.step) for c in spec.order] == P.run_order(cfg)
    assert [c.cache for c in spec.order] == list(range(len(spec.order)))
    assert spec.step_vectors == (cfg["loop"]["times"] if "loop" in cfg else 0)


def test_parameters_and_cache_kinds():
    from llm_singularity_b200.engine.runner import expected_tensors_of
    from llm_singularity_b200.models.decoder import DecoderModel
    from llm_singularity_b200.parts import CompositeCacheSpec, PagedKVSpec, Runtime, StateSpec
    cfg = U.CONFIGS["mix_a"]
    spec = _config(cfg).to_model_spec()
    names = expected_tensors_of(spec)
    assert names["l0.mix.left.q.norm"][0] == (32,) and names["l0.mix.right.i.b"][0] == (3,)
    assert names["l1.mix.q.b"][0] == (96,) and names["loop.step"][0] == (2, 72)
    assert "l2.norm2" not in names and "l2.norm2" in spec.ignorable          # the layer without feed-forward
    model = DecoderModel(spec, Runtime("cpu", torch.float32, ops=object()))
    caches = model.cache_specs()
    assert len(caches) == 5                                                    # layers 0, 1, 0, 1, 2
    pair = caches[0]
    assert isinstance(pair, CompositeCacheSpec) and pair.paged and not pair.shareable and pair.window is None
    assert pair.parts[0] == PagedKVSpec(2, 32, None, 16)
    assert pair.parts[1].parts == (StateSpec((3, 25, 16)), StateSpec((3,)))
    assert caches[1] == PagedKVSpec(3, 16, None, 32) and caches[4] == PagedKVSpec(2, 48, None, None)
    assert pair.bytes_per_page(16, 2) == 2 * 16 * (32 + 16) * 2


def test_bad_configurations_are_refused():
    from llm_singularity_b200.config.llama import ConfigError
    for change in (lambda c: c["layers"][0].update(type="other"),
                   lambda c: c["loop"].update(stop=9),
                   lambda c: c["layers"][1]["mixer"].update(kv_heads=4),
                   lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=15),
                   lambda c: c["layers"][0]["mlp"].update(kind="moe")):
        import copy
        cfg = copy.deepcopy(U.CONFIGS["mix_a"])
        change(cfg)
        with pytest.raises(ConfigError):
            _config(cfg)


def test_plain_memory_carries_its_state():
    """The plain matrix memory walked in two halves from the carried state equals one walk, and the
    plain chunked mask lets a query see exactly the keys of its own stretch."""
    cfg = U.single("parallel")
    W = {n: t.double() for n, t in U.make_weights(cfg, 3).items()}
    m = cfg["layers"][0]["mixer"]["right"]
    h = torch.randn(30, cfg["width"], dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    whole, _ = P.matrix_memory(h, W, "l0.mix.right.", m, 1e-5)
    a, st = P.matrix_memory(h[:13], W, "l0.mix.right.", m, 1e-5)
    b, _ = P.matrix_memory(h[13:], W, "l0.mix.right.", m, 1e-5, st)
    assert (torch.cat([a, b]) - whole).abs().max() < 1e-12
    ok = P.visible(torch.arange(12), 5)
    assert ok[7].tolist() == [False] * 5 + [True] * 3 + [False] * 4 and ok[10].tolist() == [False] * 10 + [True, False]
