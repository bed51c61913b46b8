"""The Ridotar tests of tests/test_ridotar_gpu.py on the CPU with the stand-in kernels
(tests/standin_ops.py), in 32-bit: configuration, tensor naming, the block arrangement, state slots,
latent pages shared between layers, batching and the scheduler need no GPU to be checked, only the
kernels do.  Also: what the configuration reader refuses."""
import copy

import pytest

import ridotar_util as U
import standin_ops
import test_ridotar_gpu as G

HOST = dict(device="cpu", ops=standin_ops)


def test_each_mixer_alone_on_the_host(tmp_path):
    G.body_single_mixers(tmp_path, "float32", **HOST)


def test_portions_on_the_host(tmp_path):
    G.body_portions(tmp_path, "float32", name="mix_a", n=70, **HOST)


def test_mixed_batches_on_the_host(tmp_path):
    G.body_mixed_batches(tmp_path, "float32", name="mix_a", **HOST)
    G.body_mixed_batches(tmp_path, "float32", name="mix_b", **HOST)
    G.body_mixed_batches(tmp_path, "float32", name="mix_c", **HOST)


def test_greedy_generation_on_the_host(tmp_path):
    G.body_greedy(tmp_path, "float32", name="mix_b", **HOST)


def test_config_round_trip_and_names():
    from llm_singularity_b200.config.ridotar import RidotarConfig
    from llm_singularity_b200.engine.runner import expected_tensors_of
    cfg = RidotarConfig.from_dict(U.CONFIGS["mix_a"])
    assert RidotarConfig.from_dict(cfg.to_dict()) == cfg
    spec = cfg.to_model_spec()
    names = expected_tensors_of(spec)
    assert names["l0.mix.dkv"][0] == (40 + 12, 72) and "l2.mix.dkv" not in names        # layer 2 reads layer 0's
    assert "l1.norm2" not in names and "l1.mlp.router" not in names                      # no feed-forward there
    assert names["l2.mlp.e6.down"][0] == (72, 24) and names["side.embed"][0] == (211, 40)
    assert [c.cache for c in spec.order] == [0, 1, 0, 3] and [c.writes_cache for c in spec.order] == [True, True, False, True]


@pytest.mark.parametrize("change, text", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=44), "equal"),
    (lambda c: c["layers"][3]["mixer"].update(decay=[0.5]), "decays"),
    (lambda c: c["norm"].update(groups=5), "groups"),
    (lambda c: c["layers"][0].update(type="window"), "type"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c.pop("width"), "width"),
])
def test_config_refusals(change, text):
    from llm_singularity_b200.config.llama import ConfigError
    from llm_singularity_b200.config.ridotar import RidotarConfig
    cfg = copy.deepcopy(U.CONFIGS["mix_a"])
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        RidotarConfig.from_dict(cfg)
