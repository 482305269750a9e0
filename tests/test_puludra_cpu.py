"""Puludra on the CPU: configuration, registry, the model built from it (tensor names and
shapes, caches, states), and the plain implementation's own consistency."""
import copy

import pytest
import torch

import plain_puludra as plain
import puludra_util as pu

from dispec_b200 import load_model_config
from dispec_b200.config.model_config import ConfigError
from dispec_b200.weights.loader import build_model


@pytest.mark.parametrize("name", sorted(pu.CONFIGS))
def test_model_declares_exactly_the_tensors_of_the_design(name):
    config = pu.CONFIGS[name]["config"]
    cfg = load_model_config(config)
    assert cfg.architecture == "Puludra" and cfg.to_dict() == config
    model = build_model(cfg)
    req = model.tensor_requirements()
    want = plain.tensor_shapes(config)
    assert {k: tuple(v.shape) for k, v in req.items()} == want
    # gains, gate bounds and activation parameters stay 32-bit in every mode
    for k, spec in req.items():
        small = k.endswith(("norm", "norm1", "norm2", "lower", "f.b", "act"))
        assert (spec.dtype == "float32") == small, k


def test_every_layer_run_has_a_cache_or_state_of_its_own():
    cfg = load_model_config(pu.CONFIGS["mix"]["config"])
    model = build_model(cfg)
    assert [c.layer for c in model.schedule] == [0, 1, 2, 0]  # the fourth runs the first's weights
    assert len(model.layers) == 3
    assert len(model.cache_groups) == 1 and model.cache_groups[0].num_slots == 2
    names = [(t.name, t.num_heads, t.width) for t in model.cache_groups[0].tensors]
    assert names == [("latent", 1, 40), ("rotated_key", 1, 8)]
    assert [s.shape for s in model.state_needs] == [(2, 16, 16), (3, 16, 32)]
    later = build_model(load_model_config(pu.CONFIGS["odd"]["config"]))
    assert [c.layer for c in later.schedule] == [0, 1, 2, 1] and len(later.layers) == 3


def test_configuration_errors_name_the_key():
    good = pu.CONFIGS["mix"]["config"]
    for path, value, text in [
            (("layers", 1, "type"), "mamba", "not implemented"),
            (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
            (("layers", 2, "mixer", "decay"), [0.5], "decays"),
            (("layers", 2, "mixer", "rot", "dims"), 7, "rot.dims"),
            (("layers", 3, "weights_of"), 3, "weights_of"),
            (("layers", 0, "mlp", "kind"), "routed", "mlp.kind"),
            (("norm",), None, "norm")]:
        bad = copy.deepcopy(good)
        at = bad
        for k in path[:-1]:
            at = at[k]
        if value is None:
            del at[path[-1]]
        else:
            at[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            load_model_config(bad)
    circle = copy.deepcopy(good)
    circle["layers"][0]["weights_of"] = 3
    with pytest.raises(ConfigError, match="circle"):
        load_model_config(circle)


def test_plain_prefix_property_and_rotation_layouts():
    """The plain implementation is causal (a prefix's logits do not change when tokens follow),
    and its two rotations turn the pairs they say they turn."""
    config, seed = pu.CONFIGS["mix"]["config"], 3
    w = plain.random_weights(config, seed)
    ids = torch.randint(0, config["vocab"], (23,), generator=torch.Generator().manual_seed(1)).tolist()
    full = plain.forward(w, config, ids)
    part = plain.forward(w, config, ids[:9])
    assert torch.allclose(full[:9], part, atol=1e-9)
    x = torch.zeros(1, 1, 8, dtype=torch.float64)
    x[0, 0, 0] = 1.0
    pos = torch.tensor([3])
    a = plain.rotate_interleaved(x, pos, 10.0, 4)[0, 0]
    b = plain.rotate_halves(x, pos, 10.0, 4)[0, 0]
    assert a[1].abs() > 0.1 and a[2] == 0 and b[2].abs() > 0.1 and b[1] == 0
    assert torch.allclose(a[[0, 1]], torch.tensor([torch.cos(torch.tensor(3.0)), torch.sin(torch.tensor(3.0))]).double())


def test_xielu_is_continuous_and_matches_its_two_branches():
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64)
    z = torch.tensor([-2.0, -1e-9, 0.0, 1e-9, 1.5], dtype=torch.float64)
    y = plain.xielu(z, p, q)
    assert abs(float(y[1] - y[3])) < 1e-8 and float(y[2]) == 0.0
    sp = torch.nn.functional.softplus
    assert torch.isclose(y[4], sp(p) * 2.25 + 0.75)
    assert torch.isclose(y[0], (0.5 + sp(q)) * (torch.exp(z[0]) - 1 - z[0]) + z[0] / 2)
