"""Murutar without a GPU: the configuration reader, the builder's tensor list against the one the
tests derive on their own, and the plain implementation against itself (a window as long as the
prompt is no window; the recurrence carried over a cut; the router's groups)."""
import copy

import pytest
import torch

import murutar_util as mu
import plain_murutar as plain
import replay_util as ru


@pytest.mark.parametrize("name", sorted(mu.CONFIGS))
def test_builder_asks_for_exactly_the_checkpoint_tensors(name):
    from dispec_b200.config.model_config import load_model_config
    from dispec_b200.weights.loader import build_model
    config = mu.CONFIGS[name]["config"]
    cfg = load_model_config(copy.deepcopy(config))
    assert load_model_config(cfg.to_dict()) == cfg
    req = build_model(cfg).tensor_requirements()
    want = mu.tensor_shapes(config)
    assert set(req) == set(want)
    for n, spec in req.items():
        assert tuple(spec.shape) == tuple(want[n]), n


def test_cache_groups_and_states_follow_the_layers():
    from dispec_b200.config.model_config import load_model_config
    from dispec_b200.weights.loader import build_model
    m = build_model(load_model_config(copy.deepcopy(mu.CONFIGS["mix"]["config"])))
    windows = sorted(g.window for g in m.cache_groups)
    assert windows == [0, 7, 20, 40]
    widths = {g.window: [(t.name, t.num_heads, t.width) for t in g.tensors] for g in m.cache_groups}
    assert widths[20] == [("key", 2, 16), ("value", 2, 8)] and widths[40] == [("key", 2, 24), ("value", 2, 8)]
    assert [tuple(s.shape) for s in m.state_needs] == [(3, 8, 12), (1, 16, 8)]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "not implemented"),
    (lambda c: c["layers"][0]["mixer"].pop("decay"), "decay"),
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=24), "agree"),
    (lambda c: c["layers"][1]["mlp"].update(kind="conv"), "not implemented"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors_name_the_key(change, word):
    from dispec_b200.config.model_config import ConfigError, load_model_config
    c = copy.deepcopy(mu.CONFIGS["mix"]["config"])
    change(c)
    with pytest.raises(ConfigError) as e:
        load_model_config(c)
    assert word in str(e.value)


def test_part_constructors_refuse_what_cannot_run():
    from dispec_b200.parts.moe import GroupedMoE
    from dispec_b200.parts.attention import SinkAttention
    with pytest.raises(ValueError):
        GroupedMoE(16, 8, 6, top=3, num_groups=3, keep_groups=1)  # three experts from a group of two
    with pytest.raises(ValueError):
        GroupedMoE(16, 8, 7, top=1, num_groups=2)
    with pytest.raises(ValueError):
        SinkAttention(16, 4, 3, 8, 8, 0.3, None)
    with pytest.raises(ValueError):
        SinkAttention(16, 4, 2, 8, 8, 0.3, None, value_mix=("other", "v"))


# ------------------------------------------------------------- the plain implementation itself
def test_plain_window_as_long_as_the_prompt_is_no_window():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(9, 4, 6, generator=g).double(), torch.randn(9, 2, 6, generator=g).double(),
               torch.randn(9, 2, 5, generator=g).double())
    a = plain.sink_window_attention(q, k, v, 0.4, 0)
    b = plain.sink_window_attention(q, k, v, 0.4, 9)
    c = plain.sink_window_attention(q, k, v, 0.4, 3)
    assert torch.allclose(a, b) and not torch.allclose(a, c)
    # the first token sees itself and the sink: its weight is exp(s) / (1 + exp(s))
    s = (q[0, 0] @ k[0, 0]) * 0.4
    assert torch.allclose(a[0, 0], torch.sigmoid(s) * v[0, 0])


def test_plain_recurrence_carries_its_state_over_a_cut():
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(11, 2, 4, generator=g).double(), torch.randn(11, 2, 4, generator=g).double(),
               torch.randn(11, 2, 3, generator=g).double())
    whole, S = plain.lightning_recurrence(q, k, v, [0.9, 1.0])
    a, Sa = plain.lightning_recurrence(q[:4], k[:4], v[:4], [0.9, 1.0])
    b, Sb = plain.lightning_recurrence(q[4:], k[4:], v[4:], [0.9, 1.0], state=Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(S, Sb)
    # o_t = sum over j <= t of decay^(t - j) (q_t . k_j) v_j
    t = 7
    want = sum(0.9 ** (t - j) * (q[t, 0] @ k[j, 0]) * v[j, 0] for j in range(t + 1))
    assert torch.allclose(whole[t, 0], want)


def test_plain_router_keeps_to_the_best_groups():
    router = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    s = torch.tensor([0.05, 0.30, 0.25, 0.02, 0.28, 0.10])
    assert sorted(plain.route(s, router).tolist()) == [0, 1]  # the group of the best expert only
    router["groups"]["keep"] = 2
    assert sorted(plain.route(s, router).tolist()) == [1, 4]  # groups {0,1} and {4,5}; expert 2 is shut out
    router["groups"] = {"count": 1, "keep": 1}
    assert sorted(plain.route(s, router).tolist()) == [1, 4]


def test_plain_forward_of_a_prefix_is_a_prefix():
    config = mu.CONFIGS["mix"]["config"]
    w = mu.random_weights(config, 3)
    ids = ru.random_ids(50, config["vocab"], 4)
    full, streams = plain.forward(config, w, ids)
    part, _ = plain.forward(config, w, ids[:31])
    assert torch.allclose(full[:31], part, atol=1e-9)
    assert streams.shape == (len(config["layers"]), 50, config["width"])
    assert full.abs().max() < 20.0  # squashed


def test_sharpening_makes_far_tokens_and_window_edges_matter():
    config = mu.CONFIGS["mix"]["config"]
    w = mu.sharpen(config, mu.random_weights(config, mu.CONFIGS["mix"]["seed"]))
    ids = ru.random_ids(120, config["vocab"], 5)
    a = plain.forward(config, w, ids)[0][-1]
    b = plain.forward(config, w, ids[6:])[0][-1]  # the linear-attention state no longer holds the first tokens
    assert (a - b).abs().max() > 0.05
