"""Vekedra's configuration and the tensors its parts declare (no GPU), and the plain implementation's own
consistency: a recurrence fed token by token equals the whole sequence, a window wider than the sequence is no window."""
import copy

import pytest
import torch

import plain_vekedra as pv
from vekedra_helpers import MIXED, ODD, dense, latent, mamba, config


def test_round_trip_and_registry():
    import cbis_b200 as cb
    assert "Vekedra" in cb.known_architectures()
    for cfgd in (MIXED, ODD):
        cfg = cb.config_from_dict(cfgd)
        assert type(cfg).__name__ == "VekedraConfig"
        assert cfg.to_dict() == cfgd
        assert cb.config_from_dict(cfg.to_dict()) == cfg


def test_spec_follows_the_layer_list():
    import cbis_b200 as cb
    spec = cb.config_from_dict(MIXED).model_spec()
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "mamba2", "latent_attention", "mamba2"]
    assert [l.feed_forward.kind for l in spec.layers] == ["gated", "routed", "nothing", "gated"]
    assert [l.cache_source for l in spec.layers] == [None, None, 0, None]
    assert all(l.arrangement == "parallel" for l in spec.layers)
    assert spec.layers[2].mixer.params["window"] == 17 and spec.layers[0].mixer.params["window"] == 10
    assert spec.token_embedding.params["multiplier"] == 4.0 and spec.max_positions == 0


def test_declared_tensors():
    import cbis_b200 as cb
    from cbis_b200.models import declared_tensors
    decl = {d.name: (tuple(d.shape), d.role) for d in declared_tensors(cb.config_from_dict(MIXED).model_spec())}
    assert decl["embed"] == ((96, 64), "table") and decl["head"] == ((96, 64), "matrix")
    assert decl["l0.norm1"] == ((64,), "norm_weight") and decl["l0.norm1.b"] == ((64,), "norm_bias")
    assert decl["final.norm.b"] == ((64,), "norm_bias")
    assert decl["l0.mix.dkv"][0] == (32, 64) and decl["l0.mix.uk"][0] == (32, 32) and decl["l0.mix.uv"][0] == (48, 32)
    assert "l2.mix.dkv" not in decl and "l2.mix.dkv.norm" not in decl and decl["l2.mix.q"][0] == (32, 64)
    assert decl["l1.mix.in"][0] == (2 * 32 + 2 * 2 * 16 + 4, 64) and decl["l1.mix.conv"][0] == (32 + 64, 3)
    assert decl["l1.mix.norm"] == ((32,), "norm_weight") and decl["l1.mix.A_log"] == ((4,), "vector")
    assert decl["l1.mlp.router"][0] == (5, 64) and decl["l1.mlp.e4.down"][0] == (64, 24) and "l1.mlp.e5.gate" not in decl
    assert not any(n.startswith("l2.mlp") for n in decl) and not any("norm2" in n for n in decl)


@pytest.mark.parametrize("change, message", [
    (lambda c: c.pop("vocab"), "'vocab' is missing"),
    (lambda c: c["layers"][0].update(type="conv"), "is not one of"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "keeps no latent"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "differs from layer 0"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "not a multiple of groups"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "exceeds experts"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "must be an integer >= 1"),
    (lambda c: c["norm"].update(eps=0), "positive number"),
])
def test_bad_configurations_are_refused(change, message):
    import cbis_b200 as cb
    c = copy.deepcopy(MIXED)
    change(c)
    with pytest.raises(cb.ConfigError, match=message):
        cb.config_from_dict(c)


def test_unknown_keys_are_reported_and_passed_over():
    import cbis_b200 as cb
    c = copy.deepcopy(MIXED)
    c["notes"] = "made on a Tuesday"
    c["layers"][1]["mixer"]["comment"] = 1
    with pytest.warns(UserWarning, match="unknown keys"):
        assert cb.config_from_dict(c) == cb.config_from_dict(MIXED)


def _weights(cfgd, seed):
    from vekedra_helpers import make_weights
    return {k: v.double() for k, v in make_weights(cfgd, seed).items()}


def test_plain_recurrence_token_by_token():
    """The plain state-space mixer is a recurrence: its output at t depends on tokens 0..t only, and
    a window wider than the sequence is the same as none."""
    w = _weights(ODD, 3)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, ODD["vocab"], (19,), generator=g).tolist()
    full = pv.forward(ODD, w, toks)
    for n in (1, 2, 7, 18):
        assert torch.allclose(pv.forward(ODD, w, toks[:n]), full[:n], atol=1e-9)
    wide = copy.deepcopy(ODD)
    wide["layers"][2]["mixer"]["mask"]["size"] = 19
    assert torch.allclose(pv.forward(wide, w, toks), full, atol=1e-12)
    narrow = copy.deepcopy(ODD)
    narrow["layers"][2]["mixer"]["mask"]["size"] = 18
    assert not torch.allclose(pv.forward(narrow, w, toks)[18], full[18], atol=1e-6)
    assert torch.allclose(pv.forward(narrow, w, toks)[:18], full[:18], atol=1e-12)


def test_plain_routing_takes_the_largest_scores_unrenormalized():
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=torch.float64)
    router = torch.tensor([[3.0, -1.0], [1.0, 1.0], [-2.0, 0.5]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    experts = [(eye * (e + 1), eye, eye) for e in range(3)]
    out = pv.routed_experts(h, router, experts, 1)
    s = torch.sigmoid(torch.tensor(3.0, dtype=torch.float64))
    v = s * h[0]
    assert torch.allclose(out[0], pv.silu(v * 1) * v)                      # row 0: expert 0 alone, fed s * h
    s1 = torch.sigmoid(torch.tensor(2.0, dtype=torch.float64))
    v1 = s1 * h[1]
    assert torch.allclose(out[1], pv.silu(v1 * 2) * v1)                    # row 1: expert 1 (score 2 beats 1 and -2)
