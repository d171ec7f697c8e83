"""Figotar's configuration, its tensor declarations and the plain implementation's own consistency (no GPU)."""
import copy

import numpy as np
import pytest

import plain_figotar as pf
from figotar_helpers import MIXED, ODD, WIDE, as_numpy, attn, config, dense, latent, make_weights, mlstm


def test_round_trip_and_registry():
    import cbis_b200 as cb
    for cfgd in (MIXED, ODD, WIDE):
        c = cb.config_from_dict(cfgd)
        assert type(c).__name__ == "FigotarConfig" and c.to_dict() == cfgd
        spec = c.model_spec()
        assert [l.arrangement for l in spec.layers] == ["sandwich"] * len(cfgd["layers"])
        assert spec.max_positions == 0 and spec.vocab_size == cfgd["vocab"]


def test_declared_tensors_follow_the_sizes():
    import cbis_b200 as cb
    from cbis_b200.models import Model
    decl = {d.name: tuple(d.shape) for d in Model(cb.config_from_dict(ODD).model_spec()).declared()}
    assert decl["embed"] == (61, 40) and decl["head"] == (61, 40) and decl["final.norm"] == (40,)
    assert decl["l0.mix.q"] == (12, 40) and decl["l0.mix.v"] == (20, 40) and decl["l0.mix.g"] == (20, 40)
    assert decl["l0.mix.i"] == (1, 40) and decl["l0.mix.f.b"] == (1,) and decl["l0.mix.norm"] == (20,)
    assert decl["l1.mix.q"] == (36, 40) and decl["l1.mix.k"] == (12, 40) and decl["l1.mix.v.b"] == (20,)
    assert decl["l1.mix.g"] == (3, 40) and decl["l1.mix.o"] == (40, 60) and "l1.mix.g.b" not in decl
    assert "l1.norm2" not in decl and "l1.mlp.gate" not in decl and decl["l1.norm1b"] == (40,)   # no feed-forward
    assert decl["l2.mix.dq"] == (12, 40) and decl["l2.mix.uq"] == (3 * 16, 12) and decl["l2.mix.dkv"] == (24, 40)
    assert decl["l2.mix.dkv.norm"] == (18,) and decl["l2.mix.uk"] == (30, 18) and decl["l2.mix.uv"] == (42, 18)
    assert decl["l2.mix.sink"] == (3,) and decl["l2.mix.g"] == (3, 40) and decl["l2.mix.o"] == (40, 42)
    assert decl["l2.mlp.gate.b"] == (56,) and decl["l2.mlp.down"] == (40, 56) and decl["l2.mlp.down.b"] == (40,)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "is not one of"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "'scale' is missing"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "at most rot_dim"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=3), "even"),
    (lambda c: c["layers"][1]["mixer"].update(gate_cap=0), "positive"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "is not one of"),
    (lambda c: c.pop("norm"), "'norm' is missing"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_bad_configurations_are_refused(change, message):
    import cbis_b200 as cb
    cfgd = copy.deepcopy(MIXED)
    change(cfgd)
    with pytest.raises(cb.ConfigError, match=message):
        cb.config_from_dict(cfgd)


def test_mixers_refuse_sizes_no_kernel_takes():
    import cbis_b200 as cb
    from cbis_b200.models import Model
    for layer in (attn(2, 2, 600, 16, 8, 0.1), latent(2, 16, 64, 16, 500, 16, 0.1), mlstm(2, 600, 16)):
        with pytest.raises(ValueError, match="outside"):
            Model(cb.config_from_dict(config(32, 40, [layer])).model_spec())


def test_plain_memory_carries_its_state():
    """The plain recurrence from a state equals the recurrence over the whole sequence."""
    g = np.random.default_rng(3)
    T, H, D, V = 23, 2, 5, 7
    q, k = g.normal(size=(T, H, D)), g.normal(size=(T, H, D))
    v = g.normal(size=(T, H, V))
    li, lf = pf.capped_gates(3 * g.normal(size=(T, H)), 3 * g.normal(size=(T, H)) + 2, 4.0)
    whole, end = pf.memory_steps(q, k, v, li, lf)
    first, mid = pf.memory_steps(q[:9], k[:9], v[:9], li[:9], lf[:9])
    rest, end2 = pf.memory_steps(q[9:], k[9:], v[9:], li[9:], lf[9:], mid)
    assert np.abs(np.concatenate([first, rest]) - whole).max() < 1e-12
    assert all(np.abs(a - b).max() < 1e-12 for a, b in zip(end, end2))
    assert (li <= 4.0).all() and (lf < 0).all()


def test_plain_attention_pieces():
    g = np.random.default_rng(4)
    assert pf.query_temperature(14, 0.5, 16) == 1.0 and pf.query_temperature(15, 0.5, 16) == 1.0 + 0.5 * np.log(2)
    assert np.allclose(pf.distance_slopes(4), [0.25, 0.0625, 2.0 ** -6, 2.0 ** -8])
    s = g.normal(size=6)
    w = pf.softmax_with_sink(s, 0.7)
    assert abs(w.sum() + np.exp(0.7) / (np.exp(s).sum() + np.exp(0.7)) - 1) < 1e-12
    assert abs(pf.softmax_with_sink(s).sum() - 1) < 1e-12
    x = g.normal(size=(3, 2, 8))
    r = pf.rotate_half(x, [0, 1, 5], 100.0, 4)
    assert np.allclose(r[0], x[0]) and np.allclose(r[..., 4:], x[..., 4:])            # position 0 and the tail pass unchanged
    assert np.allclose((r[..., :4] ** 2).sum(-1), (x[..., :4] ** 2).sum(-1))          # a rotation keeps the length
    a = 5 * 100.0 ** (-2 * 1 / 4)
    assert np.allclose(r[2, 0, 1], x[2, 0, 1] * np.cos(a) - x[2, 0, 3] * np.sin(a))


def test_plain_window_and_first_tokens():
    """A query sees itself and window - 1 tokens before it; the first tokens see what there is."""
    g = np.random.default_rng(5)
    T, H, D = 12, 2, 4
    q, k, v = g.normal(size=(T, H, D)), g.normal(size=(T, 1, D)), g.normal(size=(T, 1, 3))
    out = pf.attention_rows(q, k, v, 0.5, window=4)
    assert np.allclose(out[0, 0], v[0, 0])
    k2, v2 = k.copy(), v.copy()
    k2[:5] += 9.0
    v2[:5] -= 3.0
    assert np.allclose(pf.attention_rows(q, k2, v2, 0.5, window=4)[8:], out[8:])      # keys 0..4 are outside from row 8 on
    assert not np.allclose(pf.attention_rows(q, k2, v2, 0.5, window=4)[7], out[7])    # row 7 still sees key 4


def test_random_weights_keep_activations_in_range():
    w = make_weights(MIXED, 3)
    logits, stream = pf.forward(MIXED, as_numpy(w), list(range(20)))
    assert np.isfinite(logits).all() and 0.1 < np.abs(stream[-1]).mean() < 50
