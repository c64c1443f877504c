"""Kodupel pieces that need no GPU: the oracle's own consistency, config parsing and validation, tensor shapes, and the
registry entry."""
import copy
import math

import numpy as np
import pytest

from tests import kodupel_oracle as orc
from tests.test_kodupel_gpu import CFG_MIXED, CFG_ONES, CFG_WIDE
from zhilight_b200.kodupel import KodupelConfig


def _weights(cfg, seed=0):
    return {k: v.astype(np.float64) for k, v in orc.random_weights(cfg, seed).items()}


def test_config_round_trip_and_shapes():
    for d in (CFG_MIXED, CFG_ONES, CFG_WIDE):
        cfg = KodupelConfig.from_dict(d)
        again = KodupelConfig.from_dict(cfg.to_dict())
        for a, b in zip(cfg.layers, again.layers):
            assert {k: v for k, v in a.items() if k != "decay_rank"} == {k: v for k, v in b.items() if k != "decay_rank"}
        shapes = cfg.tensor_shapes()
        assert shapes["embed"] == (cfg.vocab, cfg.width) and shapes["final.norm"] == (cfg.width,)
    cfg = KodupelConfig.from_dict(CFG_MIXED)
    s = cfg.tensor_shapes()
    assert "l2.mix.k" not in s and "l2.mix.v.b" not in s and "l2.mix.q" in s        # a layer on another layer's cache
    assert "l1.norm2" not in s and "l1.mlp.router" not in s                           # a layer without feed-forward
    assert s["l0.mix.g"] == (4, 48) and s["l3.mix.w2"] == (48, 7) and s["l0.mlp.e4.down"] == (48, 20)


def test_config_validation():
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][2]["mixer"]["kv_from"] = 1            # a delta-rule layer has no cache to lend
    with pytest.raises(ValueError):
        KodupelConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][0]["mixer"]["kv_from"] = 2            # not an earlier layer
    with pytest.raises(ValueError):
        KodupelConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        KodupelConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][0]["type"] = "latent_attention"
    with pytest.raises(ValueError):
        KodupelConfig.from_dict(bad)
    bad = copy.deepcopy(CFG_MIXED)
    bad["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(ValueError):
        KodupelConfig.from_dict(bad)


def test_registry_knows_the_family():
    from zhilight_b200 import registry
    assert "Kodupel" in registry.registered()
    assert registry.supported_dtypes(CFG_ONES) == ("bfloat16", "float32")


def test_oracle_is_causal_and_scan_composes():
    cfg = KodupelConfig.from_dict(CFG_MIXED)
    W = _weights(cfg, 3)
    toks = np.random.default_rng(0).integers(0, cfg.vocab, 30).tolist()
    full = orc.forward(cfg, W, toks)[0]
    part = orc.forward(cfg, W, toks[:17])[0]
    assert np.abs(full[:17] - part).max() < 1e-9
    rng = np.random.default_rng(1)
    r, k, v = (rng.standard_normal((12, 2, 6)) for _ in range(3))
    w, a = rng.random((12, 2, 6)), rng.random((12, 2, 6))
    o, S = orc.delta_rule_scan(r, k, v, w, a)
    o1, S1 = orc.delta_rule_scan(r[:5], k[:5], v[:5], w[:5], a[:5])
    o2, S2 = orc.delta_rule_scan(r[5:], k[5:], v[5:], w[5:], a[5:], S0=S1)
    assert np.abs(np.concatenate([o1, o2]) - o).max() < 1e-12 and np.abs(S2 - S).max() < 1e-12


def test_oracle_mechanisms_by_hand():
    # one key: p = e^s / (1 + e^s); with a second, far lower score nothing changes visibly
    q, k, v = np.ones((1, 1, 2)), np.ones((1, 1, 2)), np.array([[[3.0, 5.0]]])
    out = orc.unit_sink_attention(q, k, v, 0.5)
    assert np.allclose(out[0, 0], np.array([3.0, 5.0]) * math.e / (1 + math.e))
    # rotation by a quarter turn of the first pair only
    cos, sin = np.array([[0.0]]), np.array([[1.0]])
    x = np.array([[[1.0, 2.0, 7.0, 9.0]]])
    assert np.allclose(orc.rotate_pairs(x, cos, sin, 2), [[[-2.0, 1.0, 7.0, 9.0]]])
    # no scaling: plain geometric frequencies, unit magnitude
    cos, sin = orc.rotation_tables(3, 4, 100.0, None)
    assert np.allclose(cos[2], [math.cos(2.0), math.cos(0.2)]) and np.allclose(sin[1], [math.sin(1.0), math.sin(0.1)])
    # scaling: fast dimensions keep their frequency, slow ones are divided by the factor, cos^2 + sin^2 = magnitude^2
    cos, sin = orc.rotation_tables(2, 8, 10000.0, dict(factor=4.0, original=64, fast=16.0, slow=2.0))
    f = np.arctan2(sin[1], cos[1])
    plain = 10000.0 ** (-2.0 * np.arange(4) / 8)
    assert np.isclose(f[0], plain[0]) and np.isclose(f[3], plain[3] / 4.0)
    assert np.allclose(cos[1] ** 2 + sin[1] ** 2, (0.1 * math.log(4.0) + 1) ** 2)
    # the gated unit clamps before the product; the correction picks the expert but does not weigh it
    W = {"gate": np.array([[10.0]]), "up": np.array([[-10.0]]), "down": np.array([[1.0]])}
    assert np.isclose(orc.expert(W, "", np.array([1.0]), 2.0)[0], 2.0 * orc.sigmoid(1.702 * 2.0) * (-2.0 + 1.0))
    chosen, weight = orc.route(np.array([[1.0]]), np.array([[0.0], [2.0]]), np.array([5.0, 0.0]), 1)
    assert chosen[0, 0] == 0 and np.isclose(weight[0, 0], 0.5)


def test_family_libraries_name_existing_sources():
    """A checkout without built files compiles only a family's sources: they must exist, and hold the family's driver."""
    import os
    from zhilight_b200 import build
    for family, names in build.FAMILY_SOURCES.items():
        assert family + "_runner" in names and "misc" in names
        for n in names:
            assert os.path.exists(os.path.join(build.CSRC, n + ".cu")), (family, n)
        assert build.family_lib_path(family).endswith("libzhilight_b200_%s.so" % family)
