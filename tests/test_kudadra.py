"""Kudadra without a device: its configuration and registry entry, tensor names, cache needs, and the plain
implementation checked against other formulations of the same mathematics."""
import math

import pytest
import torch

from lightllm_b200.cache import CacheManager
from lightllm_b200.config import ConfigError, config_from_dict, model_spec_for
from lightllm_b200.models import Model, weight_specs_of
from tests.kudadra_configs import CONFIGS, config, random_weights, tensor_shapes
from tests.plain import kudadra_plain as K


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_model_reads_exactly_the_tensors_of_the_design(name):
    spec = model_spec_for(config_from_dict(config(name)))
    got = {s.name: tuple(s.shape) for s in weight_specs_of(spec)}
    assert got == tensor_shapes(config(name))


def test_configuration_errors_name_the_key():
    for edit, word in ((lambda c: c.pop("width"), "width"), (lambda c: c["norm"].pop("eps"), "eps"),
                       (lambda c: c["layers"][0].update(type="conv"), "conv"),
                       (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
                       (lambda c: c["layers"][0]["mixer"].pop("kv_heads"), "kv_heads"),
                       (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
                       (lambda c: c["layers"][2]["mlp"].update(kind="routed"), "dense"),
                       (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank")):
        cfg = config("P")
        edit(cfg)
        with pytest.raises(ConfigError, match=word):
            config_from_dict(cfg)
    cfg = config("P")
    cfg["architecture"] = "Nobody"
    with pytest.raises(ConfigError, match="Nobody"):
        config_from_dict(cfg)


def test_cache_needs_follow_the_layers():
    lay = Model(model_spec_for(config_from_dict(config("P")))).cache_layout
    # two windowed groups of different geometry, one latent group without values, one state plane
    assert [(g.kv_heads, g.head_dim, g.value_dim, g.window) for g in lay.groups] == \
        [(2, 12, 20, 11), (1, 28, 0, None), (3, 20, 12, 40)]
    assert [s.shape for s in lay.state_planes] == [(3, 12, 20)]
    assert lay.bytes_per_token(2) == 2 * (2 * (12 + 20) + 28 + 3 * (20 + 12))
    lay = Model(model_spec_for(config_from_dict(config("R")))).cache_layout
    assert lay.groups == [] and [s.shape for s in lay.state_planes] == [(1, 16, 16), (2, 8, 24)]
    mgr = CacheManager(lay, 16, [], 2, 64)          # a model without pages still has slots and lengths
    a = mgr.open("a")
    mgr.reserve("a", 40)
    mgr.advance("a", 40)
    assert not mgr.can_reserve("a", 30) and mgr.can_reserve("a", 24)
    mgr.close("a")
    assert mgr.open("b").slot == a.slot             # the slot that was just freed is used again
    mgr.check()


def test_plain_retention_is_the_decayed_sum():
    torch.manual_seed(0)
    T, D = 9, 10
    m = {"heads": 2, "dim": 4, "vdim": 3, "decay": [0.8, 0.95], "rot": {"dims": 2, "base": 50.0}}
    w = {k: torch.randn(n, D, dtype=torch.float64) for k, n in (("q", 8), ("k", 8), ("v", 6), ("g", 6))}
    w["o"] = torch.randn(D, 6, dtype=torch.float64)
    h = torch.randn(T, D, dtype=torch.float64)
    got = K.plain_retention(h, w, m, 1e-5)
    pos = torch.arange(T)
    q = K.plain_rotate((h @ w["q"].T).view(T, 2, 4), pos, 2, 50.0)
    k = K.plain_rotate((h @ w["k"].T).view(T, 2, 4), pos, 2, 50.0) / 2.0
    v = (h @ w["v"].T).view(T, 2, 3)
    o = torch.zeros(T, 2, 3, dtype=torch.float64)
    for hh in range(2):
        for t in range(T):
            for j in range(t + 1):
                o[t, hh] += m["decay"][hh] ** (t - j) * torch.dot(q[t, hh], k[j, hh]) * v[j, hh]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)
    z = h @ w["g"].T
    want = (o.reshape(T, 6) * z / (1 + torch.exp(-z))) @ w["o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_plain_latent_attention_sink_is_a_key_without_value():
    torch.manual_seed(1)
    T, D = 7, 12
    m = {"heads": 2, "dim": 4, "vdim": 5, "kv_rank": 6, "scale": 0.3}
    w = {"q": torch.randn(8, D), "dkv": torch.randn(6, D), "dkv.norm": torch.rand(6) + 0.5, "uk": torch.randn(8, 6),
         "uv": torch.randn(10, 6), "sink": torch.tensor([0.7, -1.2]), "g": torch.randn(2, D), "o": torch.randn(D, 10)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, D, dtype=torch.float64)
    got = K.plain_latent_attention(h, w, m, 1e-5)
    c = h @ w["dkv"].T
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + 1e-5) * w["dkv.norm"]
    rows = []
    for t in range(T):
        heads = []
        for hh in range(2):
            q = (w["q"] @ h[t])[hh * 4:(hh + 1) * 4]
            logits = [float(torch.dot(q, w["uk"][hh * 4:(hh + 1) * 4] @ c[j])) * 0.3 for j in range(t + 1)]
            logits.append(float(w["sink"][hh]))                       # one more logit, its value is zero
            p = torch.softmax(torch.tensor(logits, dtype=torch.float64), 0)
            val = sum(p[j] * (w["uv"][hh * 5:(hh + 1) * 5] @ c[j]) for j in range(t + 1))
            heads.append(val * torch.sigmoid(torch.dot(w["g"][hh], h[t])))
        rows.append(w["o"] @ torch.cat(heads))
    assert torch.allclose(got, torch.stack(rows), atol=1e-10)


def test_plain_rotation_and_window():
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    pos = torch.tensor([0, 1, 2, 50, 1000])
    y = K.plain_rotate(x, pos, 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])          # position 0 and the unrotated rest
    assert torch.allclose((y[..., :4] ** 2).sum(-1), (x[..., :4] ** 2).sum(-1))
    a = 50 * 100.0 ** (-2 * 1 / 4)                                                   # pair (1, 3) at position 50
    assert torch.allclose(y[3, 0, 1], x[3, 0, 1] * math.cos(a) - x[3, 0, 3] * math.sin(a))
    assert torch.allclose(y[3, 0, 3], x[3, 0, 3] * math.cos(a) + x[3, 0, 1] * math.sin(a))
    # a window of w keeps w keys: with equal values on all keys but one, that key counts until it is w back
    cfg = config("S")
    w = {k: v.double() for k, v in random_weights(cfg, 3).items()}
    toks = [5, 9, 9, 9, 9]
    full = K.plain_forward(toks, w, cfg)
    assert torch.allclose(full[1], K.plain_forward(toks[:2], w, cfg)[1], atol=1e-12)


def test_gated_feed_forward_rejects_what_it_does_not_have():
    from lightllm_b200.parts import GatedMLP
    with pytest.raises(ValueError, match="relu"):
        GatedMLP("x", 8, 8, activation="relu")
    with pytest.raises(ValueError, match="limit"):
        GatedMLP("x", 8, 8, activation="clamped_swish")
