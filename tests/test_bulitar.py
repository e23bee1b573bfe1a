"""Bulitar without a device: configuration, tensor names, run list, cache needs, and the plain functions against other
formulations of the same mechanisms."""
import copy
import math

import pytest
import torch

from lightllm_b200.cache import CacheManager
from lightllm_b200.config import ConfigError, config_from_dict, model_spec_for
from lightllm_b200.models.model import Model
from tests.bulitar_configs import CONFIGS, config, file_config, random_weights, tensor_shapes
from tests.plain import bulitar_plain as P


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    cfg = config(name)
    model = Model(model_spec_for(config_from_dict(cfg)))
    got = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert got == tensor_shapes(cfg)


def test_ranks_come_from_the_checkpoint_when_the_configuration_leaves_them_out(tmp_path):
    from lightllm_b200.config import load_config
    from tests.bulitar_configs import write_model
    cfg = config("U")
    d = write_model(cfg, random_weights(cfg, 1, store=torch.bfloat16), str(tmp_path / "m"))
    loaded = load_config(d)
    assert [l.mixer.get("decay_rank") for l in loaded.layers] == [None, 5, None, 3]
    assert [l.mixer.get("gate_rank") for l in loaded.layers] == [None, 7, None, 4]
    assert loaded.to_json_dict()["layers"][1]["mixer"]["decay_rank"] == 5          # the configuration stands on its own
    with pytest.raises(ConfigError, match="decay_rank"):
        config_from_dict(file_config(cfg))


def test_run_list_follows_the_loop():
    for name, want in (("U", [0, 1, 2, 1, 2, 1, 2, 3]), ("V", [0, 1, 2, 3, 4] * 2), ("W", [0, 1, 2]), ("X", [0, 1, 2])):
        spec = model_spec_for(config_from_dict(config(name)))
        assert [e.layer for e in spec.run] == want == [i for i, _ in P.run_list(config(name))]
        enters = [i for i, e in enumerate(spec.run) if e.enter is not None]
        assert enters == [i for i, (_, opens) in enumerate(P.run_list(config(name))) if opens is not None]
        assert [spec.run[i].enter.params["index"] for i in enters] == list(range(len(enters)))
    # every pass has cache and state of its own
    layout = Model(model_spec_for(config_from_dict(config("U")))).cache_layout
    assert sum(layout.planes_per_group) == 4 and len(layout.state_planes) == 8


@pytest.mark.parametrize("edit,match", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown 'type'"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0]["mixer"].update(conv=0), "conv"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].pop("times"), "times"),
])
def test_configuration_errors_name_the_key(edit, match):
    cfg = config("U")
    edit(cfg)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(cfg)


def test_an_empty_loop_and_a_layer_without_convolution():
    cfg = config("U")
    cfg["loop"] = {"start": 2, "stop": 2, "times": 3}
    cfg["layers"][0]["mixer"].pop("conv")
    spec = model_spec_for(config_from_dict(cfg))
    assert [e.layer for e in spec.run] == [0, 1, 2, 3] and all(e.enter is None for e in spec.run)
    assert [i for i, _ in P.run_list(dict(cfg, loop=None))] == [0, 1, 2, 3]
    names = {s.name for s in Model(spec).weight_specs()}
    assert "l0.mix.q.conv" not in names and "l2.mix.q.conv" in names and "loop.in" not in names
    assert spec.ignored_suffixes == ("loop.in", "loop.step")          # such a checkpoint may still carry them


def test_pages_of_earlier_chunks_are_given_back():
    model = Model(model_spec_for(config_from_dict(config("U"))))
    layout = model.cache_layout
    assert sorted(g.chunk for g in layout.groups) == [11, 37]
    cm = CacheManager(layout, 4, 64, 2, 256)
    cm.open("a")
    g11 = [g.chunk for g in layout.groups].index(11)
    for n in (9, 3, 30, 1, 1):
        cm.reserve("a", n)
        cm.advance("a", n)
        cm.check()
        length = cm.get("a").length
        for g, spec in enumerate(layout.groups):
            first = (length // spec.chunk) * spec.chunk          # the next query's chunk begins here
            table = cm.block_table("a", g)
            assert all((p < 0) == ((i + 1) * 4 <= first) for i, p in enumerate(table)), (length, spec.chunk, table)
    assert cm.used_pages(g11) == sum(p >= 0 for p in cm.block_table("a", g11)) <= 3 + 1
    cm.close("a")
    assert all(cm.free_pages(g) == 64 for g in range(len(layout.groups)))


# ---- the plain functions against other formulations ----------------------------------------------------------------
def test_short_convolution_against_conv1d():
    torch.manual_seed(0)
    u, w = torch.randn(23, 7, dtype=torch.float64), torch.randn(7, 4, dtype=torch.float64)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=7)[0].T
    assert torch.allclose(P.short_conv(u, w), want, atol=1e-12)
    assert torch.allclose(P.short_conv(u, torch.ones(7, 1, dtype=torch.float64) * 2), 2 * u)


def test_chunked_attention_against_a_masked_softmax():
    torch.manual_seed(1)
    T, H, G, d, e = 29, 4, 2, 6, 5
    q, k, v = (torch.randn(T, n, w, dtype=torch.float64) for n, w in ((H, d), (G, d), (G, e)))
    for chunk in (None, 1, 7, 29, 100):
        i = torch.arange(T)
        see = i[None, :] <= i[:, None]
        if chunk:
            see &= (i[None, :] // chunk) == (i[:, None] // chunk)
        kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
        s = torch.einsum("ihd,jhd->hij", q, kk) * 0.7
        p = torch.softmax(s.masked_fill(~see, -math.inf), -1)
        want = torch.einsum("hij,jhe->ihe", p, vv)
        assert torch.allclose(P.chunked_softmax_attention(q, k, v, 0.7, chunk), want, atol=1e-12)


def test_delta_rule_against_explicit_matrices():
    """S_t = (I - beta k k^T) diag(g) S_(t-1) + beta k v^T, written with matrices instead of the three steps."""
    torch.manual_seed(2)
    T, d, e = 17, 5, 4
    q, k = torch.randn(T, d, dtype=torch.float64), torch.nn.functional.normalize(torch.randn(T, d, dtype=torch.float64), dim=-1)
    v, g, beta = torch.randn(T, e, dtype=torch.float64), torch.rand(T, d, dtype=torch.float64), torch.rand(T, dtype=torch.float64)
    S = torch.zeros(d, e, dtype=torch.float64)
    want = []
    for t in range(T):
        S = (torch.eye(d, dtype=torch.float64) - beta[t] * torch.outer(k[t], k[t])) @ torch.diag(g[t]) @ S \
            + beta[t] * torch.outer(k[t], v[t])
        want.append(S.T @ q[t])
    assert torch.allclose(P.delta_rule(q, k, v, g, beta), torch.stack(want), atol=1e-12)
    # with beta = 1 and no decay, a unit key reads back the value that was just written
    out = P.delta_rule(k, k, v, torch.ones(T, d, dtype=torch.float64), torch.ones(T, dtype=torch.float64))
    assert torch.allclose(out, v, atol=1e-12)


def test_rotation_frequencies():
    rot = {"dims": 8, "base": 100.0}
    f, m = P.rotary_frequencies(rot)
    assert m == 1.0 and torch.allclose(f, torch.tensor([100.0 ** (-i / 4) for i in range(4)], dtype=torch.float64))
    # a factor of 1 changes nothing; a large factor divides exactly the pairs beyond the ramp
    same, m1 = P.rotary_frequencies(dict(rot, scaling={"factor": 1.0, "original": 64, "fast": 8.0, "slow": 1.0}))
    assert m1 == 1.0 and torch.allclose(same, f)
    sc = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    scaled, m4 = P.rotary_frequencies(dict(rot, scaling=sc))
    assert abs(m4 - (0.1 * math.log(4.0) + 1)) < 1e-15
    turns = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(turns(8.0)), 0), min(math.ceil(turns(1.0)), 7)
    for i in range(4):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0), 1)
        assert abs(float(scaled[i]) - float(f[i]) * (ramp / 4 + 1 - ramp)) < 1e-15
    # the rotation keeps the pair's length up to the magnitude and leaves the other dimensions alone
    x = torch.randn(3, 2, 12, dtype=torch.float64)
    y = P.rotate_pairs(x, torch.tensor([0, 5, 900]), dict(rot, scaling=sc))
    assert torch.equal(y[..., 8:], x[..., 8:])
    pair = lambda z: (z[..., 0:8:2] ** 2 + z[..., 1:8:2] ** 2).sqrt()
    assert torch.allclose(pair(y), pair(x) * m4)
    assert torch.allclose(y[0], torch.cat([x[0, :, :8] * m4, x[0, :, 8:]], -1))          # position 0 only scales


def test_routing_uses_the_correction_for_the_choice_only():
    torch.manual_seed(3)
    h = torch.randn(6, 9, dtype=torch.float64)
    W = {"m.router": torch.randn(4, 9, dtype=torch.float64), "m.correction": torch.tensor([0.0, 10.0, 0.0, -10.0], dtype=torch.float64)}
    idx, w = P.route(h, W, "m", {"top": 2, "scale": 2.5})
    s = torch.sigmoid(h @ W["m.router"].T)
    assert (idx[:, 0] == 1).all() and (idx != 3).all()
    assert torch.allclose(w, torch.gather(s, 1, idx) * 2.5)


def test_whole_model_equals_itself_in_float32_and_float64():
    cfg = config("U")
    w = random_weights(cfg, 3)
    toks = list(range(5, 45))
    a, _ = P.forward(toks, cfg, w)
    b, _ = P.forward(toks, cfg, w, dtype=torch.float32)
    assert float((a - b.double()).abs().max()) < 2e-3
