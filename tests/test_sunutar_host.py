"""CPU tests of the Sunutar design: configuration parsing and the oracle's own consistency (portions against whole
prompts, the window's edge, the extra term of the softmax, the router's weights on the experts' inputs)."""
import copy

import pytest
import torch

from oracle import sunutar_oracle as so
from smoltts_b200.lm_config import SunutarConfig
from sunutar_util import MIXED, config, dense, layer, left, moe, right, tokens


def test_config_round_trip_and_shapes():
    cfg = SunutarConfig.from_dict(MIXED)
    assert SunutarConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.layer_runs() == [0, 1, 2, 3]
    w = so.random_weights(MIXED, 0)
    assert {k: tuple(v.shape) for k, v in w.items()} == cfg.tensor_shapes()
    assert cfg.layers[1].left.window == 5 and cfg.layers[1].right.conv == 4 and cfg.layers[1].top == 2
    assert cfg.layers[2].mlp_kind is None and cfg.layers[0].limit == 1.5
    with pytest.raises(ValueError):
        SunutarConfig.from_dict(config([{"type": "serial", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        SunutarConfig.from_dict(config([layer(left(heads=3, kv_heads=2))]))
    with pytest.raises(ValueError):
        SunutarConfig.from_dict(config([layer(mlp=moe(experts=2, top=3))]))
    assert cfg.weight_elements(active_only=True) < cfg.weight_elements()


def test_registry_names_the_design(tmp_path):
    from smoltts_b200 import registry

    SunutarConfig.from_dict(MIXED).save(str(tmp_path / "config.json"))
    assert registry.design_of(str(tmp_path)) == "Sunutar"
    assert registry.registered()["Sunutar"] == ("smoltts_b200.lm", "SunutarLM")


def test_oracle_portions_equal_the_whole_prompt():
    orc = so.Oracle(MIXED, so.random_weights(MIXED, 3))
    toks = tokens(40, MIXED["vocab"])
    whole = orc.forward(toks)
    parts = [orc.step(toks[lo:hi]) for lo, hi in ((0, 7), (7, 9), (9, 10), (10, 33), (33, 40))]
    assert float((torch.cat(parts) - whole).abs().max()) < 1e-9


def test_window_edge_and_extra_softmax_term():
    """Attention alone (the other branch's scale is 0), one layer: position i depends on the token window - 1 places
    back and not on the one before it; with a window of 1 the weight of the only key is e^s / (1 + e^s)."""
    cfg = config([layer(left(window=6), right_scale=0.0)])
    orc = so.Oracle(cfg, so.random_weights(cfg, 1))
    toks = tokens(30, cfg["vocab"])
    base = orc.forward(toks)
    for back, moves in ((5, True), (6, False)):
        other = list(toks)
        other[20 - back] = (other[20 - back] + 1) % cfg["vocab"]
        assert (float((orc.forward(other)[20] - base[20]).abs().max()) > 1e-6) == moves
    m = left(heads=2, kv_heads=2, dim=4, vdim=4, window=1, scale=0.5, softcap=5.0)
    g = torch.Generator().manual_seed(0)
    w = {k: torch.randn(*s, generator=g, dtype=torch.float64) for k, s in
         {"q": (8, 6), "k": (8, 6), "v": (8, 6), "o": (6, 8), "q.b": (8,), "k.b": (8,), "v.b": (8,), "o.b": (6,), "q.norm": (8,), "k.norm": (8,)}.items()}
    h = torch.randn(3, 6, generator=g, dtype=torch.float64)
    got = so.window_attention(h, w, "", m, 1e-6)
    q = so.rms_norm(h @ w["q"].T + w["q.b"], w["q.norm"], 1e-6).view(3, 2, 4)
    k = so.rms_norm(h @ w["k"].T + w["k.b"], w["k.norm"], 1e-6).view(3, 2, 4)
    v = (h @ w["v"].T + w["v.b"]).view(3, 2, 4)
    s = 5.0 * torch.tanh((q * k).sum(-1) * 0.5 / 5.0)
    want = (torch.sigmoid(s)[..., None] * v).reshape(3, 8) @ w["o"].T + w["o.b"]
    assert torch.allclose(got, want, atol=1e-12)


def test_router_scores_weigh_the_inputs():
    mlp = moe(experts=4, top=2, ff=6, limit=0.9)
    g = torch.Generator().manual_seed(1)
    w = {"router": torch.randn(4, 5, generator=g, dtype=torch.float64)}
    for e in range(4):
        w.update({f"e{e}.gate": torch.randn(6, 5, generator=g, dtype=torch.float64), f"e{e}.up": torch.randn(6, 5, generator=g, dtype=torch.float64),
                  f"e{e}.down": torch.randn(5, 6, generator=g, dtype=torch.float64)})
    h = torch.randn(7, 5, generator=g, dtype=torch.float64)
    got = so.feed_forward(h, w, "", mlp)
    s = torch.sigmoid(h @ w["router"].T)
    for t in range(7):
        best = sorted(range(4), key=lambda e: -float(s[t, e]))[:2]
        want = sum(so.clamped_glu((s[t, e] * h[t])[None], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], 0.9)[0] for e in best)
        assert torch.allclose(got[t], want, atol=1e-12)
    # the unit is not linear: weighting the output instead would differ
    e = int(s[0].argmax())
    assert not torch.allclose(so.clamped_glu((s[0, e] * h[0])[None], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], 0.9),
                              s[0, e] * so.clamped_glu(h[0][None], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], 0.9))


def test_clamp_limits_show():
    h = torch.tensor([[3.0, -3.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    out = so.clamped_glu(h, eye, eye, eye, 1.0)
    g = torch.tensor([1.0, -3.0], dtype=torch.float64)
    u = torch.tensor([1.0, -1.0], dtype=torch.float64)
    assert torch.allclose(out[0], g * torch.sigmoid(1.702 * g) * (u + 1.0))
