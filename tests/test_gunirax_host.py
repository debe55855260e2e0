"""CPU tests of the Gunirax design: configuration parsing and the oracle's own consistency (portions against whole
prompts, the chunk's edges, the stretched frequencies, the router's grouped choice, the restarting passes)."""
import copy
import math

import pytest
import torch

from gunirax_util import MIXED, config, dense, hg, left, moe, only_left, par, right, rot, tokens
from oracle import gunirax_oracle as go
from smoltts_b200.lm_config import GuniraxConfig, RotarySpec


def test_config_round_trip_shapes_and_runs():
    cfg = GuniraxConfig.from_dict(MIXED)
    assert GuniraxConfig.from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    assert cfg.layer_runs() == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert cfg.run_restarts() == [0, 0, 0, 1, 0, 1, 0, 0, 0]
    assert [(i, bool(a)) for i, a in zip(cfg.layer_runs(), cfg.run_restarts())] == go.layer_runs(MIXED)
    w = go.random_weights(MIXED, 0)
    assert {k: tuple(v.shape) for k, v in w.items()} == cfg.tensor_shapes()
    assert cfg.layers[2].left.chunk == 5 and cfg.layers[2].left.rot.factor == 0.0 and cfg.layers[1].shared_ff == 16
    assert cfg.layers[3].router.groups == 1 and cfg.layers[4].mlp_kind is None and cfg.layers[0].mixer.vdim == 12
    plain = GuniraxConfig.from_dict(config([par(), hg()]))
    assert plain.layer_runs() == [0, 1] and plain.run_restarts() == [0, 0]
    whole = GuniraxConfig.from_dict(config([par(), hg()], loop=(0, 2, 2)))
    assert whole.layer_runs() == [0, 1, 0, 1] and whole.run_restarts() == [0, 0, 1, 0]
    with pytest.raises(ValueError):
        GuniraxConfig.from_dict(config([{"type": "serial", "mixer": {}, "mlp": None}]))
    with pytest.raises(ValueError):
        GuniraxConfig.from_dict(config([par(left(heads=3, kv_heads=2))]))
    with pytest.raises(ValueError):
        GuniraxConfig.from_dict(config([par(r=right(heads=2, decay=[0.5]))]))
    with pytest.raises(ValueError):
        GuniraxConfig.from_dict(config([par()], loop=(0, 3, 2)))
    with pytest.raises(ValueError):
        GuniraxConfig.from_dict(config([par(mlp=moe(experts=8, top=5, groups=(4, 2)))]))
    assert cfg.weight_elements(active_only=True) < cfg.weight_elements()


def test_registry_names_the_design(tmp_path):
    from smoltts_b200 import registry

    GuniraxConfig.from_dict(MIXED).save(str(tmp_path / "config.json"))
    assert registry.design_of(str(tmp_path)) == "Gunirax"
    assert registry.registered()["Gunirax"] == ("smoltts_b200.lm", "GuniraxLM")


def test_stretched_frequencies_band_by_band():
    """Short wavelengths keep their frequency, long ones are divided by the factor, the band between is blended; the
    configuration's table and the oracle's agree."""
    r = rot(16, 10000.0, (8.0, 1.0, 4.0, 64))
    f = go.rotary_frequencies(r)
    plain = [10000.0 ** (-2.0 * i / 16) for i in range(8)]
    kinds = set()
    for i, p in enumerate(plain):
        wl = 2 * math.pi / p
        if wl < 64 / 4.0:
            assert float(f[i]) == pytest.approx(p); kinds.add("kept")
        elif wl > 64 / 1.0:
            assert float(f[i]) == pytest.approx(p / 8.0); kinds.add("divided")
        else:
            assert p / 8.0 < float(f[i]) < p; kinds.add("blended")
    assert kinds == {"kept", "divided", "blended"}
    assert RotarySpec.from_dict(r).frequencies() == pytest.approx([float(v) for v in f], rel=1e-12)
    assert [float(v) for v in go.rotary_frequencies(rot(16, 10000.0, None))] == pytest.approx(plain)


def test_oracle_portions_equal_the_whole_prompt():
    orc = go.Oracle(MIXED, go.random_weights(MIXED, 3))
    toks = tokens(40, MIXED["vocab"])
    whole = orc.forward(toks)
    parts = [orc.step(toks[lo:hi]) for lo, hi in ((0, 7), (7, 9), (9, 10), (10, 33), (33, 40))]
    assert float((torch.cat(parts) - whole).abs().max()) < 1e-9


def test_chunk_edges_and_plain_sums():
    """Sigmoid attention alone, one layer: position i depends on the first token of its chunk and not on the token before
    it; a key's weight is a plain sigmoid, so with one head, an identity mixing matrix and an open gate the output row is
    sum_j sigmoid(s_ij + bias) k_j projected."""
    cfg = config([par(left(chunk=6))])
    w = go.random_weights(cfg, 1)
    only_left(w)
    orc = go.Oracle(cfg, w)
    toks = tokens(30, cfg["vocab"])
    base = orc.forward(toks)
    for changed, moves in ((18, True), (17, False)):          # position 20 lies in the chunk 18..23
        other = list(toks)
        other[changed] = (other[changed] + 1) % cfg["vocab"]
        assert (float((orc.forward(other)[20] - base[20]).abs().max()) > 1e-6) == moves
    m = left(heads=1, kv_heads=1, dim=4, chunk=3, scale=0.5, r=rot(0, 10.0, None))
    g = torch.Generator().manual_seed(0)
    w0 = {"q": torch.randn(4, 6, generator=g, dtype=go.F), "k": torch.randn(4, 6, generator=g, dtype=go.F), "q.b": torch.randn(4, generator=g, dtype=go.F),
          "k.b": torch.randn(4, generator=g, dtype=go.F), "talk": torch.ones(1, 1, dtype=go.F), "pb": torch.tensor([-0.3], dtype=go.F),
          "g": torch.zeros(1, 6, dtype=go.F), "o": torch.eye(4, dtype=go.F)}
    h = torch.randn(5, 6, generator=g, dtype=go.F)
    out = go.sigmoid_attention(h, w0, "", m, 1e-6)
    q = h @ w0["q"].T + w0["q.b"]
    k = h @ w0["k"].T + w0["k.b"]
    qn, kn = go.rms(q, 1e-6), go.rms(k, 1e-6)
    for i in range(5):
        want = torch.zeros(4, dtype=go.F)
        for j in range(i // 3 * 3, i + 1):
            want += torch.sigmoid((qn[i] @ kn[j]) * 0.5 - 0.3) * k[j]
        assert float((out[i] - 0.5 * want).abs().max()) < 1e-12          # the closed gate's sigmoid(0) = 1/2


def test_rotation_acts_on_the_leading_pairs_only():
    x = torch.arange(1.0, 13.0, dtype=go.F).view(1, 1, 12)
    f = torch.tensor([0.5, 0.25], dtype=go.F)
    y = go.rotate(x, torch.tensor([3]), f)
    assert torch.equal(y[..., 4:], x[..., 4:])
    a = 3 * 0.25
    assert float(y[0, 0, 2]) == pytest.approx(3 * math.cos(a) - 4 * math.sin(a)) and float(y[0, 0, 3]) == pytest.approx(4 * math.cos(a) + 3 * math.sin(a))


def test_router_groups_rank_by_their_two_best():
    """A group with two good choice scores beats a group with the single best one; negative choice scores of a kept group
    still beat every excluded expert; the weights are the plain scores over their sum, times the scale."""

    def routed(scores, correction, r):
        s = torch.tensor([scores], dtype=go.F)
        z = torch.log(s / (1 - s))                              # a router of one feature whose logits are z
        return go.route(torch.ones(1, 1, dtype=go.F), z.T.contiguous(), torch.tensor(correction, dtype=go.F), r)

    r = {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}, "scale": 2.0}
    ids, wts = routed([0.9, 0.05, 0.6, 0.55, 0.7, 0.5], [0.0] * 6, r)       # sums 0.95, 1.15, 1.2; the best single score sits in group 0
    assert ids[0] == [4, 2, 3]
    assert [float(v) for v in wts[0]] == pytest.approx([2.0 * v / 1.85 for v in (0.7, 0.6, 0.55)])
    r = {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}, "scale": 1.0}
    ids, wts = routed([0.3, 0.2, 0.1, 0.1], [-0.5, -0.5, -0.9, -0.9], r)
    assert ids[0] == [0, 1] and [float(v) for v in wts[0]] == pytest.approx([0.6, 0.4])
    ids, _ = routed([0.3, 0.2, 0.4, 0.1], [0.0, 0.0, -0.35, 0.3], {"experts": 4, "top": 2, "scale": 1.0})      # the correction decides, one group
    assert ids[0] == [3, 0]


def test_restarting_passes_add_the_embedding_output():
    """Two passes over one layer equal two separate layers with the same weights when the embedding output is added by
    hand in between; without the addition the result differs."""
    looped = config([par(mlp=dense())], loop=(0, 1, 2))
    w = go.random_weights(looped, 5)
    toks = tokens(12, looped["vocab"], 1)
    col = []
    go.Oracle(looped, w).forward(toks, col)
    assert len(col) == 2
    twice = config([par(mlp=dense()), par(mlp=dense())])
    w2 = dict(w)
    w2.update({k.replace("l0.", "l1.", 1): v for k, v in w.items() if k.startswith("l0.")})
    col2 = []
    go.Oracle(twice, w2).forward(toks, col2)
    assert float((col2[0] - col[0]).abs().max()) < 1e-12 and float((col2[1] - col[1]).abs().max()) > 1e-3
    orc = go.Oracle(twice, w2)
    x0 = orc.w["embed"][torch.tensor(toks)] * looped["embedding"]["scale"]
    x = col[0] + x0
    x = x + go.parallel_mixer(go.dyt(x, orc.w, "l0.norm1"), orc.w, "l0.mix.", looped["layers"][0]["mixer"], 1e-5)
    x = x + go.feed_forward(go.dyt(x, orc.w, "l0.norm2"), orc.w, "l0.mlp.", looped["layers"][0]["mlp"])
    assert float((x - col[1]).abs().max()) < 1e-12


def test_linear_attentions_one_step_at_a_time():
    """Lightning attention and HGRN2 against their unrolled sums: o_t = sum_s decay^(t-s) (q_t.k_s) v_s, and for HGRN2 the
    product of the forget gates between s and t in place of the power."""
    g = torch.Generator().manual_seed(2)
    n, D = 6, 5
    h = torch.randn(n, D, generator=g, dtype=go.F)
    m = right(heads=1, dim=3, vdim=2, decay=[0.8])
    w = {nm: torch.randn(sz, D, generator=g, dtype=go.F) for nm, sz in (("q", 3), ("k", 3), ("v", 2), ("g", 2))}
    w.update({"o": torch.eye(2, dtype=go.F), "norm": torch.ones(2, dtype=go.F)})
    out = go.lightning_attention(h, w, "", m, 1e-6)
    q, k, v = go.silu(h @ w["q"].T), go.silu(h @ w["k"].T), go.silu(h @ w["v"].T)
    for t in range(n):
        o = sum(0.8 ** (t - s) * float(q[t] @ k[s]) * v[s] for s in range(t + 1))
        assert float((out[t] - go.rms(o, 1e-6) * torch.sigmoid(h[t] @ w["g"].T)).abs().max()) < 1e-12
    m = {"heads": 1, "dim": 3, "vdim": 2}
    w = {"q": torch.randn(3, D, generator=g, dtype=go.F), "f": torch.randn(3, D, generator=g, dtype=go.F), "f.b": torch.randn(3, generator=g, dtype=go.F),
         "lower": torch.tensor([0.0, 0.5, 0.9], dtype=go.F), "v": torch.randn(2, D, generator=g, dtype=go.F), "o": torch.eye(2, dtype=go.F),
         "norm": torch.tensor([1.0, 2.0], dtype=go.F)}
    out = go.hgrn2(h, w, "", m, 1e-6)
    f = w["lower"] + (1 - w["lower"]) * torch.sigmoid(h @ w["f"].T + w["f.b"])
    assert bool((f >= w["lower"]).all()) and bool((f <= 1).all())
    q, v = go.silu(h @ w["q"].T), h @ w["v"].T
    for t in range(n):
        o = torch.zeros(2, dtype=go.F)
        for s in range(t + 1):
            keep = torch.ones(3, dtype=go.F)
            for u in range(s + 1, t + 1):
                keep = keep * f[u]
            o += float(q[t] @ (keep * (1 - f[s]))) * v[s]
        assert float((out[t] - go.rms(o, 1e-6) * w["norm"]).abs().max()) < 1e-12


def test_one_decay_number_serves_every_head():
    cfg = config([par(r=right(heads=3, decay=[0.75, 0.75, 0.75]))])
    one = copy.deepcopy(cfg)
    one["layers"][0]["mixer"]["right"]["decay"] = 0.75
    assert GuniraxConfig.from_dict(one).layers[0].right.decay == GuniraxConfig.from_dict(cfg).layers[0].right.decay == [0.75] * 3
    with pytest.raises(ValueError):
        GuniraxConfig.from_dict(config([par(r=right(heads=3, decay=[0.5, 0.5]))]))
