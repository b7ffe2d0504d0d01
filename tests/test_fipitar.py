"""CPU: the Fipitar decoder's configuration, the model as data, its loader, and the plain implementation's pieces on
inputs whose answers are known."""
import json
import math

import numpy as np
import pytest
import torch

from mashbox_b200.config.fipitar import FipitarConfig
from mashbox_b200.config.registry import read_config
from mashbox_b200.errors import ConfigError, WeightError
from mashbox_b200.models.model import Model
from tests import fipitar_helpers as S
from tests.plain import fipitar as plain

F64 = torch.float64


@pytest.mark.parametrize("name", list(S.CONFIGS))
def test_configuration_round_trip(name):
    cfg = S.CONFIGS[name][0]
    entry, back = read_config(json.loads(json.dumps(cfg.to_hf())))
    assert entry.name == "Fipitar" and back == cfg


def test_configuration_refusals():
    good = S.FIP_P.to_hf()

    def broken(change):
        c = json.loads(json.dumps(good))
        change(c)
        return c
    for change, word in ((lambda c: c["layers"][0].update(type="other"), "type"),
                         (lambda c: c["layers"][0]["mixer"].pop("tau"), "tau"),
                         (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
                         (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "rot.dims"),
                         (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
                         (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
                         (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
                         (lambda c: c["layers"][3]["mixer"]["right"].update(groups=3), "groups"),
                         (lambda c: c["layers"][3]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
                         (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
                         (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="other"), "kind"),
                         (lambda c: c["layers"][0]["mlp"].pop("limit"), "limit"),
                         (lambda c: c.pop("width"), "width"),
                         (lambda c: c.pop("norm"), "eps")):
        with pytest.raises(ConfigError, match=word):
            FipitarConfig.from_hf(broken(change))


def test_absent_keys_mean_absent_parts():
    c = S.FIP_P.to_hf()
    assert c["layers"][2]["mlp"] is None and "rot" not in c["layers"][3]["mixer"]["left"]
    assert "softcap" not in c["layers"][3]["mixer"]["left"]
    cfg = FipitarConfig.from_hf(c)
    names = read_config(c)[0].stored_tensors(cfg)
    assert "l2.norm2" not in names and "l2.mlp.gate" not in names and "l2.norm1.b" in names
    assert names["l2.mix.uq"][0] == (3 * (8 + 8), 20) and names["l2.mix.dkv"][0] == (24 + 8, 64)
    assert names["l1.mix.right.in"][0] == (2 * 24 + 2 * 10 + 2, 64) and names["l1.mix.right.conv"][0] == (24 + 20, 4)
    c["layers"][1]["mixer"]["left"].pop("kv_heads")         # as many kv heads as query heads
    c["layers"][1]["mixer"].pop("left_scale")               # a weight of one
    for k in ("groups", "norm_groups", "conv"):             # one group, one norm group, one tap
        c["layers"][1]["mixer"]["right"].pop(k)
    c["layers"][2]["mixer"]["rot"].pop("scaling")           # a plain rotation
    m = FipitarConfig.from_hf(c)
    assert m.layers[1].mixer.left.kv_heads == 4 and m.layers[1].mixer.left_scale == 1.0
    assert (m.layers[1].mixer.right.groups, m.layers[1].mixer.right.norm_groups, m.layers[1].mixer.right.conv) == (1, 1, 1)
    assert m.layers[2].mixer.rot.scaling is None
    q = S.FIP_Q.to_hf()
    assert "rot_dim" not in q["layers"][3]["mixer"] and "rot" not in q["layers"][3]["mixer"]      # the sink alone


def test_model_as_data():
    cfg = S.FIP_P
    entry, _ = read_config(cfg.to_hf())
    model = Model(entry.model_spec(cfg), cfg)
    assert [(r.layer, r.cache, r.write, r.state_id) for r in model.schedule] == [(0, None, False, 0), (1, 1, True, 1),
                                                                                (2, 2, True, 2), (3, 3, True, 3)]
    needs, states = model.cache_needs()
    assert sorted(needs) == [1, 2, 3] and all(n.kind == "full" for n in needs.values())
    # keys and values of their own widths; a latent and its rotated strip in one row
    assert needs[1].tensors == ((2, 16), (2, 24)) and needs[2].tensors == ((1, 24 + 8),) and needs[3].tensors == ((2, 24), (2, 8))
    # gla: a (dim, vdim) matrix per head; beside attention: the convolution's last inputs, then (state, vdim) per head
    assert states[0].shape == (3 * 16 * 24,) and states[1].shape == (3 * (24 + 20) + 2 * 10 * 12,)
    assert states[3].shape == (1 * (24 + 32) + 4 * 8 * 6,) and 2 not in states
    assert model.graph_safe and model.portion_alignment() == 1
    wanted = {w.name for w in model.wants()}
    stored = set(entry.stored_tensors(cfg))
    canon = entry.canonical_names(cfg)
    assert {canon(n)[0] for n in stored} == wanted
    with pytest.raises(KeyError):
        canon("l0.mix.left.q")
    # recurrent layers alone: no cache group at all
    s = S.FIP_S
    needs, states = Model(entry.model_spec(s), s).cache_needs()
    assert not needs and sorted(states) == [0, 1]


def test_loader_checks_shapes_and_reads_the_inner_rank(tmp_path):
    from mashbox_b200.engine.loading import build_model
    from mashbox_b200.weights.safetensors_io import SafetensorsSource
    folder = S.make_folder(tmp_path, "P")
    c = json.load(open(folder + "/config.json"))
    src = SafetensorsSource(folder)
    del c["layers"][0]["mixer"]["a_rank"]                   # config.json does not give it: the tensors do
    model = build_model(c, src, "float32", "cpu")
    assert model.layers[0].mixer.wa1.shape == (4, 64) and model.layers[0].mixer.wa2.shape == (3 * 16, 4)
    pair = model.layers[1].mixer
    assert pair.left.w_in.shape == (4 * 16 + 2 * 16 + 2 * 24 + 4 + 4, 64)           # the gates' rows and zero rows behind them
    assert float(pair.left.w_in[-4:].abs().max()) == 0.0 and float(pair.left.sinks.abs().max()) == 0.0
    assert pair.right.w_xbc.shape == (24 + 20, 64) and pair.right.wconv.shape == (4, 44) and pair.right.w_dt.shape == (2, 64)
    assert pair.scales == (0.7, 1.3) and not any("out" in w.name for w in pair.wants())
    lat = model.layers[2].mixer
    assert lat.w_in.shape == (20 + 24 + 8, 64) and lat.sinks.shape == (3,) and abs(lat.position.gain - (0.1 * math.log(4) + 1)) < 1e-12
    c["layers"][0]["mixer"]["heads"] = 4
    with pytest.raises(WeightError, match="wrong shape"):
        build_model(c, src, "float32", "cpu")
    src.close()


def test_bent_frequencies_match_the_plain_ones():
    from mashbox_b200.parts.position import RotaryEncoding
    for dims, base, sc in ((8, 50.0, (4.0, 64.0, 4.0, 0.5)), (16, 1e4, (2.0, 4096.0, 32.0, 1.0)), (32, 1e5, (8.0, 128.0, 16.0, 2.0)),
                           (6, 70.0, (3.0, 32.0, 2.0, 0.25)), (64, 5e5, (40.0, 4096.0, 32.0, 1.0))):
        rot = dict(dims=dims, base=base, scaling=dict(zip(("factor", "original", "fast", "slow"), sc)))
        want, gain = plain.frequencies(rot)
        part = RotaryEncoding(dims, dims, base, scaling=("yarn",) + sc + (0.1,))
        np.testing.assert_allclose(part.frequencies(), want.numpy(), rtol=2e-7)
        assert abs(part.gain - gain) < 1e-12
        assert not np.allclose(want.numpy(), plain.frequencies(dict(dims=dims, base=base))[0].numpy())
    assert RotaryEncoding(8, 8, 100.0).gain == 1.0


# ------------------------------------------------------------------------------------------------ the plain pieces
def test_plain_layer_norm():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 12, generator=g, dtype=F64) * 3 + 7
    y = plain.layer_norm(x, torch.ones(12, dtype=F64), torch.zeros(12, dtype=F64), 0.0)
    assert float(y.mean(-1).abs().max()) < 1e-12 and float(((y * y).mean(-1) - 1).abs().max()) < 1e-12
    # a constant row has no deviations: what is left is the bias
    z = plain.layer_norm(torch.full((1, 4), 3.0, dtype=F64), torch.ones(4, dtype=F64), torch.tensor([1., 2., 3., 4.], dtype=F64), 1e-6)
    assert torch.equal(z, torch.tensor([[1., 2., 3., 4.]], dtype=F64))


def test_plain_rotations_by_a_quarter_turn():
    rot = dict(dims=2, base=1.0)                                                    # one pair, one radian a position
    x = torch.tensor([[[1.0, 0.0, 5.0]]], dtype=F64).repeat(2, 1, 1)
    pos = torch.tensor([0.0, math.pi / 2], dtype=F64)
    for layout in ("halves", "adjacent"):
        y = plain.rotate(x, pos, rot, layout)
        assert torch.allclose(y[0, 0], torch.tensor([1.0, 0.0, 5.0], dtype=F64))
        assert torch.allclose(y[1, 0], torch.tensor([0.0, 1.0, 5.0], dtype=F64), atol=1e-12)
    # four dims: halves pairs (0, 2) and (1, 3), adjacent pairs (0, 1) and (2, 3)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=F64)
    pos, rot = torch.tensor([1.0], dtype=F64), dict(dims=4, base=1.0)
    c, s = math.cos(1.0), math.sin(1.0)
    assert torch.allclose(plain.rotate(x, pos, rot, "halves")[0, 0], torch.tensor([c - 3 * s, 2 * c - 4 * s, 3 * c + s, 4 * c + 2 * s], dtype=F64))
    assert torch.allclose(plain.rotate(x, pos, rot, "adjacent")[0, 0], torch.tensor([c - 2 * s, 2 * c + s, 3 * c - 4 * s, 4 * c + 3 * s], dtype=F64))


def test_plain_sink_counts_once_and_has_no_value():
    s = torch.tensor([[[0.0, -math.inf], [0.0, 0.0]]], dtype=F64)                   # one head, two queries
    w = plain.softmax_with_sink(s, torch.zeros(1, 2, dtype=F64))
    assert torch.allclose(w[0, 0], torch.tensor([0.5, 0.0], dtype=F64)) and torch.allclose(w[0, 1], torch.tensor([1 / 3, 1 / 3], dtype=F64))
    w = plain.softmax_with_sink(s, torch.full((1, 2), -1e9, dtype=F64))              # a sink far below: the plain softmax
    assert torch.allclose(w[0, 1], torch.tensor([0.5, 0.5], dtype=F64))
    w = plain.softmax_with_sink(s, torch.full((1, 2), math.log(2.0), dtype=F64))
    assert torch.allclose(w[0, 0], torch.tensor([1 / 3, 0.0], dtype=F64))


def _gla_case(logits, tau):
    """One head with two key and two value channels over inputs h = [q0 q1 | k0 k1 | v0 v1 | 1]: what a token asks,
    writes under and writes is spelled out in its row; the gate is the same for both value channels, so the RATIO of a
    token's two outputs is the ratio of the recurrence's two outputs (the head norm scales both alike)."""
    pick = lambda *idx: torch.stack([torch.nn.functional.one_hot(torch.tensor(i), 7).to(F64) for i in idx])
    W = {"q": pick(0, 1), "k": pick(2, 3), "v": pick(4, 5), "g": 50.0 * pick(6, 6), "o": torch.eye(7, 2, dtype=F64),
         "norm": torch.ones(2, dtype=F64), "a1": torch.zeros(1, 7, dtype=F64), "a2": torch.zeros(2, 1, dtype=F64),
         "a2.b": torch.tensor(logits, dtype=F64)}
    return W, dict(heads=1, dim=2, vdim=2, tau=tau)


def test_plain_gla_decays_by_the_root_of_a_sigmoid():
    W, m = _gla_case([1.0, 1.0], 2.0)
    h = torch.tensor([[0, 0, 1, 0, 1, 0, 1],            # writes (1, 0) under key channel 0
                      [1, 0, 1, 0, 0, 1, 1]], dtype=F64)  # writes (0, 1) under the same channel and asks for it
    out = plain.gla(W, "", m, h, 1e-30)
    a = math.sqrt(1 / (1 + math.exp(-1.0)))             # sigmoid(1)^(1/2)
    assert abs(float(out[1, 0] / out[1, 1]) - a) < 1e-12 and float(out[0].abs().max()) == 0.0


def test_plain_gla_decays_every_key_channel_by_itself():
    W, m = _gla_case([-1.0, 2.0], 1.0)
    h = torch.tensor([[0, 0, 1, 0, 1, 0, 1],            # (1, 0) under key channel 0
                      [0, 0, 0, 1, 0, 1, 1],            # (0, 1) under key channel 1
                      [1, 1, 0, 0, 0, 0, 1]], dtype=F64)  # asks for both, writes nothing
    out = plain.gla(W, "", m, h, 1e-30)
    a0, a1 = 1 / (1 + math.exp(1.0)), 1 / (1 + math.exp(-2.0))
    assert abs(float(out[2, 0] / out[2, 1]) - a0 * a0 / a1) < 1e-12


def test_plain_convolution_is_causal_and_ends_on_the_current_token():
    u = torch.zeros(6, 2, dtype=F64)
    u[2, 0] = 1.0
    w = torch.tensor([[1.0, 2.0, 3.0], [0.0, 0.0, 1.0]], dtype=F64)                # the last column meets the current token
    y = plain.causal_conv(u, w, torch.tensor([0.0, 0.5], dtype=F64))
    assert y[:, 0].tolist() == [0.0, 0.0, 3.0, 2.0, 1.0, 0.0] and y[:, 1].tolist() == [0.5] * 6


def test_plain_ssd_state_is_a_geometric_series():
    # one head, state 1, vdim 1, one tap: x = B = C = silu(h), dt = softplus(h_dt + bias), decay exp(-dt)
    m = dict(heads=1, vdim=1, state=1, groups=1, norm_groups=1, conv=1)
    D = 5
    W = {"in": torch.eye(5, D, dtype=F64), "conv": torch.ones(3, 1, dtype=F64), "conv.b": torch.zeros(3, dtype=F64),
         "dt_bias": torch.zeros(1, dtype=F64), "A_log": torch.zeros(1, dtype=F64), "D": torch.zeros(1, dtype=F64),
         "norm": torch.ones(1, dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    big = 40.0                                                                      # silu(40) = 40 to rounding
    dt_raw = math.log(math.e - 1.0)                                                 # softplus -> 1
    h = torch.tensor([[big, big, big, big, dt_raw]] * 3, dtype=F64)                # z, x, B, C, dt
    out = plain.ssd(W, "", m, h, 0.0)
    assert torch.allclose(out, torch.ones(3, 1, dtype=F64))                         # y > 0 always: the norm of one channel leaves its sign
    W["D"] = torch.full((1,), -1e9, dtype=F64)                                      # the skip outweighs the state: the sign turns
    assert torch.allclose(plain.ssd(W, "", m, h, 0.0), -torch.ones(3, 1, dtype=F64))


def test_plain_ssd_norms_its_groups_apart_after_the_gate():
    m = dict(heads=2, vdim=1, state=1, groups=1, norm_groups=2, conv=1)
    D = 2 + 2 + 1 + 1 + 2
    W = {"in": torch.eye(D, D, dtype=F64), "conv": torch.ones(4, 1, dtype=F64), "conv.b": torch.zeros(4, dtype=F64),
         "dt_bias": torch.zeros(2, dtype=F64), "A_log": torch.zeros(2, dtype=F64), "D": torch.zeros(2, dtype=F64),
         "norm": torch.tensor([2.0, 3.0], dtype=F64), "o": torch.eye(2, dtype=F64)}
    h = torch.tensor([[40.0, 40.0, 1.0, 100.0, 1.0, 1.0, 0.0, 0.0]], dtype=F64)
    # two heads of very different size, each a norm group of its own: both come out as their weight
    assert torch.allclose(plain.ssd(W, "", m, h, 0.0), torch.tensor([[2.0, 3.0]], dtype=F64))
    m["norm_groups"] = 1                                                            # one group: the large head takes it all
    out = plain.ssd(W, "", m, h, 0.0)
    assert out[0, 1] > 4.0 and out[0, 0] < 0.1


def test_plain_feed_forward_clamps_the_gate_from_above_only():
    W = {"gate": torch.eye(2, dtype=F64), "up": torch.eye(2, dtype=F64), "down": torch.eye(2, dtype=F64)}
    f = dict(limit=1.5)
    h = torch.tensor([[10.0, 10.0], [-10.0, -10.0], [1.0, -1.0]], dtype=F64)
    out = plain.feed_forward(W, "", f, h)
    sg = lambda g: g / (1 + math.exp(-1.702 * g))
    assert torch.allclose(out[0], torch.tensor([sg(1.5) * 2.5] * 2, dtype=F64))
    assert torch.allclose(out[1], torch.tensor([sg(-10.0) * (-1.5 + 1)] * 2, dtype=F64))       # the gate keeps -10, up stops at -1.5
    assert torch.allclose(out[2], torch.tensor([sg(1.0) * 2.0, 0.0], dtype=F64))               # up = -1: (u + 1) = 0


def test_plain_capped_scores_bound_the_loudest_key():
    # one head, two tokens; the second query meets a key a thousand times louder than the cap: its weight is
    # e^cap / (1 + e^cap + e^s_own), never one
    m = dict(heads=1, kv_heads=1, dim=2, vdim=1, scale=1.0, softcap=2.0)
    W = {"q": torch.tensor([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]], dtype=F64), "k": torch.tensor([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]], dtype=F64),
         "v": torch.tensor([[0.0, 0.0, 1.0]], dtype=F64), "q.norm": torch.full((2,), 1e3, dtype=F64),
         "k.norm": torch.ones(2, dtype=F64), "g": torch.tensor([[0.0, 0.0, 1e3]], dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    h = torch.tensor([[1.0, 0.0, 1.0], [1.0, 0.0, 1.0]], dtype=F64)                 # both tokens: the same direction, value 1
    out = plain.capped_attention(W, "", m, h, 0.0)
    e = math.exp(2.0)
    assert abs(float(out[0, 0]) - e / (1 + e)) < 1e-9 and abs(float(out[1, 0]) - 2 * e / (1 + 2 * e)) < 1e-9
    m.pop("softcap")                                                                # no cap: the sink of one vanishes beside e^2000
    assert abs(float(plain.capped_attention(W, "", m, h, 0.0)[0, 0]) - 1.0) < 1e-12


def test_plain_latent_scores_add_an_unrotated_and_a_rotated_part():
    # one head; the latent is the input's first value, the strip its second; two tokens at positions 0 and 1
    m = dict(heads=1, dim=1, rot_dim=2, vdim=1, q_rank=3, kv_rank=1, scale=1.0, rot=dict(dims=2, base=1.0))
    W = {"dq": torch.eye(3, dtype=F64), "dq.norm": torch.ones(3, dtype=F64), "uq": torch.eye(3, dtype=F64),
         "dkv": torch.eye(3, dtype=F64), "dkv.norm": torch.ones(1, dtype=F64), "uk": torch.ones(1, 1, dtype=F64),
         "uv": torch.ones(1, 1, dtype=F64), "sink": torch.tensor([-1e9], dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    h = torch.tensor([[2.0, 1.0, 0.0], [2.0, 1.0, 0.0]], dtype=F64)
    out = plain.latent_attention(W, "", m, h, 0.0)
    assert torch.allclose(out, torch.ones(2, 1, dtype=F64))                         # the value is the normed latent, 1, whatever the weights
    W["sink"] = torch.tensor([0.0], dtype=F64)
    out = plain.latent_attention(W, "", m, h, 0.0)
    # token 0: cq = rms(2, 1, 0) = (2, 1, 0) / sqrt(5/3); score = u c + r . kr with c = 1 (normed), kr = (1, 0) unrotated at position 0
    cq = torch.tensor([2.0, 1.0, 0.0], dtype=F64) / math.sqrt(5.0 / 3.0)
    s00 = float(cq[0] * 1.0 + cq[1] * 1.0)
    assert abs(float(out[0, 0]) - math.exp(s00) / (1 + math.exp(s00))) < 1e-12
    # token 1 sees key 0 through a turn of one radian between them: r . kr = |r| |kr| cos(1) for parallel strips
    s10 = float(cq[0] * 1.0 + cq[1] * math.cos(1.0))
    want = (math.exp(s10) + math.exp(s00)) / (1 + math.exp(s10) + math.exp(s00))
    assert abs(float(out[1, 0]) - want) < 1e-12


def test_plain_forward_norms_outputs_not_inputs(tmp_path):
    folder = S.make_folder(tmp_path, "S")
    cfg, W = S._model(folder)
    p = S.prompts_for("S", (9,))[0]
    layers = []
    plain.forward(cfg, W, p, layers)
    x0 = W["embed"].to(F64)[torch.as_tensor(p)]
    # after the first sublayer the stream moved by a layer-normed vector: its deviations from the bias have unit scale
    y = plain.gla(W, "l0.mix.", cfg["layers"][0]["mixer"], x0, float(cfg["norm"]["eps"]))
    step = plain.layer_norm(y, W["l0.norm1"].to(F64), W["l0.norm1.b"].to(F64), float(cfg["norm"]["eps"]))
    x1 = x0 + step
    x1 = x1 + plain.layer_norm(plain.feed_forward(W, "l0.mlp.", cfg["layers"][0]["mlp"], x1), W["l0.norm2"].to(F64),
                               W["l0.norm2.b"].to(F64), float(cfg["norm"]["eps"]))
    assert torch.allclose(layers[0], x1, atol=1e-12) and len(layers) == 2
