"""CPU: the Tosevik decoder's configuration, the model as data, its loader, and the plain implementation's pieces on
inputs whose answers are known."""
import json
import math

import numpy as np
import pytest
import torch

from mashbox_b200.config.registry import read_config
from mashbox_b200.config.tosevik import TosevikConfig
from mashbox_b200.errors import ConfigError, WeightError
from mashbox_b200.models.model import Model
from tests import tosevik_helpers as S
from tests.plain import tosevik as plain

F64 = torch.float64


@pytest.mark.parametrize("name", list(S.CONFIGS))
def test_configuration_round_trip(name):
    cfg = S.CONFIGS[name][0]
    entry, back = read_config(json.loads(json.dumps(cfg.to_hf())))
    assert entry.name == "Tosevik" and back == cfg


def test_configuration_refusals():
    good = S.TOS_T.to_hf()

    def broken(change):
        c = json.loads(json.dumps(good))
        change(c)
        return c
    for change, word in ((lambda c: c["layers"][0].update(type="other"), "type"),
                         (lambda c: c["layers"][0]["mixer"].update(decay=[0.5, 0.9]), "decay"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
                         (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
                         (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
                         (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
                         (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "router"),
                         (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=5), "router"),
                         (lambda c: c["layers"][0]["mlp"].update(kind="other"), "kind"),
                         (lambda c: c.pop("width"), "width"),
                         (lambda c: c.pop("norm"), "eps")):
        with pytest.raises(ConfigError, match=word):
            TosevikConfig.from_hf(broken(change))


def test_absent_keys_mean_absent_parts():
    c = S.TOS_T.to_hf()
    assert "rot" not in c["layers"][2]["mixer"] and c["layers"][2]["mlp"] is None
    assert "q_temp" not in c["layers"][3]["mixer"]["left"] and "shared" not in c["layers"][1]["mlp"]
    cfg = TosevikConfig.from_hf(c)
    names = read_config(c)[0].stored_tensors(cfg)
    assert "l2.norm2" not in names and "l2.mlp.router" not in names and "l2.dwa" in names
    assert "l1.mlp.shared.sg" not in names and "l0.mlp.shared.sg" in names and "l1.mix.left.pb" in names
    assert names["l0.dwa"][0] == (2,) and names["l3.dwa"][0] == (5,)
    del c["layers"][0]["mlp"]["router"]["groups"]           # no groups: every expert may be chosen
    del c["layers"][0]["mlp"]["router"]["scale"]
    f = TosevikConfig.from_hf(c).layers[0].mlp
    assert f.groups == 1 and f.keep == 1 and f.scale == 1.0
    c["layers"][1]["mixer"]["left"].pop("kv_heads")         # as many kv heads as query heads
    assert TosevikConfig.from_hf(c).layers[1].mixer.left.kv_heads == 4


def test_model_as_data():
    cfg = S.TOS_T
    entry, _ = read_config(cfg.to_hf())
    model = Model(entry.model_spec(cfg), cfg)
    runs = model.schedule
    assert [(r.layer, r.cache, r.write, r.state_id) for r in runs] == [(0, None, False, 0), (1, 1, True, 1),
                                                                      (2, None, False, 2), (3, 3, True, 3)]
    needs, states = model.cache_needs()
    assert sorted(needs) == [1, 3] and needs[1].kind == "full"
    assert needs[1].tensors == ((2, 16), (2, 24)) and needs[3].tensors == ((2, 24), (2, 8))
    # a retention mixer keeps a (vdim, dim) matrix per head and nothing per position; beside attention, the same
    assert states[0].shape == (3 * 16 * 24,) and states[1].shape == (2 * 24 * 16,)
    assert states[2].shape == (2 * 8 * 40,) and states[3].shape == (4 * 8 * 8,)
    assert model.graph_safe and model.portion_alignment() == 1
    wanted = {w.name for w in model.wants()}
    stored = set(entry.stored_tensors(cfg))
    canon = entry.canonical_names(cfg)
    assert {canon(n)[0] for n in stored} == wanted
    # retention layers alone: no cache group at all
    w = S.TOS_W
    needs, states = Model(entry.model_spec(w), w).cache_needs()
    assert not needs and sorted(states) == [0, 1]


def test_loader_checks_shapes_and_names(tmp_path):
    from mashbox_b200.engine.loading import build_model
    from mashbox_b200.weights.safetensors_io import SafetensorsSource
    folder = S.make_folder(tmp_path, "T")
    c = json.load(open(folder + "/config.json"))
    src = SafetensorsSource(folder)
    model = build_model(c, src, "float32", "cpu")
    block = model.layers[1]
    assert block.coef.shape == (3,) and block.mixer.left.w_in.shape == (4 * 16 + 2 * 16 + 2 * 24, 64)
    assert block.mixer.right.w_in.shape == (2 * 24 * 2 + 2 * 16 * 2, 64)
    assert block.ffn.wr.shape == (6, 64) and model.layers[0].ffn.wr.shape == (12 + 1, 64)     # the gate's row rides along
    c["layers"][0]["mixer"]["heads"] = 4
    c["layers"][0]["mixer"]["decay"] = [0.5, 0.6, 0.7, 0.8]
    with pytest.raises(WeightError, match="wrong shape"):
        build_model(c, src, "float32", "cpu")
    src.close()


# ------------------------------------------------------------------------------------------------ the plain pieces
def test_plain_dynamic_tanh_uses_no_statistics():
    W = {"n": torch.tensor([2.0, -1.0], dtype=F64), "n.b": torch.tensor([0.5, 0.25], dtype=F64),
         "n.alpha": torch.tensor(0.5, dtype=F64)}
    x = torch.tensor([[2.0, 4.0], [2.0, -100.0]], dtype=F64)
    y = plain.dyt(W, "n", x)
    assert torch.allclose(y[:, 0], torch.full((2,), 2.0 * math.tanh(1.0) + 0.5, dtype=F64))   # whatever else the row holds
    assert abs(float(y[1, 1]) - 1.25) < 1e-12                                                # saturated: -w + b


def test_plain_rotation_on_known_cases():
    x = torch.zeros(3, 1, 6, dtype=F64)
    x[:, 0, 0] = 1.0            # dim 0 pairs with dim 2 (R = 4), dims 4 and 5 pass
    x[:, 0, 4] = 7.0
    y = plain.rotate(x, torch.tensor([0, 1, 5]), dict(dims=4, base=100.0))
    for t, p in enumerate((0, 1, 5)):
        assert abs(float(y[t, 0, 0]) - math.cos(p)) < 1e-12 and abs(float(y[t, 0, 2]) - math.sin(p)) < 1e-12
        assert float(y[t, 0, 1]) == 0.0 and float(y[t, 0, 4]) == 7.0
    x = torch.zeros(1, 1, 4, dtype=F64)
    x[0, 0, 1] = 1.0            # dim 1 pairs with dim 3 and turns by p * base^(-2 / 4)
    y = plain.rotate(x, torch.tensor([3]), dict(dims=4, base=100.0))
    assert abs(float(y[0, 0, 1]) - math.cos(0.3)) < 1e-12 and abs(float(y[0, 0, 3]) - math.sin(0.3)) < 1e-12
    assert plain.rotate(x, torch.tensor([3]), None) is x


def test_plain_retention_on_known_cases():
    # one head, dim 2, vdim 1, identity projections: k_t v_t is written, the state halves every step, no denominator
    W = {"m.q": torch.eye(2, dtype=F64), "m.k": torch.eye(2, dtype=F64), "m.v": torch.tensor([[1.0, 1.0]], dtype=F64),
         "m.g": torch.zeros(1, 2, dtype=F64), "m.o": torch.ones(1, 1, dtype=F64)}
    m = dict(heads=1, dim=2, vdim=1, decay=[0.5])
    h = torch.tensor([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0], [1.0, 0.0]], dtype=F64)
    state = [torch.zeros(2, 1, dtype=F64)]
    plain.retention(W, "m.", m, h, 1e-5, state=state)
    k = 2 ** -0.5               # k is scaled by dim^-1/2, v = 1 each step
    assert torch.allclose(state[0][:, 0], torch.tensor([k * (0.125 + 0.25 + 1.0), k * 0.5], dtype=F64))
    # carried across a cut: the second half from the first half's state is the whole
    W["m.g"] = torch.tensor([[0.3, -0.2]], dtype=F64)
    whole = plain.retention(W, "m.", m, h, 1e-5)
    state = [torch.zeros(2, 1, dtype=F64)]
    a = plain.retention(W, "m.", m, h[:1], 1e-5, state=state)
    b = plain.retention(W, "m.", m, h[1:], 1e-5, state=state, first=1)
    assert torch.allclose(torch.cat([a, b]), whole)


def test_plain_sigmoid_attention_is_causal_and_not_normalised():
    g = torch.Generator().manual_seed(3)
    m = dict(heads=2, kv_heads=1, dim=4, vdim=3, scale=0.5, q_temp=dict(coef=0.5, every=4))
    W = {"a." + n: torch.randn(*s, generator=g, dtype=F64) * 0.5 for n, s in
         dict(q=(8, 6), k=(4, 6), v=(3, 6), o=(6, 6)).items()}
    W.update({"a.q.norm": torch.ones(8, dtype=F64), "a.k.norm": torch.ones(4, dtype=F64),
              "a.pb": torch.tensor([0.3, -0.4], dtype=F64)})
    h = torch.randn(9, 6, generator=g, dtype=F64)
    full = plain.sigmoid_attention(W, "a.", m, h, 1e-5)
    h2 = h.clone()
    h2[6:] += 1.0
    assert torch.allclose(plain.sigmoid_attention(W, "a.", m, h2, 1e-5)[:6], full[:6])
    # a single token: weight sigmoid(scale q.k + pb) on its own unit-rms value, no division by the sum of weights
    W["a.o"] = torch.eye(6, dtype=F64)
    one = plain.sigmoid_attention(W, "a.", m, h[:1], 1e-5)[0].view(2, 3)
    q = plain.rms(h[:1] @ W["a.q"].T, 1e-5).view(2, 4)
    k = plain.rms(h[:1] @ W["a.k"].T, 1e-5)[0]
    v = plain.rms(h[:1] @ W["a.v"].T, 1e-5)[0]
    for a in range(2):
        assert torch.allclose(one[a], torch.sigmoid(0.5 * (q[a] @ k) + W["a.pb"][a]) * v)
    # the temperature first moves at position every - 1
    h3 = h[:1].expand(5, 6).clone()
    m0 = dict(m, q_temp=None)
    with_t, without = plain.sigmoid_attention(W, "a.", m, h3, 1e-5), plain.sigmoid_attention(W, "a.", m0, h3, 1e-5)
    assert torch.allclose(with_t[:3], without[:3]) and not torch.allclose(with_t[3], without[3])


def test_plain_choice_on_known_cases():
    s = torch.tensor([[0.30, 0.05, 0.02, 0.03, 0.25, 0.24, 0.06, 0.05]], dtype=F64)
    assert plain.choose(s, 2).tolist() == [[0, 4]]
    # two groups of four, one kept: a group is worth its best expert, so group 0 wins and 4, 5 cannot be chosen
    assert plain.choose(s, 2, count=2, keep=1).tolist() == [[0, 1]]
    assert plain.choose(s, 3, count=4, keep=2).tolist() == [[0, 4, 5]]        # groups {0,1} and {4,5}
    assert plain.choose(torch.full((1, 4), 0.25, dtype=F64), 2).tolist() == [[0, 1]]       # ties: the lower index


def test_plain_routed_weights_are_scaled_scores(tmp_path):
    g = torch.Generator().manual_seed(5)
    D, F, E = 6, 4, 4
    W = {"f.router": torch.randn(E, D, generator=g, dtype=F64)}
    for e in range(E):
        W.update({f"f.e{e}.gate": torch.randn(F, D, generator=g, dtype=F64), f"f.e{e}.up": torch.randn(F, D, generator=g, dtype=F64),
                  f"f.e{e}.down": torch.randn(D, F, generator=g, dtype=F64)})
    h = torch.randn(1, D, generator=g, dtype=F64)
    f = dict(router=dict(experts=E, top=E, scale=3.0), expert=dict(ff=F))
    s = torch.softmax(h @ W["f.router"].T, -1)[0]
    want = sum(3.0 * s[e] * plain.expert(W, f"f.e{e}.", h)[0] for e in range(E))        # all chosen: weights sum to the scale
    assert torch.allclose(plain.routed(W, "f.", f, h)[0], want)
    W.update({"f.shared.gate": torch.randn(3, D, generator=g, dtype=F64), "f.shared.up": torch.randn(3, D, generator=g, dtype=F64),
              "f.shared.down": torch.randn(D, 3, generator=g, dtype=F64), "f.shared.sg": torch.randn(1, D, generator=g, dtype=F64)})
    f["shared"] = dict(ff=3)
    extra = torch.sigmoid(h @ W["f.shared.sg"].T)[0] * plain.expert(W, "f.shared.", h)[0]
    assert torch.allclose(plain.routed(W, "f.", f, h)[0], want + extra)


def test_plain_model_runs_and_depth_average_matters(tmp_path):
    folder = S.make_folder(tmp_path, "T")
    (p,) = S.prompts_for("T", (30,))
    lg = S.plain_logits(folder, p)
    assert lg.shape == (30, 131) and np.isfinite(lg).all()
    cfg, W = S._model(folder)
    logits, handed = plain.forward(cfg, W, p, keep_layers=True)
    assert handed.shape == (4, 30, 64)
    W2 = dict(W)
    W2["l3.dwa"] = W["l3.dwa"].clone()
    W2["l3.dwa"][0] += 0.5                                  # the embedding's output reaches the last average directly
    assert np.abs(plain.forward(cfg, W2, p).numpy() - lg).max() > 1e-3
    # causal: a later token does not move earlier rows
    q = list(p)
    q[20] = (q[20] + 1) % 131
    lg2 = plain.forward(cfg, W, q).numpy()
    assert np.abs(lg2[:20] - lg[:20]).max() < 1e-12 and np.abs(lg2[20:] - lg[20:]).max() > 1e-6


def test_which_form_of_the_recurrence_a_step_takes():
    """the split form walks every token twice: it is taken for long stretches only while the scan's blocks (sequences x
    heads x 16 columns of the state) leave multiprocessors idle; its scratch is a state per segment"""
    from mashbox_b200 import ops
    assert ops.retention_scan_blocks(1, 16, 128) == 128 and ops.retention_scan_blocks(3, 2, 24) == 12
    assert ops.retention_splits(2048, 1, 16, 128) and not ops.retention_splits(2048, 1, 24, 128)
    assert not ops.retention_splits(2048, 2, 16, 128)                   # two sequences fill the device by themselves
    assert not ops.retention_splits(64, 1, 2, 16) and ops.retention_splits(65, 1, 2, 16)
    assert not ops.retention_splits(8, 8, 2, 16)                        # decode steps
    assert ops.retention_carry_rows(300, 3) == 300 // 128 + 3 and ops.retention_carry_rows(300, 3, 7) == 300 // 7 + 3
