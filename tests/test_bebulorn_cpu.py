"""CPU-side checks of the Bebulorn integration: configuration and layer-run order, tensor table, registry, and the oracle's own
consistency (a prompt fed whole, in portions and token by token gives the same logits; window and state behave as stated)."""
import json

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import registry
from lia_b200.modeling_bebulorn import BebulornConfig

import bebulorn_oracle as O
from bebulorn_cases import CASES, attention, config, delta, dense, lightning, moe


def test_layer_runs_and_shapes():
    c = BebulornConfig.from_dict(CASES["even"])
    assert c.layer_runs() == O.layer_runs(CASES["even"])
    assert [i for i, _ in c.layer_runs()] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4]
    assert [a for _, a in c.layer_runs()] == [False, False, False, False, True, False, False, True, False, False, False]
    c = BebulornConfig.from_dict(CASES["odd"])
    assert c.layer_runs() == [(0, False), (0, True), (1, False), (2, False), (3, False)] == O.layer_runs(CASES["odd"])
    c = BebulornConfig.from_dict(CASES["wide"])
    assert c.layer_runs() == [(i, False) for i in range(4)]
    for name in CASES:
        c = BebulornConfig.from_dict(CASES[name])
        assert c.tensor_shapes() == O.tensor_shapes(CASES[name])
        assert BebulornConfig.from_dict(c.to_dict()).layer_runs() == c.layer_runs()
    s = BebulornConfig.from_dict(CASES["even"]).tensor_shapes()
    assert s["l0.mix.q"] == (32, 64) and s["l0.mix.v.conv"] == (96, 4) and s["l0.mix.norm"] == (24,) and s["l0.mix.b"] == (4, 64)
    assert s["l1.mlp.e5.down"] == (64, 24) and s["l1.mlp.shared.up"] == (40, 64) and "l3.mlp.shared.up" not in s
    assert "l4.norm2" not in s and s["l4.norm1b.b"] == (64,) and s["l2.mix.temp"] == (6,)


def test_config_rejects_unknown_parts():
    with pytest.raises(ValueError):
        BebulornConfig.from_dict(config([{"type": "mlstm", "mixer": {}, "mlp": None}], 10, 8))
    with pytest.raises(ValueError):
        BebulornConfig.from_dict(config([lightning(1, 4, 4, mlp={"kind": "glu", "ff": 8})], 10, 8))
    with pytest.raises(ValueError):
        BebulornConfig.from_dict(config([attention(3, 2, 4, 4, 5)], 10, 8))
    with pytest.raises(ValueError):
        BebulornConfig.from_dict(config([lightning(2, 4, 4, decay=[0.5])], 10, 8))
    with pytest.raises(ValueError):
        BebulornConfig.from_dict(config([lightning(1, 4, 4)], 10, 8, loop={"start": 1, "stop": 0, "times": 1}))


def test_config_defaults_for_what_a_layer_leaves_out():
    a = attention(4, 4, 8, 8, 5)
    del a["mixer"]["kv_heads"], a["mixer"]["vdim"]
    li = lightning(2, 8, 8, decay=[0.5, 0.5], mlp={"ff": 16})
    li["mixer"]["decay"] = 0.5
    c = BebulornConfig.from_dict(config([a, li], 10, 8))
    s = c.tensor_shapes()
    assert s["l0.mix.k"] == (32, 8) and s["l0.mix.v"] == (32, 8) and s["l1.mlp.gate"] == (16, 8)
    assert c.layers[1]["mixer"]["decay"] == [0.5, 0.5] and c.layers[1]["mlp"]["kind"] == "dense"


def test_registry_picks_the_class_from_config_json(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(CASES["odd"]))
    assert registry.architecture_of(str(d)) == "bebulorn"
    assert registry.model_class(str(d)).__name__ == "BebulornForCausalLM"
    assert registry.model_class(str(d)).step_serving


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_portions_equal_the_whole_prompt(name):
    cfg = CASES[name]
    w = O.random_weights(cfg, 3)
    toks = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = O.forward(cfg, w, toks, O.new_states(cfg))
    for cuts in ([1] * 23, [2] * 11 + [1], [7, 1, 2, 13]):
        st, outs, at = O.new_states(cfg), [], 0
        for c in cuts:
            outs.append(O.forward(cfg, w, toks[at:at + c], st))
            at += c
        assert float((torch.cat(outs) - whole).abs().max()) < 1e-9


def test_oracle_window_sees_exactly_its_size():
    cfg = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "mask": {"size": 3}, "scale": 1.0, "softcap": 50.0}
    g = torch.Generator().manual_seed(0)
    w = {"q": torch.randn(4, 6, generator=g).double(), "k": torch.randn(4, 6, generator=g).double(),
         "v": torch.randn(4, 6, generator=g).double(), "o": torch.eye(4).double(), "temp": torch.ones(1).double()}
    h = torch.randn(9, 6, generator=g).double()
    base = O.window_attention_mixer(h, w, "", cfg, 1e-6, {})
    h2 = h.clone()
    h2[2] += 5.0                                   # position 2 is seen by positions 2, 3, 4 only
    moved = O.window_attention_mixer(h2, w, "", cfg, 1e-6, {})
    changed = [(moved[i] - base[i]).abs().max() > 1e-12 for i in range(9)]
    assert changed == [False, False, True, True, True, False, False, False, False]


def test_oracle_router_weights_sum_to_one_and_pick_the_largest():
    g = torch.Generator().manual_seed(2)
    h, wr = torch.randn(5, 8, generator=g).double(), torch.randn(7, 8, generator=g).double()
    idx, wt = O.route(h, wr, 3)
    assert torch.allclose(wt.sum(-1), torch.ones(5).double())
    s = torch.softmax(h @ wr.T, -1)
    for t in range(5):
        assert set(idx[t].tolist()) == set(s[t].argsort(descending=True)[:3].tolist())
