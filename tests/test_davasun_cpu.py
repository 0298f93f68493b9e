"""CPU-side checks of the Davasun integration: configuration, layer-run order, slot state, the engine's batching and
portioning (against a recording stand-in for the model), the registry, and the oracle's own consistency."""
import json
import os

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import registry
from lia_b200.engine import Engine
from lia_b200.modeling_davasun import DavasunConfig
from lia_b200.seq_state import SlotError, SlotState

import davasun_oracle as O
from davasun_cases import CASES, config, dense, latent, mlstm


def test_layer_runs_and_shapes():
    c = DavasunConfig.from_dict(CASES["even"])
    assert c.layer_runs() == [0, 1, 2, 1, 2, 1, 2, 3] == O.layer_runs(CASES["even"])
    c = DavasunConfig.from_dict(CASES["odd"])
    assert c.layer_runs() == [0, 1, 1, 2]
    c = DavasunConfig.from_dict(CASES["wide"])
    assert c.layer_runs() == [0, 1]
    shapes = c.tensor_shapes()
    assert shapes["l1.mix.q"] == (9 * 20, 96) and shapes["l1.mix.dkv"] == (268, 96) and shapes["l0.mix.i.b"] == (2,)
    assert "l0.norm2" not in shapes and shapes["l0.norm1b"] == ()
    assert DavasunConfig.from_dict(c.to_dict()).layer_runs() == c.layer_runs()


def test_config_rejects_unknown_parts():
    bad = config([{"type": "conv", "mixer": {}, "mlp": None}], 10, 8)
    with pytest.raises(ValueError):
        DavasunConfig.from_dict(bad)
    bad = config([mlstm(1, 4, 4, mlp={"kind": "experts", "ff": 8, "limit": 1.0})], 10, 8)
    with pytest.raises(ValueError):
        DavasunConfig.from_dict(bad)
    with pytest.raises(ValueError):
        DavasunConfig.from_dict(config([mlstm(1, 4, 4)], 10, 8, loop={"start": 1, "stop": 0, "times": 1}))


def test_registry_picks_the_class_from_config_json(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(CASES["odd"]))
    assert registry.architecture_of(str(d)) == "davasun"
    assert registry.model_class(str(d)).__name__ == "DavasunForCausalLM"
    (d / "config.json").write_text(json.dumps({"architectures": ["OPTForCausalLM"], "model_type": "opt"}))
    assert registry.model_class(str(d)).__name__ == "OPTForCausalLM"
    (d / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(KeyError):
        registry.architecture_of(str(d))


def test_slot_state_alloc_free_reuse():
    s = SlotState(2, 10, "cpu")
    rec = s.add_recurrent((3,))
    rows = s.add_rows(4, torch.float32)
    assert rows.shape == (2, 10, 4)
    a, b = s.alloc("a"), s.alloc("b")
    assert (a, b) == (0, 1)
    with pytest.raises(SlotError):
        s.alloc("c")
    rec[a] += 5.0
    assert s.reserve(a, 7) == 0 and s.reserve(a, 3) == 7
    with pytest.raises(SlotError):
        s.reserve(a, 1)
    s.free("a")
    assert s.alloc("c") == 0 and s.length[0] == 0 and float(rec[0].abs().sum()) == 0.0      # reused slot starts at zero
    assert s.live_tokens == 0
    with pytest.raises(SlotError):
        s.free("a")


class _Recorder:
    """Stands in for a model: records what each pass of a step hands to forward_rows."""

    class config:
        vocab = 50

    device = torch.device("cpu")

    def __init__(self):
        self.calls = []

    def new_state(self, n, cap):
        return SlotState(n, cap, "cpu")

    def forward_rows(self, ids, batch, want, slots, trace=None):
        self.calls.append((ids.tolist(), batch.segs.tolist(), batch.meta.tolist(), None if want is None else want.tolist()))
        return None if want is None else torch.zeros(want.numel(), 50)

    def graph_class(self, max_ctx):
        from lia_b200 import ops
        return ops.latent_attn_split_class(max_ctx)


def test_engine_lays_out_entries_and_cuts_passes():
    m = _Recorder()
    e = Engine(m, max_tokens=64, max_requests=3, max_rows=5)
    out = e.step([{"id": "x", "tokens": [1, 2, 3], "want": [2]}, {"id": "y", "tokens": [4, 5, 6, 7, 8, 9, 10], "want": [0, 6]}])
    assert out.shape == (3, 50)
    (ids0, segs0, meta0, want0), (ids1, segs1, meta1, want1) = m.calls
    assert ids0 == [1, 2, 3, 4, 5] and segs0 == [[0, 0, 0, 3], [1, 0, 3, 2]] and want0 == [2, 3]
    assert meta0 == [[0, 0], [0, 1], [0, 2], [1, 0], [1, 1]]
    assert ids1 == [6, 7, 8, 9, 10] and segs1 == [[1, 2, 0, 5]] and want1 == [4] and meta1[0] == [1, 2]
    m.calls.clear()
    assert e.step([{"id": "x", "tokens": [11], "want": []}], end=["x"]) is None
    assert m.calls[0][1] == [[0, 3, 0, 1]] and m.calls[0][3] is None
    e.step([{"id": "z", "tokens": [1, 1], "want": [1]}])                 # the freed slot 0 is handed out again, from position 0
    assert m.calls[-1][1] == [[0, 0, 0, 2]]
    with pytest.raises(ValueError):
        e.step([{"id": "z", "tokens": [50], "want": []}])
    with pytest.raises(ValueError):
        e.step([{"id": "z", "tokens": [1], "want": [1]}])


def test_engine_graph_key_names_what_a_decode_pass_launch_depends_on():
    """Which passes may replay a captured graph, and which of them may share one: only passes of single tokens, with logits
    wanted for all rows or none; the key separates row counts, the wanted pattern and the attention's key-split class, and
    the split count itself depends on a history's length through that class alone."""
    from lia_b200 import ops
    e = Engine(_Recorder(), max_tokens=4096, max_requests=4)
    assert e.graphs is False and e._graph_key([(0, [1], [0])], [(0, 5, 0, 1)], [0]) is None      # no graphs off the GPU
    e.graphs = True
    one = lambda slot, p0, row: ((slot, [7], [0]), (slot, p0, row, 1))  # noqa: E731
    (g0, s0), (g1, s1) = one(0, 10, 0), one(1, 200, 1)
    assert e._graph_key([g0, g1], [s0, s1], [0, 1]) == (2, 2, ops.latent_attn_split_class(201))
    assert e._graph_key([g0, g1], [s0, s1], []) == (2, 0, ops.latent_attn_split_class(201))
    assert e._graph_key([g0, g1], [s0, s1], [1]) is None                                         # logits of some rows only
    assert e._graph_key([g0, (1, [7, 8], [1])], [s0, (1, 200, 1, 2)], [0, 2]) is None            # a portion of two tokens
    assert e._graph_key([g0], [s0], [0]) != e._graph_key([g0, g1], [s0, s1], [0, 1])
    for ctx in (1, 63, 64, 65, 127, 128, 2047, 2048, 2049, 100000):
        cls = ops.latent_attn_split_class(ctx)
        same = [c for c in range(max(1, ctx - 70), ctx + 70) if ops.latent_attn_split_class(c) == cls]
        for M, H, sms in ((1, 16, 148), (16, 32, 148), (3, 5, 8), (4096, 16, 148)):
            assert len({ops.latent_attn_splits(M, H, c, sms) for c in same}) == 1
            assert 1 <= ops.latent_attn_splits(M, H, ctx, sms) <= max(1, min(ops.LATENT_MAX_SPLITS, ctx // ops.LATENT_SPLIT_KEYS))


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_is_consistent_under_portions(name):
    """The oracle itself: one pass over a prompt equals portions of 1, 2 and more tokens through carried state."""
    cfg = CASES[name]
    w = O.random_weights(DavasunConfig.from_dict(cfg).tensor_shapes(), seed=3)
    toks = torch.randint(0, cfg["vocab"], (19,), generator=torch.Generator().manual_seed(1)).tolist()
    with torch.no_grad():
        whole = O.forward(cfg, w, toks, O.new_states(cfg))
        st, parts, at = O.new_states(cfg), [], 0
        for n in (2, 1, 7, 1, 1, 5, 2):
            parts.append(O.forward(cfg, w, toks[at:at + n], st))
            at += n
    assert at == len(toks)
    assert torch.allclose(torch.cat(parts), whole, rtol=1e-9, atol=1e-9)


def test_oracle_mechanisms():
    # rotation: norm-preserving, identity at position 0, untouched channels beyond `dims`
    x = torch.randn(3, 2, 10, dtype=torch.float64)
    y = O.rotate_half(x, torch.tensor([0, 5, 900]), 6, 100.0)
    assert torch.allclose(y[0], x[0]) and torch.allclose(y[..., 6:], x[..., 6:])
    assert torch.allclose(y[..., :6].norm(dim=-1), x[..., :6].norm(dim=-1))
    # a pair (u, v) = (1, 0) at angle a becomes (cos a, sin a)
    e = torch.zeros(1, 4, dtype=torch.float64)
    e[0, 0] = 1.0
    r = O.rotate_half(e, torch.tensor([3]), 4, 100.0)
    assert torch.allclose(r[0, [0, 2]], torch.tensor([torch.cos(torch.tensor(3.0)), torch.sin(torch.tensor(3.0))], dtype=torch.float64))
    # recurrence: with one token, S = exp(i - m) k v^T and the running maximum starts at 0, not at -inf
    q, k, v = torch.ones(1, 1, 2, dtype=torch.float64), torch.ones(1, 1, 2, dtype=torch.float64), torch.tensor([[[2.0, 4.0]]], dtype=torch.float64)
    st = {}
    o = O.mlstm_recurrence(q, k, v, torch.tensor([[-3.0]], dtype=torch.float64), torch.tensor([[-1.0]], dtype=torch.float64), st)
    assert float(st["m"]) == pytest.approx(-1.0)           # max(f + 0, i) = max(-1, -3)
    b = torch.exp(torch.tensor(-2.0, dtype=torch.float64))
    assert torch.allclose(st["S"][0], b * torch.tensor([[2.0, 4.0], [2.0, 4.0]], dtype=torch.float64))
    den = max(float(2 * b), float(torch.exp(torch.tensor(1.0)))) + 1e-6
    assert torch.allclose(o[0, 0], 2 * b * torch.tensor([2.0, 4.0], dtype=torch.float64) / den)
    # feed-forward clamps: gate only from above, up on both sides
    h = torch.eye(2, dtype=torch.float64)
    w_gate = torch.tensor([[5.0, -5.0]], dtype=torch.float64)
    w_up = torch.tensor([[9.0, -9.0]], dtype=torch.float64)
    y = O.clamped_glu(h, w_gate, w_up, torch.ones(1, 1, dtype=torch.float64), 2.0)
    g0, g1 = torch.tensor(2.0, dtype=torch.float64), torch.tensor(-5.0, dtype=torch.float64)
    assert torch.allclose(y[:, 0], torch.stack([g0 * torch.sigmoid(1.702 * g0) * 3.0, g1 * torch.sigmoid(1.702 * g1) * (-1.0)]))
