"""GPU checks of the Bebulorn path against the plain float64 oracle (tests/bebulorn_oracle.py): every kernel and every mixer
alone, then the model through the step engine -- whole prompts, token-by-token decoding, portions down to two tokens, unequal
requests in one step, slots that are freed and reused, keys far back, at the edges of the window and of the kernels' own
tiles (32 cached positions per attention stage, 8 tokens per recurrence stage), the first tokens, long decoding, greedy
generation through generate(), the trace runner and the command line."""
import json
import os

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import ops, registry
from lia_b200.checkpoint import write_safetensors
from lia_b200.engine import Engine
from lia_b200.modeling_bebulorn import BebulornConfig, BebulornForCausalLM
from lia_b200.seq_layers import (DecayLinearAttentionMixer, DeltaRuleMixer, GatedMLP, MoEFeedForward, PlainMLP, StepBatch,
                                 WindowAttentionMixer)
from lia_b200.seq_state import SlotState

import bebulorn_oracle as O
from bebulorn_cases import CASES, attention, config, delta, dense, lightning, moe

pytestmark = pytest.mark.gpu
BF16, F32, F64 = torch.bfloat16, torch.float32, torch.float64
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def bf(t):
    """bf16-representable fp32 numbers."""
    return t.to(BF16).float()


def make_batch(portions):
    """portions: (slot, first position, tokens) in row order."""
    segs, meta, row = [], [], 0
    for slot, p0, n in portions:
        segs.append((slot, p0, row, n))
        meta += [(slot, p0 + i) for i in range(n)]
        row += n
    return StepBatch(row, i32(segs), i32(meta), max(p0 + n for _, p0, n in portions))


def run_mixer(mixer, h, cuts, slot=1, n_slots=3, capacity=None):
    """Feed ``h`` [T, W] through ``mixer`` in portions of ``cuts`` tokens as sequence ``slot``; returns the outputs [T, W]."""
    slots = SlotState(n_slots, capacity or h.shape[0], DEV)
    state = mixer.new_state(slots)
    outs, at = [], 0
    for c in cuts:
        outs.append(mixer(h[at:at + c].to(device=DEV, dtype=mixer.dtype).contiguous(), make_batch([(slot, at, c)]), state).float().cpu())
        at += c
    assert at == h.shape[0]
    return torch.cat(outs)


# ------------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("W", [44, 256, 1000])
def test_embed_and_layer_norm_kernels(W):
    g = gen(0)
    table = torch.randn(37, W, generator=g).to(BF16)
    ids = torch.randint(0, 37, (9,), generator=g)
    x = torch.empty(9, W, dtype=F32, device=DEV)
    x0 = torch.empty(9, W, dtype=F32, device=DEV)
    ops.embed_rows(ids.to(DEV), table.to(DEV), x, x0)
    assert torch.equal(x.cpu(), table.float()[ids]) and torch.equal(x0, x)
    y = torch.randn(9, W, generator=g) * 3.0 + 1.5                    # a mean far from zero: the variance is of the deviations
    post = (torch.randn(W, generator=g), torch.randn(W, generator=g))
    pre = (torch.randn(W, generator=g), torch.randn(W, generator=g))
    dev = lambda p: tuple(t.to(DEV) for t in p)  # noqa: E731
    start = table.float()[ids].double()
    for ydt, hdt, tol in ((F32, F32, 2e-6), (BF16, BF16, 6e-3)):
        x = start.float().to(DEV)
        yy = y.to(ydt)
        h = torch.empty(9, W, dtype=hdt, device=DEV)
        ops.ln_add_norm(x, yy.to(DEV), dev(post), 0.6, dev(pre), h, 1e-5)
        x_want = start + 0.6 * O.layer_norm(yy.double(), post[0].double(), post[1].double(), 1e-5)
        assert rel(x, x_want) < 2e-6                                  # the residual sum is fp32 whatever the activations are
        assert rel(h, O.layer_norm(x_want, pre[0].double(), pre[1].double(), 1e-5)) < tol
    # the embedding added back, then the norm; and the add alone
    x = start.float().to(DEV)
    h = torch.empty(9, W, dtype=F32, device=DEV)
    ops.ln_add_norm(x, None, None, 1.0, dev(pre), h, 1e-5, extra=x0)
    assert rel(x, 2 * start) < 1e-6 and rel(h, O.layer_norm(2 * start, pre[0].double(), pre[1].double(), 1e-5)) < 2e-6
    ops.ln_add_norm(x, y.to(DEV), dev(post), 1.0, None, None, 1e-5)
    x_want = 2 * start + O.layer_norm(y.double(), post[0].double(), post[1].double(), 1e-5)
    assert rel(x, x_want) < 2e-6
    rows = i32([8, 0, 3])
    hn = torch.empty(3, W, dtype=F32, device=DEV)
    ops.ln_gather(x, rows, dev(pre), hn, 1e-5)
    assert rel(hn, O.layer_norm(x.double().cpu()[[8, 0, 3]], pre[0].double(), pre[1].double(), 1e-5)) < 2e-6


def test_gated_activations():
    g = gen(1)
    a = torch.randn(7, 50, generator=g) * 2
    out = torch.empty(7, 20, dtype=F32, device=DEV)
    ops.gated_act(a.to(DEV), 20, out, ops.ACT_RELU, up_off=24)
    assert rel(out, torch.relu(a[:, :20].double()) * a[:, 24:44].double()) < 1e-6
    ops.gated_act(a.to(DEV), 20, out, ops.ACT_GELU_ERF)
    assert rel(out, O.gelu_erf(a[:, :20].double())) < 1e-6
    ops.gated_act(a.to(DEV), 20, out, ops.ACT_SILU, up_off=30)
    assert rel(out, O.silu(a[:, :20].double()) * a[:, 30:50].double()) < 1e-6
    z = a[:, :20].double()
    ops.gated_act(a.to(DEV), 20, out, ops.ACT_GELU_TANH)
    assert rel(out, 0.5 * z * (1 + torch.tanh((2 / torch.pi) ** 0.5 * (z + 0.044715 * z ** 3)))) < 1e-6
    ob = torch.empty(7, 20, dtype=BF16, device=DEV)
    ops.gated_act(a.to(BF16).to(DEV), 20, ob, ops.ACT_RELU, up_off=24)
    assert rel(ob, torch.relu(bf(a)[:, :20].double()) * bf(a)[:, 24:44].double()) < 5e-3


@pytest.mark.parametrize("M,E,top", [(1, 1, 1), (9, 5, 3), (70, 40, 1), (6, 40, 40), (33, 7, 7)])
def test_router_picks_and_weights(M, E, top):
    g = gen(2)
    z = torch.randn(M, E, generator=g) * 2
    idx = torch.empty(M, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(M, top, dtype=F32, device=DEV)
    ops.router_topk(z.to(DEV), top, idx, wt)
    s = torch.softmax(z.double(), -1)
    val, want_idx = torch.topk(s, top, dim=-1)
    assert torch.equal(idx.cpu().long(), want_idx)                      # in the order of the scores
    assert rel(wt, val / (val.sum(-1, keepdim=True) + 1e-20)) < 1e-5


@pytest.mark.parametrize("M,E,top,shared,dtype", [(5, 6, 2, 12, F32), (100, 6, 2, 12, F32), (130, 3, 3, None, F32), (64, 9, 1, 5, F32),
                                                  (200, 4, 2, 16, BF16), (3, 4, 2, 16, BF16), (700, 5, 2, 16, BF16), (300, 7, 1, None, BF16)])
def test_mixture_of_experts_in_both_forms(M, E, top, shared, dtype):
    """Few (token, choice) pairs take one warp per output, many are grouped by expert into tiles (in bf16 from 512 pairs on:
    gathered expert by expert and run through the tensor-core GEMM, one expert left without a token); all against the oracle's
    token-by-token loop.  The router's weights are scaled up so that the choice is never a near-tie."""
    g = gen(3)
    W, ff = 40, 24
    w = {"router": bf(torch.randn(E, W, generator=g) * 2.0)}
    if M >= 300:
        w["router"][E - 1] = 0.0
        w["router"][E - 1, 0] = -50.0            # with h[:, 0] = 1 below, the last expert is never chosen
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = bf(torch.randn(ff, W, generator=g) * W ** -0.5), bf(torch.randn(W, ff, generator=g) * ff ** -0.5)
    cfg = {"router": {"experts": E, "top": top}, "expert": {"ff": ff}}
    sh = None
    if shared is not None:
        w["shared.up"], w["shared.down"] = bf(torch.randn(shared, W, generator=g) * W ** -0.5), bf(torch.randn(W, shared, generator=g) * shared ** -0.5)
        cfg["shared"] = {"ff": shared}
        sh = PlainMLP({"up": w["shared.up"], "down": w["shared.down"]}, shared, ops.ACT_GELU_ERF, dtype, DEV)
    m = MoEFeedForward(w["router"], [{"up": w[f"e{e}.up"], "down": w[f"e{e}.down"]} for e in range(E)], top, ff, ops.ACT_GELU_ERF, sh, dtype, DEV)
    h = bf(torch.randn(M, W, generator=g))
    if M >= 300:
        h[:, 0] = 1.0
    got = m(h.to(device=DEV, dtype=dtype))
    assert got.dtype == F32
    want = O.moe(h.double(), {k: v.double() for k, v in w.items()}, "", cfg)
    assert rel(got, want) < (1e-5 if dtype == F32 else 2e-2)


@pytest.mark.parametrize("H,dim,vdim,dtype", [(1, 8, 5, F32), (3, 32, 40, F32), (2, 72, 136, F32), (2, 40, 24, BF16), (1, 264, 16, F32)])
def test_decay_recurrence_keeps_a_far_token(H, dim, vdim, dtype):
    """Head 0 does not decay at all: what the first token wrote is still read, unchanged, hundreds of tokens later; the other
    heads forget at their own rates.  Portions cut at and around the kernel's 8-token stages."""
    g = gen(4)
    T = 300
    q, k, v = (bf(torch.randn(T, H * d, generator=g) * 0.3) for d in (dim, dim, vdim))
    k[1:, :dim] = 0.0                                                   # head 0: only token 0 ever writes
    decay = [1.0] + [0.5 + 0.4 * i / H for i in range(1, H)]
    want = O.lightning_recurrence(q.double().view(T, H, dim), k.double().view(T, H, dim), v.double().view(T, H, vdim),
                                  torch.tensor(decay, dtype=F64), {}).reshape(T, H * vdim)
    assert rel(want[299, :vdim], (q[299, :dim].double() @ k[0, :dim].double()) * v[0, :vdim].double()) < 1e-9
    S = torch.zeros(2, H, vdim, dim, device=DEV)
    buf = torch.cat([q, k, v], 1).to(device=DEV, dtype=dtype)
    o = torch.empty(T, H * vdim, dtype=F32, device=DEV)
    at = 0
    for c in (1, 7, 8, 9, 16, 2, 1, 255, 1):
        b = make_batch([(1, at, c)])
        rows = buf[at:at + c]
        ops.linear_scan(rows[:, :H * dim], rows[:, H * dim:2 * H * dim], rows[:, 2 * H * dim:], S, b.segs, H, H, dim, vdim, o[at:at + c],
                        decay=torch.tensor(decay, device=DEV))
        at += c
    assert at == T and rel(o, want) < 2e-5
    assert float(S[0].abs().max()) == 0.0                               # the other slot was not touched


@pytest.mark.parametrize("H,G,dim,vdim", [(1, 1, 8, 5), (4, 2, 32, 40), (6, 1, 72, 136), (3, 3, 136, 16)])
def test_delta_recurrence_against_the_loop(H, G, dim, vdim):
    g = gen(5)
    T = 120
    q, k = (O.unit(torch.randn(T, G, dim, generator=g).double()) for _ in range(2))
    q = (q * dim ** -0.5).float()
    k = k.float()
    v = torch.randn(T, H * vdim, generator=g)
    beta, gt = torch.rand(T, H, generator=g), 1.0 - 0.1 * torch.rand(T, H, generator=g)
    gt[:, 0] = 1.0                                                      # head 0 never forgets
    rep = H // G
    want = O.delta_recurrence(q.double().repeat_interleave(rep, 1), k.double().repeat_interleave(rep, 1), v.double().view(T, H, vdim),
                              beta.double(), gt.double(), {}).reshape(T, H * vdim)
    S = torch.zeros(2, H, vdim, dim, device=DEV)
    qk = torch.cat([q.reshape(T, G * dim), k.reshape(T, G * dim)], 1).to(DEV)
    gates = torch.cat([beta, gt], 1).to(DEV)
    o = torch.empty(T, H * vdim, dtype=F32, device=DEV)
    at = 0
    for c in (1, 2, 8, 9, 7, 93):
        b = make_batch([(0, at, c)])
        ops.linear_scan(qk[at:at + c, :G * dim], qk[at:at + c, G * dim:], v.to(DEV)[at:at + c], S, b.segs, H, G, dim, vdim, o[at:at + c],
                        gates=gates[at:at + c].contiguous())
        at += c
    assert at == T and rel(o, want) < 5e-5


def _attention_reference(q, kc, vc, pos, H, G, window, scale, temp, cap):
    """q [H, dim]; kc [n, G, dim], vc [n, G, vdim] of one sequence; the keys pos - window < j <= pos."""
    lo = max(0, pos - window + 1)
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (kc[lo:pos + 1, g].double() @ q[h].double()) * scale * float(temp[h])
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        out.append(torch.softmax(s, 0) @ vc[lo:pos + 1, g].double())
    return torch.stack(out)


@pytest.mark.parametrize("H,G,dim,vdim,window,dtype", [(1, 1, 12, 10, 5, F32), (6, 2, 24, 16, 33, F32), (9, 3, 72, 80, 1, F32),
                                                       (4, 4, 8, 136, 64, F32), (16, 2, 16, 40, 32, F32), (5, 5, 40, 56, 31, BF16)])
def test_window_attention_kernel_at_the_edges(H, G, dim, vdim, window, dtype):
    g = gen(6)
    cap_rows = 200
    kc = torch.randn(2, cap_rows, G * dim, generator=g).to(dtype)
    vc = torch.randn(2, cap_rows, G * vdim, generator=g).to(dtype)
    temp = 0.5 + torch.rand(H, generator=g)
    positions = [0, 1, window - 1, window, window + 1, 30, 31, 32, 33, 63, 64, 65, 127, 199]
    positions = sorted({p for p in positions if 0 <= p < cap_rows})
    q = torch.randn(len(positions), H * dim + 8, generator=g).to(dtype)
    out = torch.empty(len(positions), H * vdim, dtype=dtype, device=DEV)
    ops.window_attn(q.to(DEV)[:, 8:], kc.to(DEV), vc.to(DEV), i32([(1, p) for p in positions]), temp.to(DEV), out, H, G, dim, vdim, window,
                    0.3, 4.0)
    tol = 2e-5 if dtype == F32 else 1e-2
    for r, p in enumerate(positions):
        want = _attention_reference(q[r, 8:].float().view(H, dim), kc[1].float().view(-1, G, dim), vc[1].float().view(-1, G, vdim), p, H, G,
                                    window, 0.3, temp, 4.0)
        assert rel(out[r].view(H, vdim), want) < tol, (r, p)
    if dtype != F32:
        return
    # one key made to stand out (no cap, so it takes all the weight): just inside the window it is the output; moved one place
    # further back it is not seen at all, however strong; the same at the far edge of a window that spans several stages
    for p in (150, 199, 64):
        inside, outside = p - window + 1, p - window
        for place, seen in ((inside, True), (outside, False)):
            if place < 0:
                continue
            k2 = kc[1].float().clone().view(-1, G, dim) * 0.05
            key = torch.randn(dim, generator=g)
            key /= key.norm()
            k2[place, 0] = key * 8.0
            q2 = torch.zeros(1, H * dim)
            q2[0, :dim] = key * 8.0
            kk = kc.float().clone()
            kk[1] = k2.view(-1, G * dim)
            o2 = torch.empty(1, H * vdim, dtype=F32, device=DEV)
            ops.window_attn(q2.to(DEV), kk.to(DEV), vc.float().to(DEV), i32([(1, p)]), torch.ones(H, device=DEV), o2, H, G, dim, vdim, window,
                            1.0, 0.0)
            want = _attention_reference(q2[0].view(H, dim), k2, vc[1].float().view(-1, G, vdim), p, H, G, window, 1.0, torch.ones(H), 0.0)
            assert rel(o2.view(H, vdim), want) < 2e-5
            took_it = rel(o2.view(H, vdim)[0], vc[1, place].float().view(G, vdim)[0]) < 1e-3
            assert took_it == seen, (p, place)


def test_kv_store_normalises_values_per_head():
    g = gen(7)
    G, dim, vdim, M = 3, 10, 20, 4
    k, v = torch.randn(M, G * dim + 8, generator=g), torch.randn(M, G * vdim, generator=g) * 3
    kc, vc = torch.zeros(2, 50, G * dim, device=DEV), torch.zeros(2, 50, G * vdim, device=DEV)
    meta = [(0, 0), (0, 1), (1, 40), (1, 41)]
    ops.kv_store(k.to(DEV)[:, 8:], v.to(DEV), i32(meta), kc, vc, G, dim, vdim, 1e-5)
    for r, (s, p) in enumerate(meta):
        assert torch.equal(kc[s, p].cpu(), k[r, 8:])
        assert rel(vc[s, p], O.rms_div(v[r].double().view(G, vdim), 1e-5).reshape(-1)) < 1e-6
    assert float(kc[0, 2:].abs().max()) == 0.0 and float(vc[1, :40].abs().max()) == 0.0


# ------------------------------------------------------------------------------------------------ mixers alone
def _mixer_weights(shapes, seed):
    g = gen(seed)
    out = {}
    for n, s in shapes.items():
        if n.endswith(".conv"):
            out[n] = bf(torch.randn(s, generator=g) * 0.5)
        elif len(s) == 2:
            out[n] = bf(torch.randn(s, generator=g) * s[1] ** -0.5)
        elif n in ("norm", "temp"):
            out[n] = bf(1 + 0.2 * torch.randn(s, generator=g))
        else:
            out[n] = bf(0.5 * torch.randn(s, generator=g))
    return out


CUTS = {"whole": [60], "token by token": [1] * 60, "twos": [2] * 30, "ragged": [31, 1, 1, 2, 22, 3], "stage edges": [8, 8, 1, 7, 32, 4]}


@pytest.mark.parametrize("H,dim,vdim,W", [(3, 16, 40, 64), (1, 36, 20, 44), (2, 80, 136, 96)])
def test_lightning_mixer_alone(H, dim, vdim, W):
    w = _mixer_weights({"q": (H * dim, W), "k": (H * dim, W), "v": (H * vdim, W), "g": (H * vdim, W), "o": (W, H * vdim), "norm": (H * vdim,)}, 8)
    cfg = {"heads": H, "dim": dim, "vdim": vdim, "decay": [1.0 - 0.3 / (i + 1) for i in range(H)]}
    h = bf(torch.randn(60, W, generator=gen(9)))
    want = O.lightning_mixer(h.double(), {k: v.double() for k, v in w.items()}, "", cfg, 1e-5, {})
    m = DecayLinearAttentionMixer(w, H, dim, vdim, cfg["decay"], 1e-5, F32, DEV)
    for label, cuts in CUTS.items():
        assert rel(run_mixer(m, h, cuts), want) < 5e-5, label


@pytest.mark.parametrize("H,G,dim,vdim,taps,W", [(4, 2, 16, 24, 4, 64), (3, 1, 10, 7, 1, 44), (3, 3, 12, 34, 5, 44), (2, 1, 136, 72, 3, 96),
                                                 (2, 2, 40, 8, 2, 64)])
def test_delta_mixer_alone(H, G, dim, vdim, taps, W):
    """The convolution's state crosses every cut: portions of one and two tokens are shorter than its taps - 1 inputs."""
    w = _mixer_weights({"q": (G * dim, W), "q.conv": (G * dim, taps), "k": (G * dim, W), "k.conv": (G * dim, taps), "v": (H * vdim, W),
                        "v.conv": (H * vdim, taps), "b": (H, W), "a": (H, W), "A_log": (H,), "dt_bias": (H,), "norm": (vdim,),
                        "g": (H * vdim, W), "o": (W, H * vdim)}, 10)
    cfg = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "conv": taps}
    h = bf(torch.randn(60, W, generator=gen(11)))
    want = O.delta_mixer(h.double(), {k: v.double() for k, v in w.items()}, "", cfg, 1e-5, {})
    m = DeltaRuleMixer(w, H, G, dim, vdim, taps, 1e-5, F32, DEV)
    for label, cuts in CUTS.items():
        assert rel(run_mixer(m, h, cuts), want) < 1e-4, label


@pytest.mark.parametrize("H,G,dim,vdim,window,W", [(6, 2, 24, 16, 11, 64), (1, 1, 12, 10, 500, 44), (9, 3, 72, 80, 1, 96), (4, 4, 8, 136, 33, 96)])
def test_window_attention_mixer_alone(H, G, dim, vdim, window, W):
    w = _mixer_weights({"q": (H * dim, W), "k": (G * dim, W), "v": (G * vdim, W), "temp": (H,), "o": (W, H * vdim)}, 12)
    cfg = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": dim ** -0.5 * 3, "softcap": 5.0}
    h = bf(torch.randn(60, W, generator=gen(13)))
    want = O.window_attention_mixer(h.double(), {k: v.double() for k, v in w.items()}, "", cfg, 1e-5, {})
    m = WindowAttentionMixer(w, H, G, dim, vdim, window, cfg["scale"], 5.0, 1e-5, F32, DEV)
    for label, cuts in CUTS.items():
        assert rel(run_mixer(m, h, cuts), want) < 5e-5, label


def test_two_sequences_in_one_batch_keep_their_own_state():
    """Portions of two sequences side by side in one step (rows of different slots next to each other): the convolution must
    not read across the border, and each recurrence continues from its own slot."""
    H, G, dim, vdim, taps, W = 4, 2, 16, 24, 4, 64
    w = _mixer_weights({"q": (G * dim, W), "q.conv": (G * dim, taps), "k": (G * dim, W), "k.conv": (G * dim, taps), "v": (H * vdim, W),
                        "v.conv": (H * vdim, taps), "b": (H, W), "a": (H, W), "A_log": (H,), "dt_bias": (H,), "norm": (vdim,),
                        "g": (H * vdim, W), "o": (W, H * vdim)}, 14)
    cfg = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "conv": taps}
    ha, hb = bf(torch.randn(20, W, generator=gen(15))), bf(torch.randn(9, W, generator=gen(16)))
    wd = {k: v.double() for k, v in w.items()}
    want_a, want_b = O.delta_mixer(ha.double(), wd, "", cfg, 1e-5, {}), O.delta_mixer(hb.double(), wd, "", cfg, 1e-5, {})
    m = DeltaRuleMixer(w, H, G, dim, vdim, taps, 1e-5, F32, DEV)
    slots = SlotState(3, 32, DEV)
    state = m.new_state(slots)
    got_a, got_b = [], []
    plan = [(12, 1), (1, 2), (7, 6)]                     # tokens of a, of b per step; b sits in the rows right after a
    ia = ib = 0
    for na, nb in plan:
        rows = torch.cat([ha[ia:ia + na], hb[ib:ib + nb]]).to(DEV)
        out = m(rows, make_batch([(2, ia, na), (0, ib, nb)]), state).cpu()
        got_a.append(out[:na]); got_b.append(out[na:])
        ia += na; ib += nb
    assert rel(torch.cat(got_a), want_a) < 1e-4 and rel(torch.cat(got_b), want_b) < 1e-4


def test_dense_feed_forward():
    g = gen(17)
    W, ff = 44, 30
    w = {"gate": bf(torch.randn(ff, W, generator=g) * W ** -0.5), "up": bf(torch.randn(ff, W, generator=g) * W ** -0.5),
         "down": bf(torch.randn(W, ff, generator=g) * ff ** -0.5)}
    h = bf(torch.randn(70, W, generator=g))
    got = GatedMLP(w, ff, ops.ACT_RELU, F32, DEV)(h.to(DEV))
    assert rel(got, O.relu_glu(h.double(), w["gate"].double(), w["up"].double(), w["down"].double())) < 1e-5


# ------------------------------------------------------------------------------------------------ the model
def build(name, dtype, seed=11, std_scale=1.0):
    cfg = CASES[name] if isinstance(name, str) else name
    c = BebulornConfig.from_dict(cfg)
    w = O.random_weights(cfg, seed, std_scale)
    m = BebulornForCausalLM(c, DEV, dtype).load_weights(lambda n: w[n])
    return cfg, w, m


def oracle_logits(cfg, w, toks):
    with torch.no_grad():
        return O.forward(cfg, w, toks, O.new_states(cfg))


def toks_for(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=gen(seed)).tolist()


def err(got, want, reduce="max"):
    """The measure a serving check would use: rms over the vocabulary of the centred difference, relative to the logits' rms."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    e = d.pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    return float(e.max() if reduce == "max" else e.mean())


@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompt_fp32_and_every_layer_run(name):
    cfg, w, m = build(name, F32)
    toks = toks_for(cfg, 45, 1)
    trace_o, trace_m = [], []
    with torch.no_grad():
        want = O.forward(cfg, w, toks, O.new_states(cfg), trace_o)
    eng = Engine(m, 64, 2)
    got = eng.step([{"id": 0, "tokens": toks, "want": list(range(45))}], trace=trace_m)
    assert len(trace_m) == len(trace_o) == len(O.layer_runs(cfg))
    for r, (a, b) in enumerate(zip(trace_m, trace_o)):
        assert rel(a, b) < 2e-4, f"residual stream after layer run {r}"
    assert err(got, want) < 2e-4


@pytest.mark.parametrize("name", sorted(CASES))
def test_bf16_model_stays_within_rounding(name):
    cfg, w, m = build(name, BF16)
    toks = toks_for(cfg, 70, 2)
    got = Engine(m, 80, 1).step([{"id": 0, "tokens": toks, "want": list(range(70))}])
    # bf16 rounding of the projections through up to 11 narrow layer runs: a few percent of the logits' rms, where a wrong
    # slice, state or constant shows as an error of order 1.  (A routed layer may send a token to another expert when two
    # scores are within rounding of each other; the mean shows that this is rare.)
    want = oracle_logits(cfg, w, toks)
    assert err(got, want, "mean") < 0.08


@pytest.mark.parametrize("name,dtype", [("even", F32), ("odd", F32), ("wide", F32), ("even", BF16)])
def test_portions_and_decoding_equal_the_whole_prompt(name, dtype):
    cfg, w, m = build(name, dtype)
    n = 75
    toks = toks_for(cfg, n, 3)
    eng = Engine(m, 100, 2)
    whole = eng.step([{"id": "w", "tokens": toks, "want": list(range(n))}], end=["w"])
    schedules = {"token by token": [1] * n, "twos": [2] * 37 + [1],
                 "ragged": [31, 1, 1, 2, 30, 3, 7], "stage edges": [32, 32, 8, 1, 1, 1], "prompt then decode": [n - 33] + [1] * 33}
    for label, cuts in schedules.items():
        assert sum(cuts) == n
        outs, at = [], 0
        for c in cuts:
            outs.append(eng.step([{"id": label, "tokens": toks[at:at + c], "want": list(range(c))}]))
            at += c
        eng.step([], end=[label])
        if dtype == F32:
            assert err(torch.cat(outs), whole.double().cpu()) < 1e-4, label
        else:       # bf16: GEMM tiles differ with the row count, so portions differ by rounding
            assert err(torch.cat(outs), whole.double().cpu(), "mean") < 0.08, label
    if dtype == F32:
        assert err(whole, oracle_logits(cfg, w, toks)) < 2e-4


def test_unequal_requests_in_one_step_equal_each_alone():
    cfg, w, m = build("even", F32)
    eng = Engine(m, 64, 4)
    prompts = {"a": toks_for(cfg, 40, 4), "b": toks_for(cfg, 3, 5), "c": toks_for(cfg, 17, 6)}
    alone = {}
    for k, t in prompts.items():
        alone[k] = eng.step([{"id": k, "tokens": t, "want": list(range(len(t)))}], end=[k])
    # one step holds a portion of a, the whole of b and a single token of c; later steps mix decoding with a portion
    got = {k: [] for k in prompts}
    plan = [{"a": 25, "b": 3, "c": 1}, {"a": 1, "c": 10}, {"a": 14, "c": 6}]
    at = {k: 0 for k in prompts}
    for step in plan:
        entries = [{"id": k, "tokens": prompts[k][at[k]:at[k] + n], "want": list(range(n))} for k, n in step.items()]
        out = eng.step(entries)
        o = 0
        for k, n in step.items():
            got[k].append(out[o:o + n])
            o += n
            at[k] += n
    for k in prompts:
        assert at[k] == len(prompts[k])
        assert err(torch.cat(got[k]), alone[k].double().cpu()) < 1e-4, k
        assert err(alone[k], oracle_logits(cfg, w, prompts[k])) < 2e-4


def test_freed_slots_are_reused_clean_and_passes_cut_long_entries():
    cfg, w, m = build("odd", F32)
    eng = Engine(m, 48, 2, max_rows=16)                              # a 40-token entry runs as passes of 16, 16 and 8 rows
    t1, t2, t3 = toks_for(cfg, 40, 7), toks_for(cfg, 33, 8), toks_for(cfg, 9, 9)
    a = eng.step([{"id": 1, "tokens": t1, "want": [0, 15, 16, 39]}], end=[1])
    assert err(a, oracle_logits(cfg, w, t1)[[0, 15, 16, 39]]) < 2e-4
    b = eng.step([{"id": 2, "tokens": t2, "want": [32]}, {"id": 3, "tokens": t3, "want": [8]}], end=[2])       # slot 0 again
    assert err(b[:1], oracle_logits(cfg, w, t2)[[32]]) < 2e-4 and err(b[1:], oracle_logits(cfg, w, t3)[[8]]) < 2e-4
    c = eng.step([{"id": 4, "tokens": t1[:5], "want": [4]}], end=[3, 4])                                    # and once more
    assert err(c, oracle_logits(cfg, w, t1[:5])[[4]]) < 2e-4
    assert eng.slots.live_tokens == 0


@pytest.mark.parametrize("window", [7, 32, 45])
def test_window_edge_through_the_model_in_prompts_and_in_decoding(window):
    """One attention layer with flat weights (every key of the window counts): changing the token that sits just inside the
    window of the last position changes its logits, changing the one just outside does not -- in a whole prompt and when the
    last tokens are decoded one by one, with the edge falling inside a prompt portion or among the decoded tokens."""
    cfg = config([attention(2, 1, 16, 16, window, scale=0.5, softcap=1000.0)], vocab=50, width=32, eps=1e-5)
    _, w, m = build(cfg, F32, seed=12)
    n = 100
    toks = toks_for(cfg, n, 10)
    inside, outside = n - window, n - window - 1
    eng = Engine(m, n, 1)
    base = oracle_logits(cfg, w, toks)[-1:]
    for place, seen in ((inside, True), (outside, False)):
        variant = list(toks)
        variant[place] = (variant[place] + 1) % cfg["vocab"]
        want = oracle_logits(cfg, w, variant)[-1:]
        assert (err(want, base) > 1e-3) == seen
        whole = eng.step([{"id": 0, "tokens": variant, "want": [n - 1]}], end=[0])
        assert err(whole, want) < 2e-4
        for first in (n - 3, n - window + 2, max(1, n - window - 10)):       # the edge among decoded tokens, or in the prompt
            eng.step([{"id": 1, "tokens": variant[:first], "want": []}])
            for t in variant[first:-1]:
                eng.step([{"id": 1, "tokens": [t], "want": []}])
            last = eng.step([{"id": 1, "tokens": variant[-1:], "want": [0]}], end=[1])
            assert err(last, want) < 2e-4, (place, first)


def test_recurrences_reach_far_back_through_the_model():
    """Lightning heads that do not decay and a delta layer: the logits at the end depend on an early token, 300 positions
    back; replacing it changes them, and the model follows the oracle in both cases."""
    cfg = config([lightning(2, 16, 16, decay=[1.0, 0.999]), delta(2, 1, 16, 16, 3)], vocab=40, width=32, eps=1e-5, mult=1.0)
    _, w, m = build(cfg, F32, seed=13)
    n = 300
    toks = toks_for(cfg, n, 14)
    eng = Engine(m, n, 1)
    wants = []
    for variant in (toks, toks[:2] + [toks[2] ^ 1] + toks[3:]):
        want = oracle_logits(cfg, w, variant)[n - 20:]
        wants.append(want)
        assert eng.step([{"id": 0, "tokens": variant[:n - 20], "want": []}]) is None
        outs = [eng.step([{"id": 0, "tokens": [t], "want": [0]}]) for t in variant[n - 20:]]
        eng.step([], end=[0])
        assert err(torch.cat(outs), want) < 2e-4
    assert err(wants[0], wants[1]) > 1e-3


def test_long_decoding_keeps_the_state_exact():
    cfg, w, m = build("even", F32)
    n = 260
    toks = toks_for(cfg, n, 13)
    eng = Engine(m, n, 1)
    eng.step([{"id": 0, "tokens": toks[:4], "want": []}])
    outs = [eng.step([{"id": 0, "tokens": [t], "want": [0]}]) for t in toks[4:]]
    want = oracle_logits(cfg, w, toks)[4:]
    assert err(torch.cat(outs), want) < 2e-4


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_graphed_decode_passes_equal_eager_ones_bit_for_bit(dtype):
    """Decode passes replayed as CUDA graphs against the same passes launched one kernel at a time: two requests of unequal
    history, steps that want no logits, a request that ends and another that takes over its slot while the graphs stay in use."""
    cfg, w, m = build("even", dtype)
    a, b, c = toks_for(cfg, 129, 40), toks_for(cfg, 60, 41), toks_for(cfg, 30, 42)

    def play(graphs):
        eng = Engine(m, 130, 2, graphs=graphs)
        outs = [eng.step([{"id": "a", "tokens": a[:50], "want": [49]}, {"id": "b", "tokens": b[:3], "want": [2]}])]
        for i in range(50):
            want = [] if i % 7 == 3 else [0]
            o = eng.step([{"id": "a", "tokens": [a[50 + i]], "want": want}, {"id": "b", "tokens": [b[3 + i]], "want": want}])
            assert (o is None) == (not want)
            if o is not None:
                outs.append(o)
        eng.step([], end=["b"])
        outs.append(eng.step([{"id": "c", "tokens": c[:1], "want": [0]}]))           # b's slot, state zeroed; alone in its pass
        for i in range(1, 30):
            outs.append(eng.step([{"id": "c", "tokens": [c[i]], "want": [0]}, {"id": "a", "tokens": [a[99 + i]], "want": [0]}]))
        return torch.cat(outs), eng

    eager, _ = play(False)
    graphed, eng = play(True)
    assert sum(g.graph is not None for g in eng._step_graphs.values()) >= 2           # several shapes were captured and replayed
    assert torch.equal(eager, graphed)
    if dtype == F32:
        la, lc = oracle_logits(cfg, w, a), oracle_logits(cfg, w, c)
        assert err(graphed[-2:-1], lc[29:30]) < 2e-4 and err(graphed[-1:], la[128:129]) < 2e-4      # the last pass: c, then a


def test_first_tokens_and_single_token_prompts():
    cfg, w, m = build("wide", F32)
    eng = Engine(m, 8, 3)
    for seed in (20, 21, 22):
        t = toks_for(cfg, 1, seed)
        got = eng.step([{"id": seed, "tokens": t, "want": [0]}])
        assert err(got, oracle_logits(cfg, w, t)) < 2e-4
    t = toks_for(cfg, 5, 23)
    eng.step([], end=[20, 21, 22])
    got = torch.cat([eng.step([{"id": "s", "tokens": [x], "want": [0]}]) for x in t])
    assert err(got, oracle_logits(cfg, w, t)) < 2e-4


def _write_checkpoint(tmp_path, cfg, seed):
    w = O.random_weights(cfg, seed)
    d = tmp_path / "ckpt"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: v.to(BF16) for k, v in w.items()})
    return str(d), w


def test_greedy_generation_through_generate_and_from_pretrained(tmp_path):
    cfg = CASES["even"]
    ckpt, w = _write_checkpoint(tmp_path, cfg, 14)
    m = registry.load_model(ckpt, device=DEV, dtype=F32)
    assert isinstance(m, BebulornForCausalLM)
    prompts = torch.tensor([toks_for(cfg, 12, 30), toks_for(cfg, 12, 31)])
    new = 10
    out = m.generate(prompts, max_new_tokens=new)
    out_chunked = m.generate(prompts, max_new_tokens=new, chunk=5)
    assert out.shape == (2, 12 + new) and torch.equal(out[:, :12], prompts)
    # teacher-forced against the oracle: every greedy pick is the oracle's argmax wherever its top-2 margin is not a near-tie
    for b in range(2):
        lg = oracle_logits(cfg, w, out[b].tolist())
        for t in range(new):
            top = lg[11 + t].topk(2)
            if float(top.values[0] - top.values[1]) > 1e-3:
                assert int(out[b, 12 + t]) == int(top.indices[0]), (b, t)
                assert int(out_chunked[b, 12 + t]) == int(out[b, 12 + t])


def test_trace_runner_and_command_line_as_a_user_calls_them(tmp_path):
    """The two programs a user runs, as child processes on a small checkpoint: the trace runner (steps on standard input,
    one logits file per step that wants some, 'done <step>' lines, slots given back by 'end') in both dtypes against the
    oracle, and run.py's generation summary."""
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = CASES["even"]
    ckpt, w = _write_checkpoint(tmp_path, cfg, 15)
    a, b = toks_for(cfg, 41, 50), toks_for(cfg, 6, 51)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},              # nothing wanted: no file
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:40], "want": [7]}], "end": []}]
    steps += [{"step": 3, "entries": [{"id": "a", "tokens": a[40:41], "want": [0]}], "end": ["a"]},
              {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]}]               # a's slot, handed out again
    la, lb = oracle_logits(cfg, w, a), oracle_logits(cfg, w, b)
    want = {0: la[[0, 29]], 2: la[[39]], 3: la[[40]], 4: lb[[5]]}
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 0.2)):
        out = tmp_path / ("out_" + dtype)
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", ckpt, "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == ["done %d" % s["step"] for s in steps]
        assert sorted(os.listdir(out)) == ["%d.f32" % k for k in sorted(want)]
        for k, ref in want.items():
            got = torch.from_numpy(np.fromfile(out / ("%d.f32" % k), dtype="<f4").reshape(-1, cfg["vocab"]).copy())
            assert got.shape == ref.shape and err(got, ref) < tol, (dtype, k)
    p = subprocess.run([sys.executable, os.path.join(root, "run.py"), "-m", ckpt, "--dtype", "float32", "--input-tokens", "9", "--max-new-tokens", "5",
                        "--batch-size", "2", "--num-iter", "2", "--num-warmup", "1"], text=True, capture_output=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "Inference latency:" in p.stdout and "Throughput:" in p.stdout and "[5, 5]" in p.stdout
