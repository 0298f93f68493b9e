"""GPU checks of the Davasun path against the plain float64 oracle (tests/davasun_oracle.py): every kernel alone, then the
model through the step engine -- whole prompts, token-by-token decoding, portions down to two tokens, unequal requests in
one step, slots that are freed and reused, far keys and the edges of the kernels' own tiles (32 cached rows per attention
stage, 8 tokens per recurrence stage), long decoding, greedy generation through generate()."""
import json
import math
import os

import pytest
import torch

import lia_b200  # noqa: F401
from lia_b200 import ops, registry
from lia_b200.checkpoint import write_safetensors
from lia_b200.engine import Engine
from lia_b200.modeling_davasun import DavasunConfig, DavasunForCausalLM
from lia_b200.seq_layers import Linear

import davasun_oracle as O
from davasun_cases import CASES, config, dense, latent, mlstm

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


# ------------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("W,scalar", [(44, True), (256, False), (1000, True)])
def test_embed_and_norm_kernels(W, scalar):
    g = gen(0)
    table = torch.randn(37, W, generator=g).to(BF16)
    ids = torch.randint(0, 37, (9,), generator=g)
    w0 = torch.randn(1 if scalar else W, generator=g)
    x = torch.empty(9, W, dtype=F32, device=DEV)
    ops.embed_rmsnorm(ids.to(DEV), table.to(DEV), w0.to(DEV), x, 1e-5)
    want = O.rms_norm(table.double()[ids], 1e-5) * w0.double()
    assert rel(x, want) < 1e-6
    y = torch.randn(9, W, generator=g)
    w1, w2 = torch.randn(1 if scalar else W, generator=g), torch.randn(1 if scalar else W, generator=g)
    for ydt, hdt, tol in ((F32, F32, 1e-6), (BF16, BF16, 6e-3)):
        x = want.float().to(DEV)
        yy = y.to(ydt)
        h = torch.empty(9, W, dtype=hdt, device=DEV)
        ops.rms_add_norm(x, yy.to(DEV), w1.to(DEV), w2.to(DEV), h, 1e-5)
        x_want = want.float().double() + O.rms_norm(yy.double(), 1e-5) * w1.double()
        assert rel(x, x_want) < 1e-6                              # the residual sum is fp32 whatever the activations are
        assert rel(h, O.rms_norm(x_want, 1e-5) * w2.double()) < tol
    rows = i32([8, 0, 3])
    hn = torch.empty(3, W, dtype=F32, device=DEV)
    ops.rms_gather(x, rows, w2.to(DEV), hn, 1e-5)
    assert rel(hn, O.rms_norm(x.double().cpu()[[8, 0, 3]], 1e-5) * w2.double()) < 1e-6


@pytest.mark.parametrize("M,N,K", [(5, 6, 44), (70, 2, 256), (3, 19, 33)])
def test_linear_small_gate_modes(M, N, K):
    g = gen(1)
    a, w, b = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) * 0.3, torch.randn(N, generator=g)
    out = torch.empty(M, N, dtype=F32, device=DEV)
    z = a.double() @ w.double().T + b.double()
    ops.linear_small(a.to(DEV), w.to(DEV), b.to(DEV), out, ops.GATE_NONE)
    assert rel(out, z) < 1e-5
    ops.linear_small(a.to(DEV), w.to(DEV), None, out, ops.GATE_SIGMOID)
    assert rel(out, torch.sigmoid(z - b.double())) < 1e-5
    if N % 2 == 0:
        cap = 3.0
        ops.linear_small(a.to(DEV), w.to(DEV), b.to(DEV), out, ops.GATE_LOG_INPUT_FORGET, cap)
        c = cap * torch.tanh(z / cap)
        want = torch.cat([c[:, :N // 2], torch.nn.functional.logsigmoid(c[:, N // 2:])], 1)
        assert rel(out, want) < 1e-5
    ab, wb = a.to(BF16), w.to(BF16)
    ops.linear_small(ab.to(DEV), wb.to(DEV), b.to(DEV), out, ops.GATE_NONE)
    assert rel(out, ab.double() @ wb.double().T + b.double()) < 1e-5       # bf16 inputs, fp32 products and sums


@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (65, 130, 33), (200, 64, 256)])
def test_linear_plain_and_tensor_core_linear(M, N, K):
    g = gen(2)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = torch.empty(M, N, dtype=F32, device=DEV)
    ops.linear_plain(a.to(DEV), w.to(DEV), out, scale=0.5)
    assert rel(out, 0.5 * a.double() @ w.double().T) < 1e-6
    # batched with strides: per head h, out[:, h] = a[:, h] @ w[h].T on slices of wider buffers
    H, k, n = 3, 5, 4
    A, Wb = torch.randn(M, H * (k + 2), generator=g), torch.randn(H, n, k, generator=g)
    C = torch.zeros(M, H * (n + 1), dtype=F32, device=DEV)
    ops.linear_plain(A.to(DEV), Wb.to(DEV), C, batch=H, a_batch_stride=k + 2, w_batch_stride=n * k, out_batch_stride=n + 1, n=n, k=k)
    want = torch.einsum("mhk,hnk->mhn", A.view(M, H, k + 2)[..., :k].double(), Wb.double())
    assert rel(C.view(M, H, n + 1)[..., :n], want) < 1e-6
    assert float(C.view(M, H, n + 1)[..., n].abs().max()) == 0.0


@pytest.mark.parametrize("M,K,sizes", [(3, 64, (24, 40, 6)), (150, 72, (40,)), (600, 256, (192, 80)), (130, 40, (30, 9))])
def test_stacked_linear_matches_plain(M, K, sizes):
    """The tensor-core GEMM (bf16, where the shape allows) against fp32 products of the same bf16 numbers."""
    g = gen(3)
    ws = [torch.randn(n, K, generator=g).to(BF16) for n in sizes]
    x = torch.randn(M, K, generator=g).to(BF16)
    lin = Linear(ws, BF16, DEV)
    y = lin(x.to(DEV))
    for i, w in enumerate(ws):
        assert lin.offsets[i] % 8 == 0
        assert rel(lin.part(y, i), x.double() @ w.double().T) < 6e-3
    lin32 = Linear([w.float() for w in ws], F32, DEV)
    y = lin32(x.float().to(DEV))
    for i, w in enumerate(ws):
        assert rel(lin32.part(y, i), x.double() @ w.double().T) < 1e-6


def test_clamped_glu_and_argmax():
    g = gen(4)
    F_, M = 37, 6
    gu = torch.randn(M, 40 + F_, generator=g) * 3
    out = torch.empty(M, F_, dtype=F32, device=DEV)
    ops.clamped_glu(gu.to(DEV), 40, F_, out, 1.5, 1.702)
    gg, uu = gu[:, :F_].double().clamp(max=1.5), gu[:, 40:].double().clamp(-1.5, 1.5)
    assert rel(out, gg * torch.sigmoid(1.702 * gg) * (uu + 1)) < 1e-6
    lg = torch.randn(5, 1001, generator=g)
    lg[2, 7] = lg[2, 900] = 50.0                                  # a tie: the lower index wins
    lg[3, 5] = 60.0
    pick = ops.argmax_f32(lg.to(DEV), suppress_id=5).cpu()
    want = lg.clone()
    want[:, 5] = -math.inf
    assert pick.tolist() == want.argmax(-1).tolist() and pick[2] == 7


def _scan(q, k, v, ig, fg, lens, H, d, e, dtype, state=None, slots=None):
    """Run the recurrence kernel over portions of `lens` rows (one slot each)."""
    M = q.shape[0]
    n_slots = len(lens)
    slots = slots or list(range(n_slots))
    if state is None:
        state = (torch.zeros(max(slots) + 1, H, e, d, device=DEV), torch.zeros(max(slots) + 1, H, d, device=DEV),
                 torch.zeros(max(slots) + 1, H, device=DEV))
    buf = torch.cat([q.reshape(M, H * d), k.reshape(M, H * d), v.reshape(M, H * e)], 1).to(dtype).to(DEV)
    segs, row = [], 0
    for s, n in zip(slots, lens):
        segs.append((s, 0, row, n))
        row += n
    o = torch.empty(M, H * e, dtype=F32, device=DEV)
    ops.mlstm_scan(buf[:, :H * d], buf[:, H * d:2 * H * d], buf[:, 2 * H * d:], torch.cat([ig, fg], 1).float().to(DEV), *state, i32(segs),
                   H, d, e, d ** -0.5, 1e-6, o)
    return o, state


@pytest.mark.parametrize("H,d,e,T", [(1, 4, 3, 1), (2, 32, 64, 23), (3, 10, 70, 17), (2, 80, 136, 9), (1, 36, 20, 40), (1, 300, 8, 5)])
def test_mlstm_scan_against_the_token_loop(H, d, e, T):
    g = gen(5)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, H, d, generator=g), torch.randn(T, H, e, generator=g)
    ig, fg = torch.randn(T, H, generator=g) * 3, -torch.rand(T, H, generator=g) * 2
    st = {}
    want = O.mlstm_recurrence(q.double() * d ** -0.5, k.double(), v.double(), ig.double(), fg.double(), st)
    o, state = _scan(q, k, v, ig, fg, [T], H, d, e, F32)
    assert rel(o.view(T, H, e), want) < 2e-5
    assert rel(state[0][0].transpose(1, 2), st["S"]) < 2e-5 and rel(state[1][0], st["n"]) < 2e-5 and rel(state[2][0], st["m"]) < 1e-6
    # the same tokens as portions through carried state (cuts inside and at the edges of the 8-token stage), and one by one
    for cuts in ([1] * T, [min(7, T)] + [1] * (T - min(7, T)), [min(8, T), T - min(8, T)], [min(9, T), T - min(9, T)]):
        state2, outs, at = None, [], 0
        for n in [c for c in cuts if c > 0]:
            o2, state2 = _scan(q[at:at + n], k[at:at + n], v[at:at + n], ig[at:at + n], fg[at:at + n], [n], H, d, e, F32, state2)
            outs.append(o2)
            at += n
        assert torch.equal(torch.cat(outs), o)                    # bit-identical however the tokens are cut
        assert torch.equal(state2[0], state[0]) and torch.equal(state2[2], state[2])


@pytest.mark.parametrize("d,e", [(24, 40), (12, 21), (64, 16)])          # 128-bit stage loads; element-wise ones; one column block
def test_mlstm_scan_batches_of_unequal_portions_and_bf16_inputs(d, e):
    g = gen(6)
    H, lens = 2, [5, 1, 19, 8]
    T = sum(lens)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, H, d, generator=g), torch.randn(T, H, e, generator=g)
    ig, fg = torch.randn(T, H, generator=g), -torch.rand(T, H, generator=g)
    o, _ = _scan(q, k, v, ig, fg, lens, H, d, e, BF16, slots=[3, 0, 2, 1])
    at = 0
    for n in lens:
        sl = slice(at, at + n)
        qb, kb, vb = (t[sl].to(BF16).double() for t in (q, k, v))
        want = O.mlstm_recurrence(qb * d ** -0.5, kb, vb, ig[sl].double(), fg[sl].double(), {})
        assert rel(o[sl].view(n, H, e), want) < 2e-5              # bf16 inputs, fp32 recurrence
        alone, _ = _scan(q[sl], k[sl], v[sl], ig[sl], fg[sl], [n], H, d, e, BF16)
        assert torch.equal(alone, o[sl])
        at += n


def test_mlstm_gates_saturate_like_the_equations():
    """Strong gates: the forget gate's log stays below 0, the stabiliser follows the input gate, nothing overflows."""
    H, d, e, T = 1, 8, 8, 30
    g = gen(7)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, H, d, generator=g), torch.randn(T, H, e, generator=g)
    ig = torch.linspace(-15, 15, T).view(T, 1)
    fg = torch.nn.functional.logsigmoid(torch.linspace(15, -15, T)).view(T, 1)
    want = O.mlstm_recurrence(q.double() * d ** -0.5, k.double(), v.double(), ig.double(), fg.double(), {})
    o, _ = _scan(q, k, v, ig, fg, [T], H, d, e, F32)
    assert torch.isfinite(o).all() and rel(o.view(T, H, e), want) < 2e-4


def test_headnorm_gate():
    g = gen(8)
    M, H, e = 7, 3, 70
    o, w, gate = torch.randn(M, H * e, generator=g), torch.randn(H * e, generator=g), torch.randn(M, H * e + 8, generator=g)
    out = torch.empty(M, H * e, dtype=F32, device=DEV)
    ops.headnorm_gate(o.to(DEV), w.to(DEV), gate.to(DEV)[:, 8:], out, H, e, 1e-5)
    want = O.rms_norm(o.double().view(M, H, e), 1e-5).reshape(M, H * e) * w.double() * torch.sigmoid(gate[:, 8:].double())
    assert rel(out, want) < 1e-6


def _latent_reference(qa, cache_rows, pos, H, rank, scale, gate=None):
    """softmax over rows [0, pos] of (qa . row) * scale, weighted sum of the rows' first `rank` numbers."""
    D = cache_rows.shape[1]
    s = torch.einsum("hd,sd->hs", qa.view(H, D).double(), cache_rows[:pos + 1].double()) * scale
    out = torch.softmax(s, -1) @ cache_rows[:pos + 1, :rank].double()
    return out if gate is None else out * gate.double()[:, None]


@pytest.mark.parametrize("H,rank,rot,dtype", [(1, 20, 6, F32), (4, 64, 16, F32), (9, 264, 4, F32), (12, 48, 8, BF16), (3, 520, 24, F32)])
def test_latent_attn_kernel_edges_and_far_keys(H, rank, rot, dtype):
    g = gen(9)
    D, cap = rank + rot, 200
    cache = torch.randn(2, cap, D, generator=g).to(dtype)
    positions = [0, 1, 30, 31, 32, 33, 63, 64, 65, 127, 199]          # around the 32-row stages, the first rows, the last row
    meta = [(1, p) for p in positions]
    qa = torch.randn(len(positions), H * D, generator=g)
    gate = torch.rand(len(positions), H, generator=g)
    out = torch.empty(len(positions), H * rank, dtype=F32, device=DEV)
    for max_ctx in (0, 200):                          # 200: the keys of every row are split over 3 blocks and combined
        assert ops.latent_attn_splits(len(positions), H, max_ctx, 148) == (3 if max_ctx else 1)
        out.zero_()
        ops.latent_attn(qa.to(DEV), cache.to(DEV), i32(meta), gate.to(DEV), out, H, rank, rot, 0.3, max_ctx=max_ctx)
        for r, p in enumerate(positions):
            want = _latent_reference(qa[r], cache[1].float(), p, H, rank, 0.3, gate[r])
            assert rel(out[r].view(H, rank), want) < 2e-5, (r, p, max_ctx)
    # one far key made to stand out: head 0's query is aligned with row 3 of a 190-row history, so the output is that row;
    # the row just outside the causal range (pos + 1) is made even stronger and must not be seen
    p = 189
    c1 = cache[1].float()
    far = c1[3] / c1[3].norm()
    c1[3] = far * 6.0
    c1[p + 1] = far * 30.0
    q2 = torch.randn(1, H * D, generator=g) * 0.1
    q2[0, :D] = far * 40.0
    out2 = torch.empty(1, H * rank, dtype=F32, device=DEV)
    cache2 = cache.clone().float()
    cache2[1] = c1
    ops.latent_attn(q2.to(DEV), cache2.to(DEV), i32([(1, p)]), None, out2, H, rank, rot, 1.0, max_ctx=p + 1)
    want = _latent_reference(q2[0], c1, p, H, rank, 1.0)
    assert rel(out2.view(H, rank), want) < 2e-5
    assert rel(out2.view(H, rank)[0], c1[3, :rank]) < 1e-3            # the far key took all the weight


def test_latent_prep_norm_rotation_and_cache_rows():
    g = gen(10)
    H, dim, rot, rank, dims, base, M = 3, 10, 8, 20, 6, 300.0, 5
    D = rank + rot
    q = torch.randn(M, H * (dim + rot) + 8, generator=g)
    dkv = torch.randn(M, D, generator=g)
    cw = torch.randn(rank, generator=g)
    meta = [(0, 0), (0, 1), (1, 77), (1, 78), (0, 2)]
    cache = torch.zeros(2, 100, D, device=DEV)
    qa = torch.zeros(M, H * D, device=DEV)
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F32, device=DEV)
    ops.latent_prep(q.to(DEV)[:, 8:], dkv.to(DEV), cw.to(DEV), inv, i32(meta), cache, qa, H, dim, rot, dims, rank, 1e-5)
    pos = torch.tensor([p for _, p in meta])
    lat = O.rms_norm(dkv[:, :rank].double(), 1e-5) * cw.double()
    kr = O.rotate_half(dkv[:, rank:].double(), pos, dims, base)       # dims < rot: the last channels pass unchanged
    qr = O.rotate_half(q[:, 8:].double().view(M, H, dim + rot)[..., dim:], pos, dims, base)
    for r, (s, p) in enumerate(meta):
        assert rel(cache[s, p, :rank], lat[r]) < 1e-6 and rel(cache[s, p, rank:], kr[r]) < 2e-5
        assert rel(qa[r].view(H, D)[:, rank:], qr[r]) < 2e-5
    assert float(cache[0, 3:].abs().max()) == 0.0 and float(qa.view(M, H, D)[..., :rank].abs().max()) == 0.0


# ------------------------------------------------------------------------------------------------ the model
def build(name, dtype, seed=11, std_scale=1.0):
    cfg = CASES[name] if isinstance(name, str) else name
    c = DavasunConfig.from_dict(cfg)
    w = O.random_weights(c.tensor_shapes(), seed, std_scale)
    m = DavasunForCausalLM(c, DEV, dtype).load_weights(lambda n: w[n])
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
    # bf16 rounding of the projections through up to 8 narrow layer runs: a few percent of the logits' rms, where a wrong
    # slice, state or constant shows as an error of order 1
    want = oracle_logits(cfg, w, toks)
    assert err(got, want) < 0.2 and err(got, want, "mean") < 0.06
    m32 = DavasunForCausalLM(m.config, DEV, F32).load_weights(lambda n: w[n])
    got32 = Engine(m32, 80, 1).step([{"id": 0, "tokens": toks, "want": list(range(70))}])
    assert err(got, got32.cpu()) < 0.2


@pytest.mark.parametrize("name,dtype", [("even", F32), ("odd", F32), ("wide", F32), ("even", BF16)])
def test_portions_and_decoding_equal_the_whole_prompt(name, dtype):
    cfg, w, m = build(name, dtype)
    n = 75
    toks = toks_for(cfg, n, 3)
    eng = Engine(m, 100, 2)
    whole = eng.step([{"id": "w", "tokens": toks, "want": list(range(n))}], end=["w"])
    tol = 1e-4 if dtype == F32 else 0.2        # bf16: GEMM tiles differ with the row count, so portions differ by rounding
    schedules = {"token by token": [1] * n, "twos": [2] * 37 + [1],
                 "ragged": [31, 1, 1, 2, 30, 3, 7], "stage edges": [32, 32, 8, 1, 1, 1], "prompt then decode": [n - 33] + [1] * 33}
    for label, cuts in schedules.items():
        assert sum(cuts) == n
        outs, at = [], 0
        for c in cuts:
            outs.append(eng.step([{"id": label, "tokens": toks[at:at + c], "want": list(range(c))}]))
            at += c
        eng.step([], end=[label])
        assert err(torch.cat(outs), whole.double().cpu()) < tol, label
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


def test_attention_reaches_far_back_through_the_model():
    """A model of one attention layer whose scores are sharp (large scale): the logits at the end depend on WHICH early
    token carried the matching key, hundreds of positions back; moving that token by one place changes them."""
    cfg = config([latent(2, 8, 8, 8, 16, base=10000.0, scale=6.0)], vocab=40, width=32, eps=1e-5)
    _, w, m = build(cfg, F32, seed=12, std_scale=2.0)
    n = 300
    toks = toks_for(cfg, n, 10)
    eng = Engine(m, 320, 1)
    for variant in (toks, toks[:5] + [toks[5] ^ 1] + toks[6:]):
        got = eng.step([{"id": 0, "tokens": variant[:n - 40], "want": []}])
        assert got is None
        outs = [eng.step([{"id": 0, "tokens": [t], "want": [0]}]) for t in variant[n - 40:]]
        eng.step([], end=[0])
        assert err(torch.cat(outs), oracle_logits(cfg, w, variant)[n - 40:]) < 2e-4


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
    history whose lengths cross the 64- and 128-key borders at which the attention changes its split of the keys, steps
    that want no logits, a request that ends and another that takes over its slot while the graphs stay in use."""
    cfg, w, m = build("even", dtype)
    a, b, c = toks_for(cfg, 179, 40), toks_for(cfg, 110, 41), toks_for(cfg, 30, 42)

    def play(graphs):
        eng = Engine(m, 180, 2, graphs=graphs)
        outs = [eng.step([{"id": "a", "tokens": a[:50], "want": [49]}, {"id": "b", "tokens": b[:3], "want": [2]}])]
        for i in range(100):
            want = [] if i % 7 == 3 else [0]
            o = eng.step([{"id": "a", "tokens": [a[50 + i]], "want": want}, {"id": "b", "tokens": [b[3 + i]], "want": want}])
            assert (o is None) == (not want)
            if o is not None:
                outs.append(o)
        eng.step([], end=["b"])
        outs.append(eng.step([{"id": "c", "tokens": c[:1], "want": [0]}]))           # b's slot, state zeroed; alone in its pass
        for i in range(1, 30):
            outs.append(eng.step([{"id": "c", "tokens": [c[i]], "want": [0]}, {"id": "a", "tokens": [a[149 + i]], "want": [0]}]))
        return torch.cat(outs), eng

    eager, _ = play(False)
    graphed, eng = play(True)
    assert sum(g.graph is not None for g in eng._step_graphs.values()) >= 4           # several shapes were captured and replayed
    assert torch.equal(eager, graphed)
    if dtype == F32:
        la, lc = oracle_logits(cfg, w, a), oracle_logits(cfg, w, c)
        assert err(graphed[-2:-1], lc[29:30]) < 2e-4 and err(graphed[-1:], la[178:179]) < 2e-4      # the last pass: c, then a


def test_first_tokens_and_single_token_prompts():
    cfg, w, m = build("wide", F32)
    eng = Engine(m, 8, 3)
    for seed in (20, 21, 22):
        t = toks_for(cfg, 1, seed)
        got = eng.step([{"id": seed, "tokens": t, "want": [0]}])
        assert err(got, oracle_logits(cfg, w, t)) < 2e-4
    t = toks_for(cfg, 3, 23)
    eng.step([], end=[20, 21, 22])
    got = torch.cat([eng.step([{"id": "s", "tokens": [x], "want": [0]}]) for x in t])
    assert err(got, oracle_logits(cfg, w, t)) < 2e-4


def test_greedy_generation_through_generate_and_from_pretrained(tmp_path):
    cfg = CASES["even"]
    c = DavasunConfig.from_dict(cfg)
    w = O.random_weights(c.tensor_shapes(), 14)
    d = tmp_path / "ckpt"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: v.to(BF16) for k, v in w.items()})
    m = registry.load_model(str(d), device=DEV, dtype=F32)
    assert isinstance(m, DavasunForCausalLM)
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


def _write_checkpoint(tmp_path, cfg, seed):
    w = O.random_weights(DavasunConfig.from_dict(cfg).tensor_shapes(), seed)
    d = tmp_path / "ckpt"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(d / "model.safetensors"), {k: v.to(BF16) for k, v in w.items()})
    return str(d), w


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
