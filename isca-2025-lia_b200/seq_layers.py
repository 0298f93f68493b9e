"""Sequence mixers and feed-forwards that run on a 32-bit residual stream, each with its constants as parameters so that
any model design can assemble them: a matrix-memory recurrent mixer (mLSTM), attention over a latent key/value cache with
a partly rotated query/key and an output gate, linear attention with a fixed decay per head, the gated delta rule behind a
short convolution, sliding-window attention with grouped key/value heads, and the feed-forwards -- clamped gated, plain
gated with any activation, and a routed mixture of experts with a shared expert.  Each object owns its (fused) weights,
registers its per-sequence state with a ``seq_state.SlotState`` and runs one step over a batch of portions
(``StepBatch``) through the kernels of ``ops``.

Projections go through ``Linear``: the tensor-core GEMM of the OPT path (csrc/gemm_sm100.cu) for bf16 activations, the
plain CUDA-core kernel for fp32 activations and for shapes the tensor-core kernel does not take.
"""
import os

import torch

from . import ops

BF16, F32 = torch.bfloat16, torch.float32


def _pad8(n):
    return (n + 7) // 8 * 8


class StepBatch:
    """The token rows of one step: ``segs`` int32 [n, 4] = (slot, first position, first row, rows) per portion and
    ``meta`` int32 [rows, 2] = (slot, position) per row, both on the device."""

    def __init__(self, rows, segs, meta, max_ctx=0):
        self.rows, self.segs, self.meta = rows, segs, meta
        self.max_ctx = max_ctx              # longest history (tokens cached after this step) among the step's sequences


class Linear:
    """y = x @ W.T for one or several weight matrices stacked by rows (one launch, outputs side by side; each block's
    first column is a multiple of 8 so that every slice stays 16-byte aligned in bf16)."""

    _gemm_ws = {}

    def __init__(self, weights, dtype, device):
        ws = [w.to(device=device, dtype=dtype) for w in weights]
        self.K = ws[0].shape[1]
        self.offsets, n = [], 0
        for w in ws:
            self.offsets.append(_pad8(n))
            n = self.offsets[-1] + w.shape[0]
        self.sizes = [w.shape[0] for w in ws]
        self.N = n
        self.weight = torch.zeros(n, self.K, dtype=dtype, device=device)
        for o, w in zip(self.offsets, ws):
            self.weight[o:o + w.shape[0]] = w
        self.dtype = dtype
        self.tensor_core = (dtype == BF16 and self.K % 8 == 0 and self.N % 8 == 0 and os.environ.get("LIA_PLAIN_LINEAR", "0") == "0")

    def _workspace(self, M, device):
        key = (device, M <= 128)
        need = ops.GemmWorkspace.bytes_for([(M, self.N, self.K)])
        ws = Linear._gemm_ws.get(key)
        if ws is None or ws.buf.numel() < need:
            ws = Linear._gemm_ws[key] = ops.GemmWorkspace(need, device)
        return ws

    def __call__(self, x, out=None):
        M = x.shape[0]
        if out is None:
            out = torch.empty(M, self.N, dtype=self.dtype, device=x.device)
        if self.tensor_core and x.is_contiguous() and x.data_ptr() % 16 == 0:
            ops.gemm(x, self.weight, None, out=out, workspace=self._workspace(M, x.device))
        else:
            ops.linear_plain(x, self.weight, out)
        return out

    def part(self, y, i):
        return y[:, self.offsets[i]:self.offsets[i] + self.sizes[i]]


class MLSTMMixer:
    """Matrix-memory recurrent mixer.  q = Wq h * dim^-1/2, k = Wk h, v = Wv h; per head a log input gate
    cap*tanh((Wi h + bi)/cap) and a log forget gate logsigmoid(cap*tanh((Wf h + bf)/cap)); the stabilised recurrence of
    csrc/mlstm.cu; each head's output RMS-normed, times a per-channel weight, times sigmoid(Wg h), then Wo."""

    def __init__(self, w, heads, dim, vdim, gate_cap, norm_eps, dtype, device, den_eps=1e-6):
        self.H, self.dim, self.vdim, self.cap, self.eps, self.den_eps = heads, dim, vdim, float(gate_cap), float(norm_eps), den_eps
        self.dtype = dtype
        self.proj = Linear([w["q"], w["k"], w["v"], w["g"]], dtype, device)
        self.w_gates = torch.cat([w["i"], w["f"]], 0).to(device=device, dtype=dtype).contiguous()
        self.b_gates = torch.cat([w["i.b"], w["f.b"]], 0).to(device=device, dtype=F32).contiguous()
        self.norm_w = w["norm"].to(device=device, dtype=F32).contiguous()
        self.out = Linear([w["o"]], dtype, device)
        self.q_scale = float(dim) ** -0.5

    def new_state(self, slots):
        return (slots.add_recurrent((self.H, self.vdim, self.dim)), slots.add_recurrent((self.H, self.dim)),
                slots.add_recurrent((self.H,)))

    def __call__(self, h, batch, state):
        S, n, m = state
        M, H = h.shape[0], self.H
        y = self.proj(h)
        q, k, v, g = (self.proj.part(y, i) for i in range(4))
        gates = torch.empty(M, 2 * H, dtype=F32, device=h.device)
        ops.linear_small(h, self.w_gates, self.b_gates, gates, ops.GATE_LOG_INPUT_FORGET, self.cap)
        o = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        ops.mlstm_scan(q, k, v, gates, S, n, m, batch.segs, H, self.dim, self.vdim, self.q_scale, self.den_eps, o)
        on = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.headnorm_gate(o, self.norm_w, g, on, H, self.vdim, self.eps)
        return self.out(on)


def rotary_inv_freq(dims, base, device):
    """f_i = base^(-2i/dims), i < dims/2, rounded once to fp32."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return (float(base) ** (-2.0 * i / dims)).to(F32).to(device)


class LatentAttentionMixer:
    """Attention over a latent cache: per token one normalised latent (kv_rank) and one rotated key part (rot_dim) shared by
    the heads are cached; head h's unrotated key and value are Wuk_h c and Wuv_h c.  Queries are laid out per head as
    [dim unrotated | rot_dim rotated]; rotary "rotate half" over the first ``rot_dims`` channels of the rotated part;
    causal softmax with ``scale``; head outputs times sigmoid(Wg h)_h; then Wo.  The kernels work in the latent space
    (csrc/latent_attn.cu), so Wuk is applied to the query and Wuv to the attention's output."""

    def __init__(self, w, heads, dim, rot_dim, vdim, kv_rank, rot_dims, rot_base, scale, norm_eps, dtype, device):
        self.H, self.dim, self.rot, self.vdim, self.rank = heads, dim, rot_dim, vdim, kv_rank
        self.rot_dims, self.scale, self.eps, self.dtype = rot_dims, float(scale), float(norm_eps), dtype
        self.proj = Linear([w["q"], w["dkv"]], dtype, device)
        self.w_gate = w["g"].to(device=device, dtype=dtype).contiguous()
        self.c_norm_w = w["dkv.norm"].to(device=device, dtype=F32).contiguous()
        # Wuk [H*dim, rank] -> per head [rank, dim]: the projection that carries a query into the latent space
        self.w_uk_t = w["uk"].to(device=device, dtype=dtype).view(heads, dim, kv_rank).transpose(1, 2).contiguous()
        self.w_uv = w["uv"].to(device=device, dtype=dtype).contiguous()            # [H*vdim, rank]
        self.out = Linear([w["o"]], dtype, device)
        self.inv_freq = rotary_inv_freq(rot_dims, rot_base, device)

    def new_state(self, slots):
        return (slots.add_rows(self.rank + self.rot, self.dtype),)

    def __call__(self, h, batch, state):
        (cache,) = state
        M, H, D = h.shape[0], self.H, self.rank + self.rot
        y = self.proj(h)
        q, dkv = self.proj.part(y, 0), self.proj.part(y, 1)
        gate = torch.empty(M, H, dtype=F32, device=h.device)
        ops.linear_small(h, self.w_gate, None, gate, ops.GATE_SIGMOID)
        qa = torch.empty(M, H * D, dtype=F32, device=h.device)
        ops.latent_prep(q, dkv, self.c_norm_w, self.inv_freq, batch.meta, cache, qa, H, self.dim, self.rot, self.rot_dims, self.rank,
                        self.eps)
        # q~[m, h, :rank] = Wuk_h^T q[m, h, :dim]
        ops.linear_plain(q, self.w_uk_t, qa, batch=H, a_batch_stride=self.dim + self.rot, w_batch_stride=self.rank * self.dim,
                         out_batch_stride=D, n=self.rank, k=self.dim)
        lat = torch.empty(M, H * self.rank, dtype=F32, device=h.device)
        ops.latent_attn(qa, cache, batch.meta, gate, lat, H, self.rank, self.rot, self.scale, batch.max_ctx)
        o = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.linear_plain(lat, self.w_uv, o, batch=H, a_batch_stride=self.rank, w_batch_stride=self.vdim * self.rank,
                         out_batch_stride=self.vdim, n=self.vdim, k=self.rank)
        return self.out(o)


class ClampedGLU:
    """Dense gated feed-forward: g = min(Wgate h, limit), u = clamp(Wup h, -limit, limit),
    y = g * sigmoid(alpha g) * (u + 1), output Wdown y."""

    def __init__(self, w, ff, limit, dtype, device, alpha=1.702):
        self.ff, self.limit, self.alpha, self.dtype = ff, float(limit), float(alpha), dtype
        self.gate_up = Linear([w["gate"], w["up"]], dtype, device)
        self.down = Linear([w["down"]], dtype, device)

    def __call__(self, h):
        gu = self.gate_up(h)
        y = torch.empty(h.shape[0], self.ff, dtype=self.dtype, device=h.device)
        ops.clamped_glu(gu, self.gate_up.offsets[1], self.ff, y, self.limit, self.alpha)
        return self.down(y)


class DecayLinearAttentionMixer:
    """Linear attention with a fixed decay per head ("lightning" attention): q, k, v = act(Wq h), act(Wk h), act(Wv h);
    S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (csrc/linear_scan.cu), act = SiLU; the concatenated heads RMS-normed together with a per-channel weight, times sigmoid(Wg h), then Wo."""

    def __init__(self, w, heads, dim, vdim, decay, norm_eps, dtype, device):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        self.H, self.dim, self.vdim, self.eps, self.dtype = heads, dim, vdim, float(norm_eps), dtype
        self.proj = Linear([w["q"], w["k"], w["v"], w["g"]], dtype, device)
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float64).to(device=device, dtype=F32)
        self.norm_w = w["norm"].to(device=device, dtype=F32).contiguous()
        self.out = Linear([w["o"]], dtype, device)

    def new_state(self, slots):
        return (slots.add_recurrent((self.H, self.vdim, self.dim)),)

    def __call__(self, h, batch, state):
        (S,) = state
        M, H = h.shape[0], self.H
        y = self.proj(h)
        g = self.proj.part(y, 3)
        # SiLU of q | k | v in one pass over their columns (every block of the scan that shares a head would repeat it otherwise)
        F_, offs = self.proj.offsets[3], self.proj.offsets
        act = torch.empty(M, F_, dtype=self.dtype, device=h.device)
        ops.gated_act(y, F_, act, ops.ACT_SILU)
        q, k, v = act[:, offs[0]:offs[0] + H * self.dim], act[:, offs[1]:offs[1] + H * self.dim], act[:, offs[2]:offs[2] + H * self.vdim]
        o = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        ops.linear_scan(q, k, v, S, batch.segs, H, H, self.dim, self.vdim, o, decay=self.decay)
        on = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.headnorm_gate(o, self.norm_w, g, on, 1, H * self.vdim, self.eps)       # one norm over all heads
        return self.out(on)


class DeltaRuleMixer:
    """Gated delta rule.  q, k (kv_heads x dim) and v (heads x vdim) pass a short causal convolution per channel and SiLU; q, k
    become unit vectors per head (q times dim^-1/2); per head beta = sigmoid(Wb h) and g = exp(-exp(A_log) softplus(Wa h + dt_bias));
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; each head's o RMS-normed with a weight shared by the heads, times
    silu(Wg h); then Wo.  Per-sequence state: S and the last taps - 1 inputs of the convolution."""

    def __init__(self, w, heads, kv_heads, dim, vdim, taps, norm_eps, dtype, device, unit_eps=1e-6):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads do not divide into {kv_heads} query/key heads")
        self.H, self.G, self.dim, self.vdim, self.taps = heads, kv_heads, dim, vdim, int(taps)
        self.eps, self.unit_eps, self.dtype = float(norm_eps), float(unit_eps), dtype
        self.proj = Linear([w["q"], w["k"], w["v"], w["g"]], dtype, device)
        self.w_gates = torch.cat([w["b"], w["a"]], 0).to(device=device, dtype=dtype).contiguous()        # -> beta | decay inputs
        self.w_conv = torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]], 0).to(device=device, dtype=F32).contiguous()
        self.a_log = w["A_log"].to(device=device, dtype=F32).contiguous()
        self.dt_bias = w["dt_bias"].to(device=device, dtype=F32).contiguous()
        self.norm_w = w["norm"].to(device=device, dtype=F32).repeat(heads).contiguous()
        self.out = Linear([w["o"]], dtype, device)
        self.channels = 2 * kv_heads * dim + heads * vdim

    def new_state(self, slots):
        return (slots.add_recurrent((self.H, self.vdim, self.dim)), slots.add_recurrent((max(self.taps - 1, 1), self.channels)))

    def __call__(self, h, batch, state):
        S, conv = state
        M, H, G = h.shape[0], self.H, self.G
        y = self.proj(h)
        gates = torch.empty(M, 2 * H, dtype=F32, device=h.device)
        ops.linear_small(h, self.w_gates, None, gates, ops.GATE_NONE)
        qk = torch.empty(M, 2 * G * self.dim, dtype=F32, device=h.device)
        v = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        offs = self.proj.offsets[:3]
        ops.conv_prep(y, offs, self.w_conv, conv, batch.meta, gates, self.a_log, self.dt_bias, qk, v, G, H, self.dim, self.vdim, self.taps,
                      float(self.dim) ** -0.5, self.unit_eps)
        ops.conv_state_update(y, offs, G * self.dim, H * self.vdim, conv, batch.segs, self.taps)
        o = torch.empty(M, H * self.vdim, dtype=F32, device=h.device)
        ops.linear_scan(qk[:, :G * self.dim], qk[:, G * self.dim:], v, S, batch.segs, H, G, self.dim, self.vdim, o, gates=gates)
        on = torch.empty(M, H * self.vdim, dtype=self.dtype, device=h.device)
        ops.headnorm_gate(o, self.norm_w, self.proj.part(y, 3), on, H, self.vdim, self.eps, gate_silu=True)
        return self.out(on)


class WindowAttentionMixer:
    """Softmax attention over the last ``window`` positions, ``kv_heads`` key/value heads shared by groups of query heads, no
    positional rotation.  Values are divided by their per-head root mean square before they are cached; a score is
    (q . k) * scale * temp_h, then softcap * tanh(score / softcap) (csrc/window_attn.cu); output Wo on the concatenated heads."""

    def __init__(self, w, heads, kv_heads, dim, vdim, window, scale, softcap, norm_eps, dtype, device, norm_values=True):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads do not divide into {kv_heads} key/value heads")
        self.H, self.G, self.dim, self.vdim, self.window = heads, kv_heads, dim, vdim, int(window)
        self.scale, self.softcap, self.eps, self.dtype, self.norm_values = float(scale), float(softcap), float(norm_eps), dtype, norm_values
        self.proj = Linear([w["q"], w["k"], w["v"]], dtype, device)
        temp = w.get("temp")
        self.temp = (temp if temp is not None else torch.ones(heads)).to(device=device, dtype=F32).contiguous()
        self.out = Linear([w["o"]], dtype, device)

    def new_state(self, slots):
        return (slots.add_rows(self.G * self.dim, self.dtype), slots.add_rows(self.G * self.vdim, self.dtype))

    def __call__(self, h, batch, state):
        kc, vc = state
        M = h.shape[0]
        y = self.proj(h)
        q, k, v = (self.proj.part(y, i) for i in range(3))
        ops.kv_store(k, v, batch.meta, kc, vc, self.G, self.dim, self.vdim, self.eps, self.norm_values)
        o = torch.empty(M, self.H * self.vdim, dtype=self.dtype, device=h.device)
        ops.window_attn(q, kc, vc, batch.meta, self.temp, o, self.H, self.G, self.dim, self.vdim, self.window, self.scale, self.softcap,
                        nseg=batch.segs.shape[0], max_ctx=batch.max_ctx)
        return self.out(o)


class GatedMLP:
    """Dense gated feed-forward: Wdown (act(Wgate h) * (Wup h))."""

    def __init__(self, w, ff, act, dtype, device):
        self.ff, self.act, self.dtype = ff, act, dtype
        self.gate_up = Linear([w["gate"], w["up"]], dtype, device)
        self.down = Linear([w["down"]], dtype, device)

    def __call__(self, h):
        gu = self.gate_up(h)
        y = torch.empty(h.shape[0], self.ff, dtype=self.dtype, device=h.device)
        ops.gated_act(gu, self.ff, y, self.act, up_off=self.gate_up.offsets[1])
        return self.down(y)


class PlainMLP:
    """Wdown act(Wup h)."""

    def __init__(self, w, ff, act, dtype, device):
        self.ff, self.act, self.dtype = ff, act, dtype
        self.up = Linear([w["up"]], dtype, device)
        self.down = Linear([w["down"]], dtype, device)

    def __call__(self, h):
        u = self.up(h)
        y = torch.empty(h.shape[0], self.ff, dtype=self.dtype, device=h.device)
        ops.gated_act(u, self.ff, y, self.act)
        return self.down(y)


class MoEFeedForward:
    """Routed mixture of experts: router logits in fp32, softmax over all experts, the ``top`` largest scores renormalised
    (divided by their sum + 1e-20); every expert is Wdown act(Wup h); a shared expert (optional) runs for every token and is
    added.  ``experts_w``: list of {"up", "down"} per expert.  The (token, choice) pairs are grouped by expert on the device
    (no host round trip) and each projection runs as one grouped launch; a handful of pairs (decoding) take the form with one
    warp per output instead.  The result is fp32."""

    FEW_PAIRS = 48            # up to here: one warp per output, no plan
    TENSOR_CORE_PAIRS = 512   # from here (bf16, sizes that are multiples of 8): every expert's rows through the tensor-core GEMM

    def __init__(self, router_w, experts_w, top, ff, act, shared, dtype, device):
        self.E, self.top, self.ff, self.act, self.dtype = len(experts_w), int(top), ff, act, dtype
        if not 1 <= self.top <= self.E:
            raise ValueError(f"top = {top} of {self.E} experts")
        self.router = router_w.to(device=device, dtype=dtype).contiguous()
        self.w_up = torch.stack([e["up"] for e in experts_w]).to(device=device, dtype=dtype).contiguous()         # [E, ff, W]
        self.w_down = torch.stack([e["down"] for e in experts_w]).to(device=device, dtype=dtype).contiguous()     # [E, W, ff]
        self.shared = shared
        W = self.w_up.shape[2]
        self.tensor_core = dtype == BF16 and W % 8 == 0 and ff % 8 == 0 and os.environ.get("LIA_PLAIN_LINEAR", "0") == "0"

    def _workspace(self, rows, N, K, device):
        """One split-K workspace large enough for every row count among the experts' launches."""
        key = (device, "experts")
        need = ops.GemmWorkspace.bytes_for([(m, N, K) for m in set(rows)])
        ws = Linear._gemm_ws.get(key)
        if ws is None or ws.buf.numel() < need:
            ws = Linear._gemm_ws[key] = ops.GemmWorkspace(need, device)
        return ws

    def _experts_tensor_core(self, h, idx, wt, y):
        """Prompts: the pairs grouped by expert (tiles of 64 rows), the rows gathered into that order, then one tensor-core
        GEMM per expert and projection on its contiguous rows (launched back to back from the library).  The tile table comes to the host once per call (the only
        round trip; decode steps never take this path, so they stay capturable)."""
        M, W = h.shape
        E, top, ff, dev = self.E, self.top, self.ff, h.device
        pairs = M * top
        n_tiles, tm = ops.moe_tiles(pairs, E)
        perm = torch.empty(n_tiles * tm, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(n_tiles, dtype=torch.int32, device=dev)
        pos_of = torch.empty(pairs, dtype=torch.int32, device=dev)
        ops.moe_plan(idx, E, perm, tile_expert, pos_of)
        xs = torch.empty(n_tiles * tm, W, dtype=self.dtype, device=dev)
        ops.moe_gather(h, perm, xs, top)
        counts = torch.bincount(tile_expert.cpu().long() + 1, minlength=E + 1)[1:].tolist()          # tiles per expert
        used, rows = sum(counts) * tm, [n * tm for n in counts if n]
        up = torch.empty(used, ff, dtype=self.dtype, device=dev)
        ops.moe_expert_gemms(xs, self.w_up, up, counts, tm, self._workspace(rows, ff, W, dev))
        mid = torch.empty(used, ff, dtype=self.dtype, device=dev)
        ops.gated_act(up, ff, mid, self.act)
        ys = torch.empty(used, W, dtype=self.dtype, device=dev)
        ops.moe_expert_gemms(mid, self.w_down, ys, counts, tm, self._workspace(rows, W, ff, dev))
        ops.moe_combine(ys, self.shared(h) if self.shared is not None else None, y, top, pos_of=pos_of, wt=wt)
        return y

    def __call__(self, h):
        M, W, dev = h.shape[0], h.shape[1], h.device
        E, top = self.E, self.top
        logits = torch.empty(M, E, dtype=F32, device=dev)
        ops.linear_small(h, self.router, None, logits, ops.GATE_NONE)
        idx = torch.empty(M, top, dtype=torch.int32, device=dev)
        wt = torch.empty(M, top, dtype=F32, device=dev)
        ops.router_topk(logits, top, idx, wt)
        pairs = M * top
        y = torch.empty(M, W, dtype=F32, device=dev)
        if self.tensor_core and pairs >= self.TENSOR_CORE_PAIRS and h.is_contiguous() and not torch.cuda.is_current_stream_capturing():
            return self._experts_tensor_core(h, idx, wt, y)
        ypair = torch.empty(pairs, W, dtype=F32, device=dev)
        if pairs <= self.FEW_PAIRS:
            mid = torch.empty(pairs, self.ff, dtype=self.dtype, device=dev)
            ops.moe_gemm(h, self.w_up, mid, idx, wt, top, True, self.act)
            ops.moe_gemm(mid, self.w_down, ypair, idx, wt, top, False)
        else:
            n_tiles, tm = ops.moe_tiles(pairs, E)
            perm = torch.empty(n_tiles * tm, dtype=torch.int32, device=dev)
            tile_expert = torch.empty(n_tiles, dtype=torch.int32, device=dev)
            pos_of = torch.empty(pairs, dtype=torch.int32, device=dev)
            ops.moe_plan(idx, E, perm, tile_expert, pos_of)
            mid = torch.empty(n_tiles * tm, self.ff, dtype=self.dtype, device=dev)
            ops.moe_gemm(h, self.w_up, mid, idx, wt, top, True, self.act, perm, tile_expert)
            ops.moe_gemm(mid, self.w_down, ypair, idx, wt, top, False, ops.ACT_NONE, perm, tile_expert)
        ops.moe_combine(ypair, self.shared(h) if self.shared is not None else None, y, top)
        return y
