"""Sequence mixers and feed-forwards that run on a 32-bit residual stream, each with its constants as parameters so that
any model design can assemble them: a matrix-memory recurrent mixer (mLSTM), attention over a latent key/value cache with
a partly rotated query/key and an output gate, and a clamped gated feed-forward.  Each object owns its (fused) weights,
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
