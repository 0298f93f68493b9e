"""Plain, slow restatement of the Davasun design, one function per mechanism, in float64 PyTorch on the CPU.  It shares no
code with the product: attention expands every head's keys and values from the latent (the product works in the latent
space), the recurrence is a Python loop over tokens, and state is a dict per layer run.

Weights: dict name -> tensor ('l<i>.mix.q', ...), config: the dict of config.json.
"""
import math

import torch

F64 = torch.float64


def rms_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_like_gate(g, alpha=1.702):
    return g * torch.sigmoid(alpha * g)


def clamped_glu(h, w_gate, w_up, w_down, limit):
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, min=-limit, max=limit)
    return (gelu_like_gate(g) * (u + 1.0)) @ w_down.T


def rotate_half(x, positions, dims, base):
    """x [T, ..., n]; channel i < dims/2 is paired with i + dims/2; channels >= dims pass unchanged."""
    half = dims // 2
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def mlstm_gates(h, w_i, b_i, w_f, b_f, cap):
    i = cap * torch.tanh((h @ w_i.T + b_i) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w_f.T + b_f) / cap))
    return i, f


def mlstm_recurrence(q, k, v, i, f, state, den_eps=1e-6):
    """q, k [T, H, d], v [T, H, e], i, f [T, H]; state dict with S [H, d, e], n [H, d], m [H] (created at zero)."""
    T, H, d = q.shape
    e = v.shape[-1]
    if not state:
        state.update(S=torch.zeros(H, d, e, dtype=F64), n=torch.zeros(H, d, dtype=F64), m=torch.zeros(H, dtype=F64))
    S, n, m = state["S"], state["n"], state["m"]
    out = []
    for t in range(T):
        m_new = torch.maximum(f[t] + m, i[t])
        a, b = torch.exp(f[t] + m - m_new), torch.exp(i[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hde,hd->he", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + den_eps
        out.append(num / den[:, None])
    state.update(S=S, n=n, m=m)
    return torch.stack(out)


def mlstm_mixer(h, w, p, cfg, eps, state):
    H, d, e = cfg["heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, e)
    i, f = mlstm_gates(h, w[p + "i"], w[p + "i.b"], w[p + "f"], w[p + "f.b"], cfg["gate_cap"])
    o = mlstm_recurrence(q, k, v, i, f, state)
    o = rms_norm(o, eps).reshape(T, H * e) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def latent_attention_mixer(h, w, p, cfg, eps, state):
    H, d, r, e, c = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    dims, base = cfg["rot"]["dims"], cfg["rot"]["base"]
    T = h.shape[0]
    past = state.get("len", 0)
    pos = torch.arange(past, past + T)
    q = (h @ w[p + "q"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_half(q[..., d:], pos, dims, base)
    dkv = h @ w[p + "dkv"].T
    lat = rms_norm(dkv[:, :c], eps) * w[p + "dkv.norm"]
    k_rot = rotate_half(dkv[:, c:], pos, dims, base)
    if past:
        lat, k_rot = torch.cat([state["lat"], lat]), torch.cat([state["k_rot"], k_rot])
    state.update(lat=lat, k_rot=k_rot, len=past + T)
    k_plain = (lat @ w[p + "uk"].T).view(-1, H, d)
    val = (lat @ w[p + "uv"].T).view(-1, H, e)
    s = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_rot, k_rot)) * cfg["scale"]
    visible = torch.arange(past + T)[None, :] <= pos[:, None]
    s = s.masked_fill(~visible[None], -math.inf)
    a = torch.softmax(s, -1)
    o = torch.einsum("hts,she->the", a, val) * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * e) @ w[p + "o"].T


def layer_runs(config):
    lp, n = config.get("loop") or {"start": 0, "stop": 0, "times": 1}, len(config["layers"])
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def new_states(config):
    return [dict() for _ in layer_runs(config)]


def forward(config, w, tokens, states, trace=None):
    """tokens: the next tokens of ONE sequence whose earlier tokens are in ``states``; returns logits [T, vocab] (float64)."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = rms_norm(w["embed"][torch.as_tensor(tokens)], eps) * w["embed.norm"]
    for r, i in enumerate(layer_runs(config)):
        L, p = config["layers"][i], f"l{i}."
        h = rms_norm(x, eps) * w[p + "norm1"]
        mix = mlstm_mixer if L["type"] == "mlstm" else latent_attention_mixer
        x = x + rms_norm(mix(h, w, p + "mix.", L["mixer"], eps, states[r]), eps) * w[p + "norm1b"]
        if L.get("mlp") is not None:
            h = rms_norm(x, eps) * w[p + "norm2"]
            y = clamped_glu(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"], L["mlp"]["limit"])
            x = x + rms_norm(y, eps) * w[p + "norm2b"]
        if trace is not None:
            trace.append(x.clone())
    return (rms_norm(x, eps) * w["final.norm"]) @ w["head"].T * config.get("logit_scale", 1.0)


def random_weights(shapes, seed, std_scale=1.0):
    """bf16-representable random weights for the given name -> shape table."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shp in shapes.items():
        if len(shp) == 2:
            t = torch.randn(shp, generator=g) * std_scale * shp[1] ** -0.5
        elif name.endswith(".b"):
            t = torch.randn(shp, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shp, generator=g)
        out[name] = t.to(torch.bfloat16).float()
    return out
