"""Plain, slow restatement of the Bebulorn design, one function per mechanism, in float64 PyTorch on the CPU.  It shares no
code with the product: every recurrence is a Python loop over tokens, attention builds the full score matrix with an
explicit mask, experts are visited token by token, and state is a dict per layer run.

Weights: dict name -> tensor ('l<i>.mix.q', ...), config: the dict of config.json.
"""
import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ norms and activations
def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_div(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------------------------------ feed-forwards
def relu_glu(h, w_gate, w_up, w_down):
    return (torch.relu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def expert(h, w_up, w_down):
    return gelu_erf(h @ w_up.T) @ w_down.T


def route(h, w_router, top):
    """Chosen experts [T, top] and their weights (softmax scores of the chosen, renormalised)."""
    s = torch.softmax(h @ w_router.T, -1)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val / (val.sum(-1, keepdim=True) + 1e-20)


def moe(h, w, p, cfg):
    idx, wt = route(h, w[p + "router"], cfg["router"]["top"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * expert(h[t], w[p + f"e{e}.up"], w[p + f"e{e}.down"])
    if cfg.get("shared") is not None:
        out = out + expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


# ------------------------------------------------------------------------------------------------ mixers
def lightning_recurrence(q, k, v, decay, state):
    """q, k [T, H, d], v [T, H, e], decay [H]; S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, d = q.shape
    S = state.get("S")
    if S is None:
        S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    state["S"] = S
    return torch.stack(out)


def lightning_mixer(h, w, p, cfg, eps, state):
    H, d, e = cfg["heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, e)
    o = lightning_recurrence(q, k, v, torch.tensor(cfg["decay"], dtype=F64), state).reshape(T, H * e)
    o = rms_div(o, eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def window_attention_mixer(h, w, p, cfg, eps, state):
    H, G, d, e = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    win, scale, cap = cfg["mask"]["size"], cfg["scale"], cfg["softcap"]
    T = h.shape[0]
    past = state.get("len", 0)
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = rms_div((h @ w[p + "v"].T).view(T, G, e), eps)
    if past:
        k, v = torch.cat([state["k"], k]), torch.cat([state["v"], v])
    state.update(k=k, v=v, len=past + T)
    out = torch.zeros(T, H, e, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * scale * w[p + "temp"][hd]
        s = cap * torch.tanh(s / cap)
        i = torch.arange(past, past + T)[:, None]
        j = torch.arange(past + T)[None, :]
        seen = (i - j >= 0) & (i - j < win)
        s = s.masked_fill(~seen, -math.inf)
        out[:, hd] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * e) @ w[p + "o"].T


def short_conv(x, w_conv, state, key):
    """x [T, C]; w_conv [C, taps] (last column: the current token); the taps - 1 inputs before x come from ``state``."""
    taps = w_conv.shape[1]
    prev = state.get(key)
    if prev is None:
        prev = torch.zeros(taps - 1, x.shape[1], dtype=F64)
    full = torch.cat([prev, x])
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[j:j + x.shape[0]] * w_conv[:, j]
    state[key] = full[full.shape[0] - (taps - 1):]
    return y


def delta_recurrence(q, k, v, beta, g, state):
    """q, k [T, H, d] (unit vectors, q scaled), v [T, H, e], beta, g [T, H]."""
    T, H, d = q.shape
    S = state.get("S")
    if S is None:
        S = torch.zeros(H, d, v.shape[-1], dtype=F64)
    out = []
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hde,hd->he", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hde,hd->he", S, q[t]))
    state["S"] = S
    return torch.stack(out)


def delta_mixer(h, w, p, cfg, eps, state):
    H, G, d, e = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"], state, "cq")).view(T, G, d)
    k = silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"], state, "ck")).view(T, G, d)
    v = silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"], state, "cv")).view(T, H, e)
    q, k = unit(q) * d ** -0.5, unit(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_recurrence(q, k, v, beta, g, state)
    o = rms_div(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).view(T, H, e)
    return o.reshape(T, H * e) @ w[p + "o"].T


MIXERS = {"lightning": lightning_mixer, "attention": window_attention_mixer, "delta": delta_mixer}


# ------------------------------------------------------------------------------------------------ the model
def layer_runs(config):
    """(layer index, first of a repeated pass) for every layer run."""
    lp, n = config.get("loop") or {"start": 0, "stop": 0, "times": 1}, len(config["layers"])
    runs = [(i, False) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t > 0 and i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, False) for i in range(lp["stop"], n)]


def new_states(config):
    return [dict() for _ in layer_runs(config)]


def forward(config, w, tokens, states, trace=None):
    """tokens: the next tokens of ONE sequence whose earlier tokens are in ``states``; returns logits [T, vocab] (float64)."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps, m = config["norm"]["eps"], config["residual_mult"]
    x0 = w["embed"][torch.as_tensor(tokens)]
    x = x0
    for r, (i, again) in enumerate(layer_runs(config)):
        L, p = config["layers"][i], f"l{i}."
        if again:
            x = x + x0
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        y = MIXERS[L["type"]](h, w, p + "mix.", L["mixer"], eps, states[r])
        x = x + m * layer_norm(y, w[p + "norm1b"], w[p + "norm1b.b"], eps)
        if L.get("mlp") is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            if L["mlp"]["kind"] == "dense":
                y = relu_glu(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
            else:
                y = moe(h, w, p + "mlp.", L["mlp"])
            x = x + m * layer_norm(y, w[p + "norm2b"], w[p + "norm2b.b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T


def tensor_shapes(config):
    """name -> shape of every tensor of a checkpoint of this configuration."""
    W, V = config["width"], config["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,), "head": (V, W)}
    for i, L in enumerate(config["layers"]):
        p, c = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") is not None else ()):
            out[p + n] = out[p + n + ".b"] = (W,)
        H, d, e = c["heads"], c["dim"], c["vdim"]
        if L["type"] == "lightning":
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * e, W), p + "mix.g": (H * e, W),
                        p + "mix.o": (W, H * e), p + "mix.norm": (H * e,)})
        elif L["type"] == "attention":
            G = c["kv_heads"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * e, W), p + "mix.temp": (H,),
                        p + "mix.o": (W, H * e)})
        else:
            G, taps = c["kv_heads"], c["conv"]
            out.update({p + "mix.q": (G * d, W), p + "mix.q.conv": (G * d, taps), p + "mix.k": (G * d, W), p + "mix.k.conv": (G * d, taps),
                        p + "mix.v": (H * e, W), p + "mix.v.conv": (H * e, taps), p + "mix.b": (H, W), p + "mix.A_log": (H,),
                        p + "mix.norm": (e,), p + "mix.a": (H, W), p + "mix.dt_bias": (H,), p + "mix.g": (H * e, W), p + "mix.o": (W, H * e)})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            f = mlp["expert"]["ff"]
            for e_ in range(mlp["router"]["experts"]):
                out.update({p + f"mlp.e{e_}.up": (f, W), p + f"mlp.e{e_}.down": (W, f)})
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared") is not None:
                out.update({p + "mlp.shared.up": (mlp["shared"]["ff"], W), p + "mlp.shared.down": (W, mlp["shared"]["ff"])})
    return out


def random_weights(config, seed, std_scale=1.0):
    """bf16-representable random weights: projections N(0, 1/in), norm weights near 1, biases and small vectors near 0."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shp in tensor_shapes(config).items():
        if name.endswith(".conv"):
            t = torch.randn(shp, generator=g) * 0.5
        elif len(shp) == 2:
            t = torch.randn(shp, generator=g) * std_scale * shp[1] ** -0.5
        elif name.endswith(".b") or name.endswith("dt_bias") or name.endswith("A_log"):
            t = 0.5 * torch.randn(shp, generator=g)
        else:
            t = 1.0 + 0.2 * torch.randn(shp, generator=g)
        out[name] = t.to(torch.bfloat16).float()
    return out
