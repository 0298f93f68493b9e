"""Bebulorn: a decoder-only language model that mixes three kinds of sequence mixer -- linear attention with a fixed decay per
head ("lightning"), sliding-window softmax attention with grouped key/value heads, and the gated delta rule behind a short
convolution -- with dense (ReLU-gated) or mixture-of-experts feed-forwards, on a 32-bit residual stream between layer norms,
with a block of layers that is run several times over (same weights, separate state per pass; the embedding is added back
before every pass but the first).

    x0  = embed[token];  x = x0
    per layer run:  (x += x0 at the first layer of a repeated pass)
                    x += m * LN1b(mixer(LN1(x)));   if the layer has a feed-forward:  x += m * LN2b(ff(LN2(x)))
    logits = head(LN_final(x))                                    m = residual_mult, LN with weight and bias

``config.json`` gives every size and constant (``BebulornConfig``); tensor names are ``embed``, ``l<i>.norm1|norm1b|norm2|
norm2b`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm`` (+ ``.b``), ``head``.  The mixers and feed-forwards are the
general ones of ``seq_layers``; per-sequence state lives in a ``seq_state.SlotState``; serving goes through ``engine.Engine``
(the model only implements ``new_state`` and ``forward_rows``).

dtype bfloat16: projections, convolution inputs and their activations in bf16 with fp32 accumulation; norms, routers, gates,
decays, unit vectors, attention scores and weights, the recurrences and the residual stream in fp32.  dtype float32:
everything in true fp32.
"""
import json
import os
from dataclasses import dataclass, field

import torch

from . import _lib, ops
from .seq_layers import (DecayLinearAttentionMixer, DeltaRuleMixer, GatedMLP, Linear, MoEFeedForward, PlainMLP,
                         WindowAttentionMixer)
from .seq_state import SlotState

BF16, F32 = torch.bfloat16, torch.float32
MIXERS = ("lightning", "attention", "delta")
MLP_KINDS = ("dense", "moe")


@dataclass
class BebulornConfig:
    vocab: int = 0
    width: int = 0
    layers: list = field(default_factory=list)          # dicts: type, mixer {...}, mlp {...} | None
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    name: str = "bebulorn"
    architectures: list = field(default_factory=lambda: ["Bebulorn"])
    eos_token_id: int = -1

    @classmethod
    def from_dict(cls, c, name="bebulorn"):
        layers = c["layers"]
        for i, l in enumerate(layers):
            if l.get("type") not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {l.get('type')!r} (known: {MIXERS})")
            mlp = l.get("mlp")
            if mlp is not None:
                mlp.setdefault("kind", "moe" if "router" in mlp else "dense")
                if mlp["kind"] not in MLP_KINDS:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r} (known: {MLP_KINDS})")
            m = l["mixer"]
            m.setdefault("vdim", m["dim"])                       # value heads as wide as query/key heads unless said otherwise
            if l["type"] != "lightning":
                m.setdefault("kv_heads", m["heads"])             # ungrouped unless said otherwise
            if l["type"] != "lightning" and m["heads"] % m["kv_heads"]:
                raise ValueError(f"layer {i}: {m['heads']} heads do not divide into {m['kv_heads']} groups")
            if l["type"] == "lightning":
                if not isinstance(m["decay"], (list, tuple)):
                    m["decay"] = [float(m["decay"])] * m["heads"]          # one decay for all heads
                if len(m["decay"]) != m["heads"]:
                    raise ValueError(f"layer {i}: {len(m['decay'])} decays for {m['heads']} heads")
        loop = c.get("loop") or {"start": 0, "stop": 0, "times": 1}
        start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ValueError(f"bad loop {loop} for {len(layers)} layers")
        return cls(vocab=int(c["vocab"]), width=int(c["width"]), layers=layers, loop_start=start, loop_stop=stop, loop_times=times,
                   norm_eps=float(c["norm"]["eps"]), residual_mult=float(c.get("residual_mult", 1.0)), name=name)

    def to_dict(self):
        return {"architecture": "Bebulorn", "vocab": self.vocab, "width": self.width, "layers": self.layers,
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult}

    def layer_runs(self):
        """(layer index, starts a repeated pass) of every run, in order: the layers before the loop once, the looped block
        ``times`` times in a row, the rest once.  The flag marks the first layer of every pass but the first."""
        runs = [(i, False) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            runs += [(i, t > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, False) for i in range(self.loop_stop, len(self.layers))]

    def tensor_shapes(self):
        """name -> shape of every tensor of a checkpoint of this configuration."""
        W, V = self.width, self.vocab
        out = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,), "head": (V, W)}
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            norms = ("norm1", "norm1b") + (("norm2", "norm2b") if l.get("mlp") is not None else ())
            for n in norms:
                out[p + n] = out[p + n + ".b"] = (W,)
            H, d, v = m["heads"], m["dim"], m["vdim"]
            if l["type"] == "lightning":
                out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * v, W), p + "mix.g": (H * v, W),
                            p + "mix.o": (W, H * v), p + "mix.norm": (H * v,)})
            elif l["type"] == "attention":
                G = m["kv_heads"]
                out.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * v, W), p + "mix.temp": (H,),
                            p + "mix.o": (W, H * v)})
            else:
                G, taps = m["kv_heads"], m["conv"]
                out.update({p + "mix.q": (G * d, W), p + "mix.q.conv": (G * d, taps), p + "mix.k": (G * d, W), p + "mix.k.conv": (G * d, taps),
                            p + "mix.v": (H * v, W), p + "mix.v.conv": (H * v, taps), p + "mix.b": (H, W), p + "mix.a": (H, W),
                            p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.norm": (v,), p + "mix.g": (H * v, W), p + "mix.o": (W, H * v)})
            mlp = l.get("mlp")
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                f = mlp["ff"]
                out.update({p + "mlp.gate": (f, W), p + "mlp.up": (f, W), p + "mlp.down": (W, f)})
            else:
                f = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    out.update({p + f"mlp.e{e}.up": (f, W), p + f"mlp.e{e}.down": (W, f)})
                out[p + "mlp.router"] = (mlp["router"]["experts"], W)
                if mlp.get("shared") is not None:
                    fs = mlp["shared"]["ff"]
                    out.update({p + "mlp.shared.up": (fs, W), p + "mlp.shared.down": (W, fs)})
        return out


class _Layer:
    def __init__(self, mixer, mlp, norms):
        self.mixer, self.mlp = mixer, mlp
        self.norm1, self.norm1b, self.norm2, self.norm2b = norms      # (weight, bias) pairs


class BebulornForCausalLM:
    step_serving = True          # served through engine.Engine (requests, slots, portions)

    def __init__(self, config, device="cuda", dtype=BF16):
        _lib.load()
        if dtype not in (BF16, F32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.config, self.device, self.dtype = config, torch.device(device), dtype
        self.layers = []
        self.runs = config.layer_runs()
        self.embed = self.head = self.final_norm = None

    # ---- weights
    def load_weights(self, get):
        """``get(name)`` -> CPU tensor (checkpoint dtype).  Projection weights take the model's dtype; norm weights, biases and
        the small per-head vectors stay fp32."""
        cfg, dev, dt = self.config, self.device, self.dtype
        shapes = cfg.tensor_shapes()

        def fetch(name):
            t = get(name)
            if tuple(t.shape) != tuple(shapes[name]):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration needs {tuple(shapes[name])}")
            return t.float()

        def norm(name):
            return fetch(name).to(dev).contiguous(), fetch(name + ".b").to(dev).contiguous()

        self.embed = fetch("embed").to(device=dev, dtype=dt).contiguous()
        self.head = Linear([fetch("head")], dt, dev)
        self.final_norm = norm("final.norm")
        self.layers = []
        for i, l in enumerate(cfg.layers):
            p, m = f"l{i}.", l["mixer"]
            w = {k[len(p) + 4:]: fetch(k) for k in shapes if k.startswith(p + "mix.")}
            if l["type"] == "lightning":
                mixer = DecayLinearAttentionMixer(w, m["heads"], m["dim"], m["vdim"], m["decay"], cfg.norm_eps, dt, dev)
            elif l["type"] == "attention":
                mixer = WindowAttentionMixer(w, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"], m["scale"], m.get("softcap", 0.0),
                                             cfg.norm_eps, dt, dev)
            else:
                mixer = DeltaRuleMixer(w, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], cfg.norm_eps, dt, dev)
            mlp, n2, n2b = None, None, None
            spec = l.get("mlp")
            if spec is not None:
                q = p + "mlp."
                if spec["kind"] == "dense":
                    mlp = GatedMLP({k: fetch(q + k) for k in ("gate", "up", "down")}, spec["ff"], ops.ACT_RELU, dt, dev)
                else:
                    shared = None
                    if spec.get("shared") is not None:
                        shared = PlainMLP({k: fetch(q + "shared." + k) for k in ("up", "down")}, spec["shared"]["ff"], ops.ACT_GELU_ERF, dt, dev)
                    experts = [{k: fetch(q + f"e{e}." + k) for k in ("up", "down")} for e in range(spec["router"]["experts"])]
                    mlp = MoEFeedForward(fetch(q + "router"), experts, spec["router"]["top"], spec["expert"]["ff"], ops.ACT_GELU_ERF, shared, dt, dev)
                n2, n2b = norm(p + "norm2"), norm(p + "norm2b")
            self.layers.append(_Layer(mixer, mlp, (norm(p + "norm1"), norm(p + "norm1b"), n2, n2b)))
        return self

    def init_weights(self, seed=0, std=None):
        """Random weights (bf16-representable) for tests and benchmarks: N(0, K^-1/2) projections, norm weights near 1, biases
        and the small per-head vectors near 0."""
        g = torch.Generator().manual_seed(seed)
        shapes = self.config.tensor_shapes()

        def make(name):
            shp = shapes[name]
            if name.endswith(".conv"):
                t = torch.randn(shp, generator=g) * 0.5
            elif len(shp) == 2:
                t = torch.randn(shp, generator=g) * (std if std is not None else shp[1] ** -0.5)
            elif name.endswith((".b", "dt_bias", "A_log")):
                t = 0.5 * torch.randn(shp, generator=g)
            else:
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            return t.to(BF16)

        cache = {}
        return self.load_weights(lambda n: cache.setdefault(n, make(n)))

    @classmethod
    def from_pretrained(cls, path, device="cuda", dtype=BF16, **unused):
        from .checkpoint import SafetensorsFile
        cfg = BebulornConfig.from_dict(json.load(open(os.path.join(path, "config.json"))),
                                       name=os.path.basename(os.path.abspath(path)) or "bebulorn")
        f = SafetensorsFile(os.path.join(path, "model.safetensors"))
        try:
            return cls(cfg, device, dtype).load_weights(f.get)
        finally:
            f.close()

    def eval(self):
        return self

    # ---- serving interface (engine.Engine)
    def new_state(self, n_slots, capacity):
        slots = SlotState(n_slots, capacity, self.device)
        slots.run_state = [self.layers[i].mixer.new_state(slots) for i, _ in self.runs]      # one state per layer RUN
        return slots

    def forward_rows(self, ids, batch, want, slots, trace=None):
        """One step: ``ids`` int64 [rows] on the device, ``batch`` a StepBatch, ``want`` int32 row indices (device) whose
        logits are returned as fp32 [len(want), vocab] (None when empty).  ``trace``: a list that receives a copy of the
        residual stream after every layer run."""
        cfg, dev, dt = self.config, self.device, self.dtype
        M, W, eps, mult = batch.rows, cfg.width, cfg.norm_eps, cfg.residual_mult
        repeats = any(again for _, again in self.runs)
        x = torch.empty(M, W, dtype=F32, device=dev)
        x0 = torch.empty(M, W, dtype=F32, device=dev) if repeats else None
        h = torch.empty(M, W, dtype=dt, device=dev)
        ops.embed_rows(ids, self.embed, x, x0)
        if self.runs:
            ops.ln_add_norm(x, None, None, mult, self.layers[self.runs[0][0]].norm1, h, eps)
        for r, (li, again) in enumerate(self.runs):
            layer = self.layers[li]
            if again:                                    # a repeated pass: the embedding is added back, then this layer's norm
                ops.ln_add_norm(x, None, None, mult, layer.norm1, h, eps, extra=x0)
            # the norm before the next run's mixer rides on this run's last residual update, unless that run starts a pass
            nxt = None
            if r + 1 < len(self.runs) and not self.runs[r + 1][1]:
                nxt = self.layers[self.runs[r + 1][0]].norm1
            y = layer.mixer(h, batch, slots.run_state[r])
            if layer.mlp is not None:
                ops.ln_add_norm(x, y, layer.norm1b, mult, layer.norm2, h, eps)
                y = layer.mlp(h)
                ops.ln_add_norm(x, y, layer.norm2b, mult, nxt, h if nxt is not None else None, eps)
            else:
                ops.ln_add_norm(x, y, layer.norm1b, mult, nxt, h if nxt is not None else None, eps)
            if trace is not None:
                trace.append(x.clone())
        if want is None or want.numel() == 0:
            return None
        n = want.numel()
        hn = torch.empty(n, W, dtype=dt, device=dev)
        ops.ln_gather(x, want, self.final_norm, hn, eps)
        logits = torch.empty(n, cfg.vocab, dtype=F32, device=dev)
        ops.linear_plain(hn, self.head.weight, logits)
        return logits

    def graph_class(self, max_ctx):
        """What a decode pass's launches depend on besides the contents of the static buffers: the number of key ranges each
        attention layer splits the longest history's window into."""
        return tuple(sorted({ops.window_attn_split_class(max_ctx, l.mixer.window) for l in self.layers if isinstance(l.mixer, WindowAttentionMixer)}))

    def generate(self, input_ids, max_new_tokens=32, chunk=None, **unused):
        """Greedy generation of a batch of prompts through the step engine; returns ids [B, S + new] on the input's device."""
        from .engine import Engine
        prompts = [[int(t) for t in row] for row in input_ids.tolist()]
        eng = Engine(self, max_tokens=len(prompts[0]) + max_new_tokens, max_requests=len(prompts))
        out = eng.generate(prompts, max_new_tokens, chunk=chunk)
        return torch.tensor(out, dtype=torch.int64, device=input_ids.device)
