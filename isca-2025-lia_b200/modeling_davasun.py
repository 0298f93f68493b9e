"""Davasun: a decoder-only language model that interleaves matrix-memory recurrent mixers (mLSTM) with attention over a
latent key/value cache, on a 32-bit residual stream with a scalar-weight RMS norm before AND after every sublayer, and
with a block of layers that is run several times over (same weights, separate state per pass).

    x   = norm_embed(embed[token])
    per layer run:  x += norm1b(mixer(norm1(x)));  if the layer has a feed-forward:  x += norm2b(ff(norm2(x)))
    logits = head(norm_final(x)) * logit_scale

``config.json`` gives every size and constant (``DavasunConfig``); tensor names are ``embed``, ``embed.norm``,
``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.  The mixers and the
feed-forward are the general ones of ``seq_layers``; per-sequence state lives in a ``seq_state.SlotState``; serving goes
through ``engine.Engine`` (the model only implements ``new_state`` and ``forward_rows``).

dtype bfloat16: projections and their activations in bf16 with fp32 accumulation; positions and angles, norms, gates,
attention scores and weights, the recurrence and the residual stream in fp32.  dtype float32: everything in true fp32.
"""
import json
import os
from dataclasses import dataclass, field

import torch

from . import _lib, ops
from .seq_layers import ClampedGLU, LatentAttentionMixer, Linear, MLSTMMixer, StepBatch
from .seq_state import SlotState

BF16, F32 = torch.bfloat16, torch.float32
MIXERS = ("mlstm", "latent_attention")


@dataclass
class DavasunConfig:
    vocab: int = 0
    width: int = 0
    layers: list = field(default_factory=list)          # dicts: type, mixer {...}, mlp {...} | None
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    norm_eps: float = 1e-6
    logit_scale: float = 1.0
    name: str = "davasun"
    architectures: list = field(default_factory=lambda: ["Davasun"])
    eos_token_id: int = -1

    @classmethod
    def from_dict(cls, c, name="davasun"):
        layers = c["layers"]
        for i, l in enumerate(layers):
            if l.get("type") not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {l.get('type')!r} (known: {MIXERS})")
            mlp = l.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        loop = c.get("loop") or {"start": 0, "stop": 0, "times": 1}
        start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ValueError(f"bad loop {loop} for {len(layers)} layers")
        return cls(vocab=int(c["vocab"]), width=int(c["width"]), layers=layers, loop_start=start, loop_stop=stop, loop_times=times,
                   norm_eps=float(c["norm"]["eps"]), logit_scale=float(c.get("logit_scale", 1.0)), name=name)

    def to_dict(self):
        return {"architecture": "Davasun", "vocab": self.vocab, "width": self.width, "layers": self.layers,
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
                "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale}

    def layer_runs(self):
        """Layer index of every run, in order: the layers before the loop once, the looped block ``times`` times in a row,
        the rest once."""
        n = len(self.layers)
        return (list(range(0, self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times
                + list(range(self.loop_stop, n)))

    def tensor_shapes(self):
        """name -> shape of every tensor of a checkpoint of this configuration."""
        W, out = self.width, {"embed": (self.vocab, self.width), "embed.norm": (), "final.norm": (), "head": (self.vocab, self.width)}
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l["mixer"]
            out[p + "norm1"] = out[p + "norm1b"] = ()
            if l["type"] == "mlstm":
                H, d, v = m["heads"], m["dim"], m["vdim"]
                out.update({p + "mix.q": (H * d, W), p + "mix.k": (H * d, W), p + "mix.v": (H * v, W), p + "mix.g": (H * v, W),
                            p + "mix.o": (W, H * v), p + "mix.norm": (H * v,), p + "mix.i": (H, W), p + "mix.i.b": (H,),
                            p + "mix.f": (H, W), p + "mix.f.b": (H,)})
            else:
                H, d, r, v, c = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
                out.update({p + "mix.q": (H * (d + r), W), p + "mix.dkv": (c + r, W), p + "mix.dkv.norm": (c,), p + "mix.uk": (H * d, c),
                            p + "mix.uv": (H * v, c), p + "mix.g": (H, W), p + "mix.o": (W, H * v)})
            if l.get("mlp") is not None:
                f = l["mlp"]["ff"]
                out[p + "norm2"] = out[p + "norm2b"] = ()
                out.update({p + "mlp.gate": (f, W), p + "mlp.up": (f, W), p + "mlp.down": (W, f)})
        return out


class _Layer:
    def __init__(self, mixer, mlp, norms):
        self.mixer, self.mlp = mixer, mlp
        self.norm1, self.norm1b, self.norm2, self.norm2b = norms


class DavasunForCausalLM:
    step_serving = True          # served through engine.Engine (requests, slots, portions)

    def __init__(self, config, device="cuda", dtype=BF16):
        _lib.load()
        if dtype not in (BF16, F32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.config, self.device, self.dtype = config, torch.device(device), dtype
        self.layers = []
        self.runs = config.layer_runs()
        self.embed = self.head = self.embed_norm = self.final_norm = None

    # ---- weights
    def load_weights(self, get):
        """``get(name)`` -> CPU tensor (checkpoint dtype).  Projection weights take the model's dtype; norm weights and
        biases stay fp32."""
        cfg, dev, dt = self.config, self.device, self.dtype
        shapes = cfg.tensor_shapes()

        def fetch(name):
            t = get(name)
            if tuple(t.shape) != tuple(shapes[name]):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration needs {tuple(shapes[name])}")
            return t.float()

        scalar = lambda name: fetch(name).reshape(1).to(dev)  # noqa: E731
        self.embed = fetch("embed").to(device=dev, dtype=dt).contiguous()
        self.head = Linear([fetch("head")], dt, dev)
        self.embed_norm, self.final_norm = scalar("embed.norm"), scalar("final.norm")
        self.layers = []
        for i, l in enumerate(cfg.layers):
            p, m = f"l{i}.", l["mixer"]
            names = [k[len(p) + 4:] for k in shapes if k.startswith(p + "mix.")]
            w = {k: fetch(p + "mix." + k) for k in names}
            if l["type"] == "mlstm":
                mixer = MLSTMMixer(w, m["heads"], m["dim"], m["vdim"], m["gate_cap"], cfg.norm_eps, dt, dev)
            else:
                rot = m["rot"]
                if rot["dims"] > m["rot_dim"]:
                    raise ValueError(f"layer {i}: rot.dims {rot['dims']} exceeds rot_dim {m['rot_dim']}")
                mixer = LatentAttentionMixer(w, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], rot["dims"], rot["base"],
                                             m["scale"], cfg.norm_eps, dt, dev)
            mlp, n2, n2b = None, None, None
            if l.get("mlp") is not None:
                mw = {k: fetch(p + "mlp." + k) for k in ("gate", "up", "down")}
                mlp = ClampedGLU(mw, l["mlp"]["ff"], l["mlp"]["limit"], dt, dev)
                n2, n2b = scalar(p + "norm2"), scalar(p + "norm2b")
            self.layers.append(_Layer(mixer, mlp, (scalar(p + "norm1"), scalar(p + "norm1b"), n2, n2b)))
        return self

    def init_weights(self, seed=0, std=None):
        """Random weights (bf16-representable) for tests and benchmarks: N(0, K^-1/2) projections, norm weights near 1."""
        g = torch.Generator().manual_seed(seed)
        shapes = self.config.tensor_shapes()

        def make(name):
            shp = shapes[name]
            if len(shp) == 2:
                t = torch.randn(shp, generator=g) * (std if std is not None else shp[1] ** -0.5)
            elif name.endswith(".b"):
                t = torch.randn(shp, generator=g)
            else:
                t = 1.0 + 0.1 * torch.randn(shp, generator=g)
            return t.to(BF16)

        cache = {}
        return self.load_weights(lambda n: cache.setdefault(n, make(n)))

    @classmethod
    def from_pretrained(cls, path, device="cuda", dtype=BF16, **unused):
        from .checkpoint import SafetensorsFile
        cfg = DavasunConfig.from_dict(json.load(open(os.path.join(path, "config.json"))),
                                      name=os.path.basename(os.path.abspath(path)) or "davasun")
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
        slots.run_state = [self.layers[i].mixer.new_state(slots) for i in self.runs]      # one state per layer RUN
        return slots

    def forward_rows(self, ids, batch, want, slots, trace=None):
        """One step: ``ids`` int64 [rows] on the device, ``batch`` a StepBatch, ``want`` int32 row indices (device) whose
        logits are returned as fp32 [len(want), vocab] (None when empty).  ``trace``: a list that receives a copy of the
        residual stream after every layer run."""
        cfg, dev, dt = self.config, self.device, self.dtype
        M, W, eps = batch.rows, cfg.width, cfg.norm_eps
        x = torch.empty(M, W, dtype=F32, device=dev)
        h = torch.empty(M, W, dtype=dt, device=dev)
        ops.embed_rmsnorm(ids, self.embed, self.embed_norm, x, eps)
        first = self.layers[self.runs[0]] if self.runs else None
        if first is not None:
            ops.rms_add_norm(x, None, None, first.norm1, h, eps)
        for r, li in enumerate(self.runs):
            layer = self.layers[li]
            nxt = self.layers[self.runs[r + 1]].norm1 if r + 1 < len(self.runs) else None
            y = layer.mixer(h, batch, slots.run_state[r])
            if layer.mlp is not None:
                ops.rms_add_norm(x, y, layer.norm1b, layer.norm2, h, eps)
                y = layer.mlp(h)
                ops.rms_add_norm(x, y, layer.norm2b, nxt, h if nxt is not None else None, eps)
            else:
                ops.rms_add_norm(x, y, layer.norm1b, nxt, h if nxt is not None else None, eps)
            if trace is not None:
                trace.append(x.clone())
        if want is None or want.numel() == 0:
            return None
        n = want.numel()
        hn = torch.empty(n, W, dtype=dt, device=dev)
        ops.rms_gather(x, want, self.final_norm, hn, eps)
        logits = torch.empty(n, cfg.vocab, dtype=F32, device=dev)
        ops.linear_plain(hn, self.head.weight, logits, scale=cfg.logit_scale)
        return logits

    def graph_class(self, max_ctx):
        """What a decode pass's launches depend on besides the contents of the static buffers: the number of key ranges the
        attention splits the longest history into."""
        return ops.latent_attn_split_class(max_ctx)

    def generate(self, input_ids, max_new_tokens=32, chunk=None, **unused):
        """Greedy generation of a batch of prompts through the step engine; returns ids [B, S + new] on the input's device."""
        from .engine import Engine
        prompts = [[int(t) for t in row] for row in input_ids.tolist()]
        eng = Engine(self, max_tokens=len(prompts) * (len(prompts[0]) + max_new_tokens), max_requests=len(prompts))
        out = eng.generate(prompts, max_new_tokens, chunk=chunk)
        return torch.tensor(out, dtype=torch.int64, device=input_ids.device)
