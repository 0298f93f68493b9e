"""Small Bebulorn configurations for the tests (none of them a real model's sizes): odd head counts, sizes that are not
multiples of 8 or 32, grouped and ungrouped heads, convolutions of 1 to 5 taps, windows shorter and longer than the prompts,
routers that take one expert or all of them, layers without a feed-forward, loops at the start, in the middle and absent."""


def lightning(heads, dim, vdim, decay=None, mlp=None):
    decay = decay if decay is not None else [1.0 - 0.5 ** (i + 1) for i in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, window, scale=None, softcap=30.0, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                                           "scale": scale if scale is not None else dim ** -0.5, "softcap": softcap}, "mlp": mlp}


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def config(layers, vocab, width, loop=None, eps=1e-5, mult=1.0):
    return {"architecture": "Bebulorn", "vocab": vocab, "width": width, "layers": layers,
            "loop": loop or {"start": 0, "stop": 0, "times": 1}, "norm": {"eps": eps}, "residual_mult": mult}


CASES = {
    # sizes that are multiples of 8: bf16 projections run on the tensor-core GEMM; loop in the middle, three passes
    "even": config([delta(4, 2, 16, 24, 4, mlp=dense(72)), lightning(3, 16, 40, mlp=moe(6, 2, 24, shared=40)),
                    attention(6, 2, 24, 16, 11, mlp=dense(40)), lightning(2, 40, 24, decay=[0.9, 1.0], mlp=moe(4, 4, 16)),
                    delta(2, 2, 40, 8, 2)], vocab=120, width=64, loop={"start": 1, "stop": 4, "times": 3}, eps=1e-5, mult=0.7),
    # nothing divides by 8: every projection takes the plain kernel; one head, one tap, one expert of one; a loop of one layer
    # at the very start; a window longer than any prompt of the tests
    "odd": config([attention(1, 1, 12, 10, 500, softcap=3.0, mlp=moe(1, 1, 9, shared=5)), delta(3, 1, 10, 7, 1, mlp=dense(30)),
                   lightning(1, 36, 20), delta(3, 3, 12, 34, 5, mlp=moe(5, 3, 11))], vocab=61, width=44,
                  loop={"start": 0, "stop": 1, "times": 2}, eps=1e-6, mult=1.3),
    # a stack without a loop; wide heads (dim > 64, vdim > 64); nine query heads on three key/value heads; a window of one
    "wide": config([lightning(2, 80, 136), attention(9, 3, 72, 80, 1), attention(4, 4, 8, 136, 40, mlp=dense(16)),
                    delta(2, 1, 136, 72, 3)], vocab=90, width=96, mult=0.25),
}
