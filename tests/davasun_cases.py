"""Small Davasun configurations for the tests (none of them a real model's sizes): odd head counts, sizes that are not
multiples of 8 or 32, loops that cover part of the stack, feed-forwards on either kind of layer."""


def mlstm(heads, dim, vdim, cap=15.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def latent(heads, dim, rot, vdim, rank, base=10000.0, scale=None, mlp=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "rot": {"base": base, "dims": rot},
                      "scale": scale if scale is not None else (dim + rot) ** -0.5},
            "mlp": mlp}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(layers, vocab, width, loop=None, eps=1e-5, logit_scale=1.0):
    return {"architecture": "Davasun", "vocab": vocab, "width": width, "layers": layers,
            "loop": loop or {"start": 0, "stop": 0, "times": 1}, "norm": {"eps": eps}, "logit_scale": logit_scale}


CASES = {
    # sizes that are multiples of 8: bf16 projections run on the tensor-core GEMM
    "even": config([mlstm(3, 16, 40), latent(3, 24, 8, 16, 48, mlp=dense(72, 1.5)), mlstm(2, 40, 24, cap=8.0, mlp=dense(40, 3.0)),
                    latent(5, 8, 16, 24, 32, base=500.0)], vocab=120, width=64, loop={"start": 1, "stop": 3, "times": 3},
                   eps=1e-5, logit_scale=0.7),
    # nothing divides by 8: every projection takes the plain kernel; one head, loop of one layer, no loop at the ends
    "odd": config([latent(1, 12, 6, 10, 20, mlp=dense(30, 0.8)), mlstm(1, 36, 20), mlstm(3, 10, 70, cap=4.0)], vocab=61, width=44,
                  loop={"start": 1, "stop": 2, "times": 2}, eps=1e-6, logit_scale=3.0),
    # a stack without a loop, wide heads (dim > 64, vdim > 64), rank > 256
    "wide": config([mlstm(2, 80, 136), latent(9, 16, 4, 8, 264)], vocab=90, width=96, logit_scale=1.0),
}
