"""GPU checks of the paths that were added last -- the only GPU tests that had not yet run on
hardware when committed, which is why the file is named to run after the others.  Each path re-uses the kernels the
other GPU files verify, in a new order or layout whose HOST side is pinned bit-exactly on CPU (tests/test_host_model_cpu.py,
tests/test_kv_spill.py):

  * opt-350m's variant of the layer: LayerNorm AFTER each residual add (decoder.py:250-259, 320-321), no final LayerNorm
    (lia/modeling_opt.py:1001-1006), bias-free project_in / project_out around a narrower token table
    (lia/modeling_opt.py:988-996, 1139-1140, 1566-1567) -- against the golden made from the reference's own layer code and
    against the oracle run on the same GPU;
  * --no-overlap (lia/modeling_opt.py:1173) as a pure scheduling knob;
  * head_dim 80 (opt-2.7b) on the head_dim-128 kernels with zero-padded heads, against the oracle on the unpadded weights."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
REL_TOL = 1e-2     # north_star: per-layer hidden-state max relative error


@pytest.fixture(scope="module")
def lia():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import lia_b200
    return lia_b200


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(BF16)


def rel_err(got, ref):
    got, ref = got.float().cpu(), ref.float().cpu()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


def oracle_model(m, device):
    dec = m.model.decoder
    hq = dec.layout.hq
    layers = []
    for v in dec.resident_views:
        w = {k: v[k] for k in ("ln1_w", "ln1_b", "o_w", "o_b", "ln2_w", "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b")}
        w["q_w"], w["k_w"], w["v_w"] = v["qkv_w"][:hq], v["qkv_w"][hq:2 * hq], v["qkv_w"][2 * hq:]
        w["q_b"], w["k_b"], w["v_b"] = v["qkv_b"][:hq], v["qkv_b"][hq:2 * hq], v["qkv_b"][2 * hq:]
        layers.append({k: t.to(device) for k, t in w.items()})
    mv = lambda t: None if t is None else t.to(device)  # noqa: E731
    return {"H": m.config.num_attention_heads, "layers": layers, "pre_ln": m.config.do_layer_norm_before,
            "embed_tokens": mv(dec.embed_tokens), "embed_positions": mv(dec.embed_positions), "final_ln_w": mv(dec.final_ln_w),
            "final_ln_b": mv(dec.final_ln_b), "project_in": mv(dec.project_in), "project_out": mv(dec.project_out)}


def test_postln_layer_vs_reference_golden(lia, golden_dir):
    """decoder_layer(...) face with do_layer_norm_before=False against outputs of the reference's own
    OPTDecoderLayer_forward (oracle/gen_golden.py -> layer_postln.npz)."""
    from lia_b200.weights import LAYER_KEYS
    z = np.load(os.path.join(golden_dir, "layer_postln.npz"))
    assert int(z["pre_ln"]) == 0
    B, S, h, H, new = (int(z[k]) for k in ("B", "S", "h", "H", "new"))
    w = {k[2:]: _bf16(z[k]) for k in z.files if k.startswith("w_")}
    cfg = lia.OPTConfig(hidden_size=h, num_hidden_layers=1, num_attention_heads=H, ffn_dim=4 * h, vocab_size=64,
                        max_position_embeddings=64, do_layer_norm_before=False)
    m = lia.OPTForCausalLM(cfg, "cuda")
    layer = m.model.decoder.layers[0]
    gl = [w[k].cuda() for k in LAYER_KEYS]
    past = None
    for step in range(new + 1):
        x = _bf16(z[f"x{step}"]).cuda()
        out = layer(x, past_key_value=past, use_cache=True, gpu_layer=gl, policy=3, max_new_tokens=new)
        y, past = out[0], out[1]
        assert past[0].shape[2] == S + step
        e = rel_err(y, _bf16(z[f"y{step}"]))
        assert e <= REL_TOL, (step, e)
    T = S + new
    assert rel_err(past[1][:T], _bf16(z["kcache"])) <= REL_TOL and rel_err(past[2][:T], _bf16(z["vcache"])) <= REL_TOL


def test_postln_projected_model_vs_oracle(lia):
    """Whole surface (embeddings + project_in, post-LN layers, project_out, lm_head) against the oracle on the same GPU;
    M = 160 rows in prefill (one-CTA GEMM, bias-free residual epilogue) and M = 4 in decode (swap-AB)."""
    from oracle import opt_ref
    cfg = lia.OPTConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, ffn_dim=1024, vocab_size=512,
                        max_position_embeddings=96, do_layer_norm_before=False, word_embed_proj_dim=128)
    m = lia.OPTForCausalLM(cfg, "cuda").init_weights(seed=6, bias_std=0.02, ln_std=0.05)
    dec = m.model.decoder
    assert dec.final_ln_w is None and dec.project_in.shape == (256, 128)
    om = oracle_model(m, "cuda")
    B, S, new = 4, 40, 6
    ids = torch.randint(3, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(8))
    ones = torch.ones(B, S, dtype=torch.long, device="cuda")
    hidden, past = dec(input_ids=ids.cuda(), attention_mask=ones, max_new_tokens=new)
    assert hidden.shape == (B, S, 128)                                   # project_out: back in the token table's width
    nxt = torch.randint(3, cfg.vocab_size, (B, 1), generator=torch.Generator().manual_seed(9))
    ones1 = torch.ones(B, S + 1, dtype=torch.long, device="cuda")
    hidden1, _ = dec(input_ids=nxt.cuda(), attention_mask=ones1, past_key_values=past, max_new_tokens=new)
    with torch.no_grad():
        cache = opt_ref.new_cache(om, B, S + new)
        hs = []
        href = opt_ref.decoder_forward(om, ids.cuda(), ones, cache, 0, collect=hs)
        href1 = opt_ref.decoder_forward(om, nxt.cuda(), ones1, cache, S)
        x0 = opt_ref.embed(om, ids.cuda(), ones, 0)
    assert rel_err(hidden, href) <= 3 * REL_TOL and rel_err(hidden1, href1) <= 3 * REL_TOL      # chained through 2 layers
    for li, layer in enumerate(dec.layers):                               # per layer, each fed the oracle's input
        inp = x0 if li == 0 else hs[li - 1]
        y = layer(inp, use_cache=True, policy=3, max_new_tokens=new)[0]
        assert rel_err(y, hs[li]) <= REL_TOL, (li, rel_err(y, hs[li]))
    logits, _ = m(input_ids=ids.cuda(), attention_mask=ones, max_new_tokens=new)
    with torch.no_grad():
        lref = opt_ref.lm_logits(om, href)
    assert logits.shape == (B, 1, cfg.vocab_size) and rel_err(logits, lref) <= 5 * REL_TOL
    toks = [m.generate(ids, max_new_tokens=new, min_new_tokens=new, num_minibatch=2).cpu() for _ in range(3)]
    assert torch.equal(toks[0], toks[1]) and torch.equal(toks[1], toks[2])     # eager, graph capture, graph replay
    assert torch.equal(toks[0][:, :S], ids) and not (toks[0][:, S:] == cfg.eos_token_id).any()
    # first generated token: must be the oracle's wherever the oracle's top-2 margin exceeds what the measured logit
    # error can bridge (4 x the largest logit difference seen above: generate() runs the prefill in two minibatches,
    # i.e. through the other GEMM mode, so its logits may differ from the forward face's by about as much again)
    lg = lref[:, -1].float().cpu()
    eps = (logits[:, -1].float().cpu() - lg).abs().max().item()
    lg[:, cfg.eos_token_id] = float("-inf")
    top2 = lg.topk(2, dim=-1)
    safe = (top2.values[:, 0] - top2.values[:, 1]) > 4 * eps + 2.0 ** -8 * top2.values[:, 0].abs()
    assert torch.equal(toks[0][safe, S], top2.indices[safe, 0])


def test_no_overlap_is_a_scheduling_knob(lia):
    """--no-overlap (lia/modeling_opt.py:1173: the reference's ablation of its prefetch pipeline): streamed layers and
    spilled K/V go through ONE device slot, nothing is fetched ahead.  Tokens must stay bit-identical, with the flag on,
    off again, and across repeated generate() calls (the slot bookkeeping survives the switch)."""
    cfg = lia.modeling_opt.get_config("opt-1.3b")
    cfg.num_hidden_layers = 5
    ids = torch.randint(3, cfg.vocab_size, (8, 64), generator=torch.Generator().manual_seed(7))
    kw = dict(max_new_tokens=6, min_new_tokens=6, prefill_policy=0, decoding_policy=0)
    ref = lia.OPTForCausalLM(cfg, "cuda").init_weights(seed=5).generate(ids, **kw)
    for pct, kv_res in [(40, None), (0, 2), (100, 1)]:
        m = lia.OPTForCausalLM(cfg, "cuda").init_weights(seed=5, gpu_percentage=pct)
        m.kv_resident_layers = kv_res
        for no_overlap in (True, True, False, True, False):
            tok = m.generate(ids, gpu_percentage=pct, no_overlap=no_overlap, num_minibatch=2, **kw)
            assert torch.equal(tok, ref), (pct, kv_res, no_overlap)
        del m
        torch.cuda.empty_cache()


def test_padded_head_dim_vs_unpadded_oracle(lia):
    """head_dim 80 (opt-2.7b's) runs on the head_dim-128 kernels with zero-padded heads (weights.padded_head_dim): hidden
    states against the oracle on the UNPADDED weights, padded lanes of the cache exactly zero, deterministic tokens."""
    from oracle import opt_ref
    from lia_b200.weights import random_embeddings, random_layer
    H, d = 4, 80
    cfg = lia.OPTConfig(hidden_size=H * d, num_hidden_layers=2, num_attention_heads=H, ffn_dim=4 * H * d, vocab_size=512,
                        max_position_embeddings=96)
    m = lia.OPTForCausalLM(cfg, "cuda").init_weights(seed=4, bias_std=0.02, ln_std=0.05)
    assert (m.layout.d, m.layout.dp, m.layout.hq) == (80, 128, H * 128)
    e = random_embeddings(cfg.vocab_size, cfg.hidden_size, cfg.max_position_embeddings, 4 * 100003 + 17, "cuda", "normal",
                          cfg.init_std, 0.05, cfg.pad_token_id)
    layers = [random_layer(cfg.hidden_size, cfg.ffn_dim, 4 * 100003 + 1000 + i, "cuda", "normal", cfg.init_std, 0.02, 0.05)
              for i in range(cfg.num_hidden_layers)]
    om = {"H": H, "layers": layers, **e}
    assert torch.equal(om["embed_tokens"], m.model.decoder.embed_tokens)
    B, S, new = 4, 40, 6
    ids = torch.randint(3, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(8))
    ones = torch.ones(B, S, dtype=torch.long, device="cuda")
    hidden, past = m.model.decoder(input_ids=ids.cuda(), attention_mask=ones, max_new_tokens=new)
    nxt = torch.randint(3, cfg.vocab_size, (B, 1), generator=torch.Generator().manual_seed(9))
    ones1 = torch.ones(B, S + 1, dtype=torch.long, device="cuda")
    hidden1, past1 = m.model.decoder(input_ids=nxt.cuda(), attention_mask=ones1, past_key_values=past, max_new_tokens=new)
    with torch.no_grad():
        cache = opt_ref.new_cache(om, B, S + new)
        href = opt_ref.decoder_forward(om, ids.cuda(), ones, cache, 0)
        href1 = opt_ref.decoder_forward(om, nxt.cuda(), ones1, cache, S)
    assert rel_err(hidden, href) <= 3 * REL_TOL and rel_err(hidden1, href1) <= 3 * REL_TOL      # chained through 2 layers
    for li in range(cfg.num_hidden_layers):
        k, v = past1[li][1], past1[li][2]
        assert k.shape == (S + new, B, H, 128) and not k[..., d:].any() and not v[..., d:].any()
        assert rel_err(k[:S + 1, ..., :d], cache[li][0][:S + 1]) <= 3 * REL_TOL
        assert rel_err(v[:S + 1, ..., :d], cache[li][1][:S + 1]) <= 3 * REL_TOL
    toks = [m.generate(ids, max_new_tokens=new, min_new_tokens=new, num_minibatch=2).cpu() for _ in range(3)]
    assert torch.equal(toks[0], toks[1]) and torch.equal(toks[1], toks[2])     # eager, graph capture, graph replay
