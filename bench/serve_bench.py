"""Serving throughput of the hybrid step engine (Nezavik) beside the paged-KV transformer engine (Qwen2) at equal size,
plus each new kernel against its roofline and against the like kernel of the transformer path; with ``--serve-model vilosun``
the Vilosun family beside Nezavik (same engine) at equal size, and the kernels it adds beside Nezavik's like kernels; with
``--serve-model damilix`` the Damilix family beside Vilosun in the same way, ``--serve-model lukarax`` the Lukarax family beside Damilix.

Run through ``python bench.py --serve-bench`` (one GPU).  Random weights, synthetic token ids.  End-to-end numbers go
through the engines' public ``generate`` (two runs that differ by `new` generated tokens: the difference is `new` decode steps,
the rest of the shorter run is the prompt pass); kernel numbers are CUDA-event timed after warm-up with inputs larger than L2 where the size allows.
"""
from __future__ import annotations

import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


SMALL = False          # --small: one warm-up and one timed launch per kernel (the target of profiler captures)


def _time(fn, iters=10, warm=3):
    if SMALL:
        iters, warm = 1, 1
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3          # seconds


def nezavik_config(width: int, n_layers: int, vocab: int, window: int = 1024, max_positions: int = 8192):
    from nanorlhf_b200.models.nezavik import NezavikConfig
    H = width // 128
    par = {"type": "parallel", "mlp": {"ff": 4 * width, "kind": "dense"},
           "mixer": {"left": {"dim": 128, "vdim": 128, "heads": H, "kv_heads": max(1, H // 4), "mask": {"size": window},
                              "scale": 128 ** -0.5},
                     "right": {"conv": 4, "groups": 1, "heads": width // 64, "norm_groups": 1, "state": 128, "vdim": 64},
                     "left_scale": 1.0, "right_scale": 1.0}}
    dl = {"type": "delta", "mlp": {"ff": 4 * width, "kind": "dense"},
          "mixer": {"conv": 4, "dim": 128, "vdim": 128, "heads": H, "kv_heads": H}}
    cd = dict(dl, type="channel_delta")
    pattern = [par, dl, cd, par]
    return NezavikConfig.from_dict({"architecture": "Nezavik", "layers": [pattern[i % 4] for i in range(n_layers)],
                                    "max_positions": max_positions, "norm": {"eps": 1e-6}, "vocab": vocab, "width": width})


def vilosun_config(width: int, n_layers: int, vocab: int, chunk: int = 1024, experts: int = 16, top: int = 2):
    """Head sizes 128, a quarter as many key/value heads, layer pattern attention / delta / delta / attention; the `top` active
    experts hold as many weights as the dense 4 x width feed-forward of the model beside it."""
    from nanorlhf_b200.models.vilosun import VilosunConfig
    H = width // 128
    ff = max(128, (8 * width // (3 * top) + 127) // 128 * 128)
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    at = {"type": "attention", "mlp": mlp,
          "mixer": {"conv": 4, "dim": 128, "vdim": 128, "heads": H, "kv_heads": max(1, H // 4), "mask": {"size": chunk},
                    "scale": 128 ** -0.5, "v_mix": True}}
    dl = {"type": "delta", "mlp": mlp, "mixer": {"conv": 4, "dim": 128, "vdim": 128, "heads": H, "kv_heads": H}}
    pattern = [at, dl, dl, at]
    return VilosunConfig.from_dict({"architecture": "Vilosun", "layers": [pattern[i % 4] for i in range(n_layers)],
                                    "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 48271, "mul_cur": 16807}},
                                    "logit_scale": 1.0, "norm": {"eps": 1e-6, "groups": 2}, "vocab": vocab, "width": width})


def _gen_times(gen, prompts, new, base=4):
    """(prefill seconds, seconds per decode step): generate `base` and `base + new` tokens (median of 3 after a warm-up);
    the difference is `new` decode steps, the rest of the shorter run is the prompt pass."""
    out = []
    for mt in (base, base + new):
        ts = []
        for it in range(4):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            gen(prompts, mt)
            torch.cuda.synchronize()
            if it:
                ts.append(time.perf_counter() - t0)
        out.append(sorted(ts)[1])
    step = max(out[1] - out[0], 1e-9) / new
    return max(out[0] - base * step, 1e-9), step


def end_to_end_vilosun(width, n_layers, batch, prompt_len, new=128, vocab=32768):
    """Vilosun beside Nezavik (the closest family: same engine, attention + delta-rule layers) at equal width and depth."""
    from nanorlhf_b200.models.nezavik import NezavikForCausalLM
    from nanorlhf_b200.models.vilosun import VilosunForCausalLM
    from nanorlhf_b200.sampler.hybrid_sampler import HybridSampler
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, vocab - 2, (batch, prompt_len), generator=g).tolist()
    res = {"width": width, "layers": n_layers, "batch": batch, "prompt_len": prompt_len, "new_tokens": new}
    for name, make in (("vilosun", lambda: VilosunForCausalLM.from_config(vilosun_config(width, n_layers, vocab), torch.bfloat16, dev, seed=0)),
                       ("nezavik", lambda: NezavikForCausalLM.from_config(nezavik_config(width, n_layers, vocab), torch.bfloat16, dev, seed=0, rank=64))):
        model = make()
        eng = HybridSampler(model, dtype="bf16", max_num_seqs=batch, prefill_token_budget=16384)
        pre, step = _gen_times(lambda p, mt: eng.generate(p, 1, 1.0, 1.0, mt, None, vocab - 1, 1), prompts, new)
        res[name] = {"params_m": round(sum(p.numel() for p in model.parameters()) / 1e6, 1),
                     "prefill_tok_s": round(batch * prompt_len / pre), "decode_tok_s": round(batch / step),
                     "decode_ms_per_step": round(step * 1e3, 3)}
        eng.release()
        del eng, model
        torch.cuda.empty_cache()
    return res


def kernels_vilosun(width=2048, batch=16, prompt_len=2048, chunk=1024, decode_batch=256, ctx=2048, experts=16, top=2):
    """The kernels Vilosun adds to the step engine, each beside the like kernel of the Nezavik path."""
    from nanorlhf_b200 import _C
    from nanorlhf_b200.ops import hybrid as hy
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    hbm, flops_peak, which = _peaks()
    dev = torch.device("cuda:0")
    out = {"roofline": which, "width": width}
    H, Hkv, D = width // 128, max(1, width // 512), 128
    ff = max(128, (8 * width // (3 * top) + 127) // 128 * 128)

    def plan_for(B, n_new, n_old):
        s = _C.StepScheduler((n_old + n_new + 15) // 16 * B + 8, 16, B)
        sids = [s.open() for _ in range(B)]
        if n_old:
            s.plan(sids, [n_old] * B)
        data, E, T, MB = s.plan(sids, [n_new] * B)
        return StepPlan(torch.from_numpy(data).to(dev), E, T, MB), s

    def report(name, sec, bytes_, flops=0.0):
        floor = max(bytes_ / hbm, flops / flops_peak)
        out[name] = {"us": round(sec * 1e6, 1), "gb_s": round(bytes_ / sec / 1e9, 1), "tflop_s": round(flops / sec / 1e12, 2),
                     "roofline_frac": round(floor / sec, 3)}

    for phase, B, n_new, n_old in (("prefill", batch, prompt_len, 0), ("decode", decode_batch, 1, ctx - 1)):
        plan, sched = plan_for(B, n_new, n_old)
        T = plan.T
        f32 = dict(dtype=torch.float32, device=dev)
        plan.tokens.copy_(torch.randint(0, 32000, (T,), dtype=torch.int32, device=dev))
        # -- embeddings
        emb, pair = torch.randn(32768, width, device=dev).bfloat16(), torch.randn(65522, width, device=dev).bfloat16()
        prev, x0 = torch.zeros(B, dtype=torch.int32, device=dev), torch.empty(T, width, **f32)
        sec = _time(lambda: hy.embed_hashed(emb, pair, plan, prev, 1.0, 48271, 16807, 65521, x0))
        report(f"{phase}.embed_hashed", sec, T * width * 8.0)
        pos_t = torch.randn(8192, width, device=dev).bfloat16()
        sec = _time(lambda: hy.embed_pos(emb, pos_t, plan.tokens, plan.pos, x0))
        report(f"{phase}.nezavik.embed_pos", sec, T * width * 8.0)
        # -- sublayer boundary: gate, post-norm, residual, next pre-norm vs the depth-weighted boundary at depth 1
        x, o, gate = torch.randn(T, width, **f32), torch.randn(T, width, **f32), torch.randn(T, width, **f32)
        gb, wa, wb = torch.randn(width, **f32), torch.ones(width, **f32), torch.ones(width, **f32)
        h = torch.empty(T, width, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.group_norm_residual(x, o, gate, gb, wa, wb, 2, 1e-6, h))
        report(f"{phase}.group_norm_residual", sec, T * width * (4.0 * 4 + 2))
        results = torch.randn(2, T, width, **f32)
        xc, dw, gain = torch.empty(T, width, **f32), torch.rand(2, **f32), torch.ones(1, **f32)
        sec = _time(lambda: hy.stream_norm(results, 1, o, x, dw, gain, 1e-6, xc, h, T))
        report(f"{phase}.nezavik.stream_norm(depth 1)", sec, T * width * (4.0 * 5 + 2))
        # -- attention: convolution, page write, chunked attention vs q/k norm + page write, sliding-window attention
        nq, nk = H * D, Hkv * D
        raw, cw, cb = torch.randn(T, nq + 2 * nk, **f32), torch.randn(nq + 2 * nk, 4, **f32), torch.randn(nq + 2 * nk, **f32)
        cst, qkv = torch.zeros(B, 3, nq + 2 * nk, **f32), torch.empty(T, nq + 2 * nk, **f32)
        sec = _time(lambda: hy.causal_conv(raw, cw, None, cst, qkv, plan, in_bias=cb, act="none"))
        report(f"{phase}.causal_conv(qkv, biased)", sec, T * (nq + 2 * nk) * 8.0 + B * 3 * (nq + 2 * nk) * 8.0)
        kc = torch.randn(sched.num_free_blocks() + plan.max_blocks * B + 8, Hkv, 16, D, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        q, k, v = qkv[:, :nq], qkv[:, nq:nq + nk], qkv[:, nq + nk:]
        vo, lam = torch.randn(T, nk, **f32), torch.full((1,), 0.3, **f32)
        sec = _time(lambda: hy.kv_write_blend(k, v, vo, lam, kc, vc, plan))
        report(f"{phase}.kv_write_blend", sec, T * nk * (4.0 * 4 + 2 * 2))
        qw_, kw_ = torch.ones(D, **f32), torch.ones(D, **f32)
        sec = _time(lambda: hy.qknorm_kv_write(q, k, v, qw_, kw_, 1e-6, kc, vc, plan))
        report(f"{phase}.nezavik.qknorm_kv_write", sec, T * (H + 2 * Hkv) * D * 4.0 + T * H * D * 4.0 + T * 2 * Hkv * D * 2.0)
        ao = torch.empty(T, H * D, dtype=torch.bfloat16, device=dev)
        temp, slope, hg = torch.rand(H, **f32) + 0.5, torch.rand(H, **f32) * 0.1, torch.randn(T, H, **f32)
        if phase == "prefill":
            keys_c = sum(p % chunk + 1 for p in range(n_new)) * B
            keys_w = sum(min(p + 1, chunk) for p in range(n_new)) * B
        else:
            keys_c, keys_w = ((ctx - 1) % chunk + 1) * B, min(ctx, chunk) * B
        byt = lambda keys: (T * H * D * 6.0 + T * 2 * Hkv * D * 2.0) if phase == "prefill" else (keys * 2 * Hkv * D * 2.0 + T * H * D * 6.0)
        sec = _time(lambda: hy.window_attention(q, kc, vc, plan, chunk, D ** -0.5, 1.0, ao, chunked=True, head_scale=temp,
                                                head_slope=slope, gate=hg), iters=3, warm=1)
        report(f"{phase}.chunk_attention(c={chunk})", sec, byt(keys_c), flops=4.0 * keys_c * H * D)
        sec = _time(lambda: hy.window_attention(q, kc, vc, plan, chunk, D ** -0.5, 1.0, ao), iters=3, warm=1)
        report(f"{phase}.nezavik.window_attention(w={chunk})", sec, byt(keys_w), flops=4.0 * keys_w * H * D)
        del kc, vc
        # -- feed-forward: routing + expert activations vs the dense squared-ReLU activation
        U = torch.randn(T, experts + experts * 2 * ff, **f32)
        A = torch.empty(T, experts * ff, dtype=torch.bfloat16, device=dev)
        rb = torch.zeros(experts, **f32)
        sec = _time(lambda: hy.moe_route(U[:, :experts], rb, top, gu=U[:, experts:], ff=ff, act=A))
        report(f"{phase}.moe_route(dense form, {experts} experts top {top})", sec, T * (experts * 4.0 + top * ff * 8.0 + experts * ff * 2.0))
        ids_, wts_ = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, **f32)
        sec = _time(lambda: hy.moe_route(U[:, :experts], rb, top, ids=ids_, wts=wts_))
        report(f"{phase}.moe_route(ids and weights only)", sec, T * (experts * 4.0 + top * 8.0))
        up = torch.randn(T, 4 * width, **f32)
        ub = torch.empty(T, 4 * width, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.act_cols(up, ub, "relu2"))
        report(f"{phase}.nezavik.relu2", sec, T * 4 * width * 6.0)
        del U, A, up, ub
        # -- the experts on the grouped GEMM (routing plan, gather, two grouped GEMMs, SwiGLU, combine) vs the dense pair of GEMMs
        #    of a feed-forward with as many active weights (4 x width, squared ReLU)
        from nanorlhf_b200.ops import gemm as _gemm
        hb_ = torch.randn(T, width, device=dev).bfloat16()
        zr = torch.randn(T, experts, **f32)
        ids, wts = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, **f32)
        hy.moe_route(zr, None, top, ids=ids, wts=wts)
        wgu = (torch.randn(experts * 2 * ff, width, device=dev) * width ** -0.5).bfloat16()
        wdn = (torch.randn(experts * width, ff, device=dev) * ff ** -0.5).bfloat16()
        yo = torch.empty(T, width, **f32)
        sec = _time(lambda: hy.moe_grouped_ffn(hb_, ids, wts, wgu, wdn, experts, ff, yo, fused_act=ff % 32 == 0), iters=5, warm=2)
        active = min(experts, T * top)                     # experts whose weights a step has to read
        wbytes = active * 3.0 * ff * width * 2.0
        report(f"{phase}.moe_grouped_ffn({experts} experts top {top}, ff {ff})", sec, wbytes + T * width * 6.0, flops=6.0 * T * top * width * ff)
        w1 = (torch.randn(4 * width, width, device=dev) * width ** -0.5).bfloat16()
        w2 = (torch.randn(width, 4 * width, device=dev) * (4 * width) ** -0.5).bfloat16()
        u1, a1, o1 = torch.empty(T, 4 * width, **f32), torch.empty(T, 4 * width, dtype=torch.bfloat16, device=dev), torch.empty(T, width, **f32)

        def dense_ffn():
            _gemm.gemm(hb_, w1, out_f32=u1)
            hy.act_cols(u1, a1, "relu2")
            _gemm.gemm(a1, w2, out_f32=o1)
        sec = _time(dense_ffn, iters=5, warm=2)
        report(f"{phase}.nezavik.dense_ffn(4 x width)", sec, 8.0 * width * width * 2.0 + T * width * 6.0, flops=16.0 * T * width * width)
    return out


def damilix_config(width: int, n_layers: int, vocab: int, experts: int = 16, top: int = 2, kv_rank: int = 256, rot_dim: int = 64):
    """Heads of 128 (unrotated) + `rot_dim` (rotated) query columns over a latent of `kv_rank` columns, gated linear attention with
    128 x 128 states, layer pattern latent / gla / gla / latent (second rotation layout); experts as in ``vilosun_config`` plus two
    identity experts and a shared expert of the same width; a token input of 64 columns per layer."""
    from nanorlhf_b200.models.damilix import DamilixConfig
    H = width // 128
    ff = max(128, (8 * width // (3 * top) + 127) // 128 * 128)
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": 2, "top": top, "scale": 1.5}, "shared": {"ff": ff}}
    rot = {"base": 1e6, "dims": rot_dim}
    la = {"type": "latent_attention", "mlp": mlp,
          "mixer": {"heads": H, "dim": 128, "rot_dim": rot_dim, "vdim": 128, "kv_rank": kv_rank, "scale": (128 + rot_dim) ** -0.5,
                    "rot": dict(rot, scaling={"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0})}}
    lb = {"type": "latent_attention_2", "mlp": mlp, "mixer": dict(la["mixer"], rot=rot)}
    gl = {"type": "gla", "mlp": mlp, "mixer": {"heads": H, "dim": 128, "vdim": 128, "tau": 16.0}}
    pattern = [la, gl, gl, lb]
    return DamilixConfig.from_dict({"architecture": "Damilix", "layers": [pattern[i % 4] for i in range(n_layers)], "norm": {"eps": 1e-6},
                                    "token_side": {"dim": 64}, "vocab": vocab, "width": width})


def end_to_end_damilix(width, n_layers, batch, prompt_len, new=128, vocab=32768):
    """Damilix beside Vilosun (the closest family: same engine, attention + recurrent layers, mixture-of-experts feed-forwards) at
    equal width, depth and expert sizes."""
    from nanorlhf_b200.models.damilix import DamilixForCausalLM
    from nanorlhf_b200.models.vilosun import VilosunForCausalLM
    from nanorlhf_b200.sampler.hybrid_sampler import HybridSampler
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, vocab - 2, (batch, prompt_len), generator=g).tolist()
    res = {"width": width, "layers": n_layers, "batch": batch, "prompt_len": prompt_len, "new_tokens": new}
    for name, make in (("damilix", lambda: DamilixForCausalLM.from_config(damilix_config(width, n_layers, vocab), torch.bfloat16, dev, seed=0, gla_rank=64)),
                       ("vilosun", lambda: VilosunForCausalLM.from_config(vilosun_config(width, n_layers, vocab), torch.bfloat16, dev, seed=0))):
        model = make()
        eng = HybridSampler(model, dtype="bf16", max_num_seqs=batch, prefill_token_budget=16384)
        pre, step = _gen_times(lambda p, mt: eng.generate(p, 1, 1.0, 1.0, mt, None, vocab - 1, 1), prompts, new)
        res[name] = {"params_m": round(sum(p.numel() for p in model.parameters()) / 1e6, 1),
                     "prefill_tok_s": round(batch * prompt_len / pre), "decode_tok_s": round(batch / step),
                     "decode_ms_per_step": round(step * 1e3, 3)}
        eng.release()
        del eng, model
        torch.cuda.empty_cache()
    return res


def kernels_damilix(width=2048, batch=16, prompt_len=2048, decode_batch=256, ctx=2048, experts=16, top=2, kv_rank=256, rot_dim=64):
    """The kernels Damilix adds to the step engine, each beside the like kernel of the Vilosun path."""
    from nanorlhf_b200 import _C
    from nanorlhf_b200.ops import hybrid as hy
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    hbm, flops_peak, which = _peaks()
    dev = torch.device("cuda:0")
    out = {"roofline": which, "width": width}
    H, Hkv, D = width // 128, max(1, width // 512), 128
    DL = kv_rank + rot_dim
    ff = max(128, (8 * width // (3 * top) + 127) // 128 * 128)

    def plan_for(B, n_new, n_old):
        s = _C.StepScheduler((n_old + n_new + 15) // 16 * B + 8, 16, B)
        sids = [s.open() for _ in range(B)]
        if n_old:
            s.plan(sids, [n_old] * B)
        data, E, T, MB = s.plan(sids, [n_new] * B)
        return StepPlan(torch.from_numpy(data).to(dev), E, T, MB), s

    def report(name, sec, bytes_, flops=0.0):
        floor = max(bytes_ / hbm, flops / flops_peak)
        out[name] = {"us": round(sec * 1e6, 1), "gb_s": round(bytes_ / sec / 1e9, 1), "tflop_s": round(flops / sec / 1e12, 2),
                     "roofline_frac": round(floor / sec, 3)}

    for phase, B, n_new, n_old in (("prefill", batch, prompt_len, 0), ("decode", decode_batch, 1, ctx - 1)):
        plan, sched = plan_for(B, n_new, n_old)
        T = plan.T
        f32 = dict(dtype=torch.float32, device=dev)
        plan.tokens.copy_(torch.randint(0, 32000, (T,), dtype=torch.int32, device=dev))
        # -- embedding: normed rows vs scaled rows + hashed pair rows
        emb, pair = torch.randn(32768, width, device=dev).bfloat16(), torch.randn(65522, width, device=dev).bfloat16()
        x0, h = torch.empty(T, width, **f32), torch.empty(T, width, dtype=torch.bfloat16, device=dev)
        wa, wb = torch.ones(width, **f32), torch.ones(width, **f32)
        sec = _time(lambda: hy.embed_norm(emb, plan.tokens, wa, 1e-6, x0, h))
        report(f"{phase}.embed_norm", sec, T * width * 8.0)
        prev = torch.zeros(B, dtype=torch.int32, device=dev)
        sec = _time(lambda: hy.embed_hashed(emb, pair, plan, prev, 1.0, 48271, 16807, 65521, x0))
        report(f"{phase}.vilosun.embed_hashed", sec, T * width * 8.0)
        # -- sublayer boundary: norm of the result + residual add + operand cast vs gate, post-norm, residual, pre-norm
        x, o, gate = torch.randn(T, width, **f32), torch.randn(T, width, **f32), torch.randn(T, width, **f32)
        sw, gb = torch.rand(T, **f32), torch.randn(width, **f32)
        sec = _time(lambda: hy.post_norm_residual(x, o, sw, wa, None, 1e-6, h))
        report(f"{phase}.post_norm_residual", sec, T * width * (4.0 * 3 + 2))
        sec = _time(lambda: hy.group_norm_residual(x, o, gate, gb, wa, wb, 2, 1e-6, h))
        report(f"{phase}.vilosun.group_norm_residual", sec, T * width * (4.0 * 4 + 2))
        # -- token input gate and the shared expert's gated SwiGLU vs the squared-ReLU activation
        u = torch.randn(T, 64, **f32)
        table = torch.randn(32768, 8 * 64, device=dev).bfloat16()
        sg_out = torch.empty(T, 64, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.side_gate(u, table, 128, plan.tokens, sg_out, 64))
        report(f"{phase}.side_gate", sec, T * 64 * (4.0 + 2 + 2))
        gu, rg = torch.randn(T, 2 * ff, **f32), torch.randn(T, 1, **f32)
        act = torch.empty(T, ff, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.swiglu_cols(gu, rg, act))
        report(f"{phase}.swiglu_cols(row gate)", sec, T * ff * (8.0 + 2))
        up, ub = torch.randn(T, 2 * ff, **f32), torch.empty(T, 2 * ff, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.act_cols(up, ub, "relu2"))
        report(f"{phase}.nezavik.relu2", sec, T * 2 * ff * 6.0)
        del gu, up, ub, act
        # -- routing
        zr, corr = torch.randn(T, experts + 2, **f32), torch.randn(experts + 2, **f32) * 0.01
        ids, wts, selfw = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, **f32), torch.empty(T, **f32)
        sec = _time(lambda: hy.moe_route_all(zr, corr, experts, top, 1.5, ids=ids, wts=wts, self_w=selfw))
        report(f"{phase}.moe_route_all(ids and weights)", sec, T * ((experts + 2) * 4.0 + top * 8.0 + 4.0))
        sec = _time(lambda: hy.moe_route(zr[:, :experts], corr[:experts], top, ids=ids, wts=wts))
        report(f"{phase}.vilosun.moe_route(ids and weights)", sec, T * (experts * 4.0 + top * 8.0))
        # -- latent attention: cache write + rotation, attention over the latent rows vs page write, chunk attention
        q = torch.randn(T, H * (128 + rot_dim), **f32)
        dkv, nw = torch.randn(T, DL, **f32), torch.ones(kv_rank, **f32)
        fr, mult = hy.rotary_frequencies(rot_dim, 1e6, {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0})
        freq = torch.tensor(fr, dtype=torch.float64, device=dev)
        n_pages = sched.num_free_blocks() + plan.max_blocks * B + 8
        lc = torch.randn(n_pages, 1, 16, DL, device=dev).bfloat16()
        qa = torch.randn(T, H * DL, **f32)
        sec = _time(lambda: hy.latent_kv_write(q, H, 128, rot_dim, dkv, nw, 1e-6, freq, rot_dim, mult, True, plan, lc, qa))
        report(f"{phase}.latent_kv_write", sec, T * (DL * 4.0 + DL * 2.0 + H * rot_dim * 8.0))
        nq, nk = H * D, Hkv * D
        kc = torch.randn(n_pages, Hkv, 16, D, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        k_, v_, vo, lam = torch.randn(T, nk, **f32), torch.randn(T, nk, **f32), torch.randn(T, nk, **f32), torch.full((1,), 0.3, **f32)
        sec = _time(lambda: hy.kv_write_blend(k_, v_, vo, lam, kc, vc, plan))
        report(f"{phase}.vilosun.kv_write_blend", sec, T * nk * (4.0 * 4 + 2 * 2))
        sink, hg = torch.randn(H, **f32), torch.randn(T, H, **f32)
        lat = torch.empty(T, H * kv_rank, dtype=torch.bfloat16, device=dev)
        keys = (sum(p + 1 for p in range(n_new)) if phase == "prefill" else ctx) * B
        byt = (T * H * DL * 4.0 + T * H * kv_rank * 2.0 + T * DL * 2.0) if phase == "prefill" else (keys * DL * 2.0 + T * H * (DL * 4.0 + kv_rank * 2.0))
        it, wm = (3, 1) if phase == "prefill" else (20, 5)
        sec = _time(lambda: hy.window_attention(qa, lc, lc, plan, 1 << 30, 0.07, 1.0, lat, gate=hg, head_sink=sink, value_size=kv_rank), iters=it, warm=wm)
        report(f"{phase}.latent_attention(row {DL}, value {kv_rank})", sec, byt, flops=2.0 * keys * H * (DL + kv_rank))
        qv = torch.randn(T, nq, **f32)
        ao = torch.empty(T, nq, dtype=torch.bfloat16, device=dev)
        temp, slope = torch.rand(H, **f32) + 0.5, torch.rand(H, **f32) * 0.1
        chunk = 1024
        keys_c = (sum(p % chunk + 1 for p in range(n_new)) if phase == "prefill" else ((ctx - 1) % chunk + 1)) * B
        byt_c = (T * H * D * 6.0 + T * 2 * Hkv * D * 2.0) if phase == "prefill" else (keys_c * 2 * Hkv * D * 2.0 + T * H * D * 6.0)
        sec = _time(lambda: hy.window_attention(qv, kc, vc, plan, chunk, D ** -0.5, 1.0, ao, chunked=True, head_scale=temp,
                                                head_slope=slope, gate=hg), iters=it, warm=wm)
        report(f"{phase}.vilosun.chunk_attention(c={chunk})", sec, byt_c, flops=4.0 * keys_c * H * D)
        del kc, vc, lc, qa, lat
        # -- gated linear attention vs the gated delta rule (same state size)
        nkk = H * D
        qkv = torch.randn(T, 3 * nkk, **f32) * 0.1
        z, ab = torch.randn(T, nkk, **f32), torch.full((nkk,), 3.0, **f32)
        decay, og = torch.empty(T, nkk, **f32), torch.empty(T, nkk, **f32)
        state = torch.zeros(B, H, D, D, **f32)
        sec = _time(lambda: hy.gla_prep(qkv, z, ab, 16.0, decay, H, D))
        report(f"{phase}.gla_prep", sec, T * nkk * 16.0)
        sec = _time(lambda: hy.delta_scan(qkv, nkk, 2 * nkk, None, decay, state, og, plan, H, True), iters=3, warm=1)
        sbytes = B * H * D * D * 8.0 + T * nkk * 20.0
        report(f"{phase}.gla_scan", sec, sbytes, flops=0.0)
        out[f"{phase}.gla_scan"]["fp32_fma_frac"] = round(4.0 * T * H * D * D / sec / 72e12, 3)
        beta = torch.rand(T, H, **f32)
        sec = _time(lambda: hy.delta_scan(qkv, nkk, 2 * nkk, beta, decay, state, og, plan, H, True), iters=3, warm=1)
        report(f"{phase}.vilosun.delta_scan(per channel)", sec, sbytes)
        out[f"{phase}.vilosun.delta_scan(per channel)"]["fp32_fma_frac"] = round(6.0 * T * H * D * D / sec / 72e12, 3)
    return out


def lukarax_config(width: int, n_layers: int, vocab: int, experts: int = 16, top: int = 2, streams: int = 4):
    """Heads of 128 columns, four query heads per key/value head; layer pattern parallel (windowed attention with kept first keys and
    a distance bias beside a matrix memory with 128 x 128 states) / attention_2 / attention / attention reading the pages of the
    layer before; experts as in ``damilix_config`` (two identity experts, groups of neighbours, no shared expert)."""
    from nanorlhf_b200.models.lukarax import LukaraxConfig
    H = width // 128
    G = max(1, H // 4)
    ff = max(128, (8 * width // (3 * top) + 127) // 128 * 128)
    n_out = experts + 2
    groups = next(g for g in (6, 4, 3, 2, 1) if n_out % g == 0)
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": 2, "top": top, "scale": 1.5,
                                                             "groups": {"count": groups, "keep": max(1, groups // 2)}}}
    par = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": {"heads": H // 2, "kv_heads": max(1, G // 2), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "bias_max": 2048,
                              "mask": {"size": 1024, "keep_first": 64}},
                     "right": {"heads": H // 2, "dim": 128, "vdim": 128, "gate_cap": 15.0}, "left_scale": 0.7, "right_scale": 1.0}}
    a2 = {"type": "attention_2", "mlp": mlp,
          "mixer": {"heads": H, "kv_heads": G, "dim": 128, "vdim": 128, "scale": 1.0, "softcap": 50.0, "mask": {"size": 1024},
                    "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    da = {"type": "attention", "mlp": mlp,
          "mixer": {"heads": H // 2, "kv_heads": max(1, G // 2), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "diff": 0.2,
                    "rot": {"base": 1e6, "dims": 128}}}
    layers = []
    for i in range(n_layers):
        layer = json.loads(json.dumps([par, a2, da, da][i % 4]))
        if i % 4 == 3:
            layer["mixer"]["kv_from"] = i - 1
        layers.append(layer)
    return LukaraxConfig.from_dict({"architecture": "Lukarax", "layers": layers, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
                                    "streams": streams, "vocab": vocab, "width": width})


def end_to_end_lukarax(width, n_layers, batch, prompt_len, new=128, vocab=32768):
    """Lukarax beside Damilix (the closest family: same engine, attention + recurrent layers, routed experts with identity experts)
    at equal width, depth and expert sizes."""
    from nanorlhf_b200.models.damilix import DamilixForCausalLM
    from nanorlhf_b200.models.lukarax import LukaraxForCausalLM
    from nanorlhf_b200.sampler.hybrid_sampler import HybridSampler
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, vocab - 2, (batch, prompt_len), generator=g).tolist()
    res = {"width": width, "layers": n_layers, "batch": batch, "prompt_len": prompt_len, "new_tokens": new}
    for name, make in (("lukarax", lambda: LukaraxForCausalLM.from_config(lukarax_config(width, n_layers, vocab), torch.bfloat16, dev, seed=0)),
                       ("damilix", lambda: DamilixForCausalLM.from_config(damilix_config(width, n_layers, vocab), torch.bfloat16, dev, seed=0, gla_rank=64))):
        model = make()
        eng = HybridSampler(model, dtype="bf16", max_num_seqs=batch, prefill_token_budget=16384)
        pre, step = _gen_times(lambda p, mt: eng.generate(p, 1, 1.0, 1.0, mt, None, vocab - 1, 1), prompts, new)
        res[name] = {"params_m": round(sum(p.numel() for p in model.parameters()) / 1e6, 1),
                     "prefill_tok_s": round(batch * prompt_len / pre), "decode_tok_s": round(batch / step),
                     "decode_ms_per_step": round(step * 1e3, 3)}
        eng.release()
        del eng, model
        torch.cuda.empty_cache()
    return res


def kernels_lukarax(width=2048, batch=16, prompt_len=2048, decode_batch=256, ctx=2048, experts=16, top=2, streams=4, window=1024):
    """The kernels Lukarax adds to the step engine, each beside the like kernel of the Damilix / Vilosun / Nezavik paths."""
    from nanorlhf_b200 import _C
    from nanorlhf_b200.ops import hybrid as hy
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    hbm, flops_peak, which = _peaks()
    dev = torch.device("cuda:0")
    out = {"roofline": which, "width": width}
    H, Hkv, D = width // 128, max(1, width // 512), 128

    def plan_for(B, n_new, n_old):
        s = _C.StepScheduler((n_old + n_new + 15) // 16 * B + 8, 16, B)
        sids = [s.open() for _ in range(B)]
        if n_old:
            s.plan(sids, [n_old] * B)
        data, E, T, MB = s.plan(sids, [n_new] * B)
        return StepPlan(torch.from_numpy(data).to(dev), E, T, MB), s

    def report(name, sec, bytes_, flops=0.0):
        floor = max(bytes_ / hbm, flops / flops_peak)
        out[name] = {"us": round(sec * 1e6, 1), "gb_s": round(bytes_ / sec / 1e9, 1), "tflop_s": round(flops / sec / 1e12, 2),
                     "roofline_frac": round(floor / sec, 3)}

    for phase, B, n_new, n_old in (("prefill", batch, prompt_len, 0), ("decode", decode_batch, 1, ctx - 1)):
        plan, sched = plan_for(B, n_new, n_old)
        T = plan.T
        f32 = dict(dtype=torch.float32, device=dev)
        plan.tokens.copy_(torch.randint(0, 32000, (T,), dtype=torch.int32, device=dev))
        # -- embedding into every stream vs the normed embedding
        emb = torch.randn(32768, width, device=dev).bfloat16()
        xs, h = torch.empty(T, streams, width, **f32), torch.empty(T, width, dtype=torch.bfloat16, device=dev)
        x0, wa, wb = torch.empty(T, width, **f32), torch.ones(width, **f32), torch.zeros(width, **f32)
        sec = _time(lambda: hy.embed_streams(emb, plan.tokens, 2.0, xs))
        report(f"{phase}.embed_streams(S={streams})", sec, T * width * (2.0 + 4.0 * streams))
        sec = _time(lambda: hy.embed_norm(emb, plan.tokens, wa, 1e-6, x0, h))
        report(f"{phase}.damilix.embed_norm", sec, T * width * 8.0)
        # -- sublayer boundary over S streams (read and write all of them) vs one stream
        o, sw, ob = torch.randn(T, width, **f32), torch.rand(T, **f32), torch.randn(width, **f32)
        mix, ow, iw = torch.eye(streams, **f32) + 0.1, torch.ones(streams, **f32), torch.full((streams,), 0.3, **f32)
        xs.normal_()
        sec = _time(lambda: hy.hyper_boundary(xs, o, ob, sw, mix, ow, iw, wa, wb, 1e-6, h))
        report(f"{phase}.hyper_boundary(S={streams})", sec, T * width * (8.0 * streams + 4.0 + 2.0 * 2))
        x = torch.randn(T, width, **f32)
        sec = _time(lambda: hy.post_norm_residual(x, o, sw, wa, None, 1e-6, h))
        report(f"{phase}.damilix.post_norm_residual", sec, T * width * (4.0 * 3 + 2))
        del xs, x, o
        # -- routing with and without groups
        zr, corr = torch.randn(T, experts + 2, **f32), torch.randn(experts + 2, **f32) * 0.01
        ids, wts, selfw = torch.empty(T, top, dtype=torch.int32, device=dev), torch.empty(T, top, **f32), torch.empty(T, **f32)
        groups = next(g for g in (6, 4, 3, 2, 1) if (experts + 2) % g == 0)
        rb = T * ((experts + 2) * 4.0 + top * 8.0 + 4.0)
        sec = _time(lambda: hy.moe_route_all(zr, corr, experts, top, 1.5, ids=ids, wts=wts, self_w=selfw, groups=groups, keep=max(1, groups // 2)))
        report(f"{phase}.moe_route_all(groups={groups})", sec, rb)
        sec = _time(lambda: hy.moe_route_all(zr, corr, experts, top, 1.5, ids=ids, wts=wts, self_w=selfw))
        report(f"{phase}.damilix.moe_route_all", sec, rb)
        # -- write side: bias + rotation + unit norm + pages vs q / k norm + pages
        n_pages = sched.num_free_blocks() + plan.max_blocks * B + 8
        nq, nk = H * D, Hkv * D
        q, k_, v_ = torch.randn(T, nq, **f32), torch.randn(T, nk, **f32), torch.randn(T, nk, **f32)
        qb, kb = torch.randn(nq, **f32), torch.randn(nk, **f32)
        kc = torch.randn(n_pages, Hkv, 16, D, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        fr, mult = hy.rotary_frequencies(64, 1e6, {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0})
        freq = torch.tensor(fr, dtype=torch.float64, device=dev)
        sec = _time(lambda: hy.rot_kv_write(q, qb, k_, kb, None, freq, 64, mult, False, True, None, None, 1e-6, plan, kc, vc))
        report(f"{phase}.rot_kv_write(values = keys)", sec, T * (nq * 8.0 + nk * (4.0 + 4.0)))
        sec = _time(lambda: hy.rot_kv_write(q, None, k_, None, v_, freq, 64, mult, True, False, None, None, 1e-6, plan, kc, vc))
        report(f"{phase}.rot_kv_write(q, k, v)", sec, T * (nq * 8.0 + nk * (8.0 + 4.0)))
        sec = _time(lambda: hy.qknorm_kv_write(q, k_, v_, torch.ones(D, **f32), torch.ones(D, **f32), 1e-6, kc, vc, plan))
        report(f"{phase}.nezavik.qknorm_kv_write", sec, T * (nq * 8.0 + nk * (8.0 + 4.0)))
        # -- attention forms
        q.normal_()
        ao = torch.empty(T, nq, dtype=torch.bfloat16, device=dev)
        it, wm = (3, 1) if phase == "prefill" else (20, 5)
        sink = torch.randn(H, **f32)
        keys_w = (sum(min(p + 1, window) for p in range(n_new)) if phase == "prefill" else min(ctx, window)) * B
        byt_w = (T * H * D * 6.0 + T * 2 * Hkv * D * 2.0) if phase == "prefill" else (keys_w * 2 * Hkv * D * 2.0 + T * H * D * 6.0)
        sec = _time(lambda: hy.window_attention(q, kc, vc, plan, window, 1.0, 1.0, ao, head_sink=sink, softcap=50.0), iters=it, warm=wm)
        report(f"{phase}.attention(window {window}, cap, sink)", sec, byt_w, flops=4.0 * keys_w * H * D)
        table = torch.randn(2049, H, **f32) * 0.1
        keys_k = keys_w + (sum(min(64, max(0, p + 1 - window)) for p in range(n_new)) if phase == "prefill" else min(64, max(0, ctx - window))) * B
        sec = _time(lambda: hy.window_attention(q, kc, vc, plan, window, D ** -0.5, 1.0, ao, keep_first=64, dist_bias=table), iters=it, warm=wm)
        report(f"{phase}.attention(window {window}, kept 64, distance bias)", sec, byt_w * keys_k / keys_w if phase == "decode" else byt_w,
               flops=4.0 * keys_k * H * D)
        sec = _time(lambda: hy.window_attention(q, kc, vc, plan, window, D ** -0.5, 1.0, ao), iters=it, warm=wm)
        report(f"{phase}.nezavik.window_attention(window {window})", sec, byt_w, flops=4.0 * keys_w * H * D)
        # two score maps over shared values: twice the query and key heads, one set of values
        kc2 = torch.randn(n_pages, 2 * Hkv, 16, D, device=dev).bfloat16()
        a2 = torch.empty(T, 2 * H * D, dtype=torch.bfloat16, device=dev)
        q2 = torch.randn(T, 2 * nq, **f32)
        keys_c = (sum(p + 1 for p in range(n_new)) if phase == "prefill" else ctx) * B
        byt_c = (T * 2 * H * D * 6.0 + T * 3 * Hkv * D * 2.0) if phase == "prefill" else (keys_c * 3 * Hkv * D * 2.0 + T * 2 * H * D * 6.0)
        sec = _time(lambda: hy.window_attention(q2, kc2, vc, plan, 1 << 30, D ** -0.5, 1.0, a2, v_div=2), iters=it, warm=wm)
        report(f"{phase}.attention(causal, two maps, shared values)", sec, byt_c, flops=4.0 * keys_c * 2 * H * D)
        kc1 = torch.randn(n_pages, 2 * Hkv, 16, D, device=dev).bfloat16()
        sec = _time(lambda: hy.window_attention(q2, kc2, kc1, plan, 1 << 30, D ** -0.5, 1.0, a2), iters=it, warm=wm)
        report(f"{phase}.nezavik.window_attention(causal, twice the heads)", sec, byt_c + (T if phase == "prefill" else keys_c) * Hkv * D * 2.0,
               flops=4.0 * keys_c * 2 * H * D)
        gate = torch.randn(T, nq, **f32)
        sec = _time(lambda: hy.diff_combine(a2, 0.4, 0.7, 1e-6, gate, 1.0, ao, H, Hkv))
        report(f"{phase}.diff_combine", sec, T * nq * (4.0 + 4.0 + 2.0))
        del kc, vc, kc2, kc1, a2, q2
        # -- matrix memory vs gated linear attention (same state size) and their read-out norms
        nkk = H * D
        U = torch.randn(T, 3 * nkk + 2 * H, **f32) * 0.1
        state, mst = torch.zeros(B, H, D, D + 8, **f32), torch.zeros(B, H, **f32)
        om, mo = torch.empty(T, H * (D + 1), **f32), torch.empty(T, H, **f32)
        ib = torch.zeros(H, **f32)
        sec = _time(lambda: hy.mlstm_scan(U, 0, nkk, 2 * nkk, 3 * nkk, 3 * nkk + H, ib, ib, 15.0, D ** -0.5, state, mst, om, mo, plan), iters=3, warm=1)
        sbytes = B * H * D * D * 8.0 + T * nkk * 16.0
        report(f"{phase}.mlstm_scan", sec, sbytes)
        out[f"{phase}.mlstm_scan"]["fp32_fma_frac"] = round(4.0 * T * H * D * (D + 1) / sec / 72e12, 3)
        nw = torch.ones(nkk, **f32)
        sec = _time(lambda: hy.mlstm_out(om, mo, gate, nw, 1e-6, 1.0, ao, H))
        report(f"{phase}.mlstm_out", sec, T * nkk * (4.0 + 4.0 + 2.0))
        qkv, decay, og = torch.randn(T, 3 * nkk, **f32) * 0.1, torch.rand(T, nkk, **f32) * 0.1 + 0.9, torch.empty(T, nkk, **f32)
        st2 = torch.zeros(B, H, D, D, **f32)
        sec = _time(lambda: hy.delta_scan(qkv, nkk, 2 * nkk, None, decay, st2, og, plan, H, True), iters=3, warm=1)
        report(f"{phase}.damilix.gla_scan", sec, B * H * D * D * 8.0 + T * nkk * 20.0)
        out[f"{phase}.damilix.gla_scan"]["fp32_fma_frac"] = round(4.0 * T * H * D * D / sec / 72e12, 3)
        sec = _time(lambda: hy.gated_part_rmsnorm(og, gate, torch.ones(D, **f32), D, "silu", False, 1e-6, 1.0, ao))
        report(f"{phase}.damilix.gated_part_rmsnorm", sec, T * nkk * (4.0 + 4.0 + 2.0))
    return out


def end_to_end(width, n_layers, batch, prompt_len, new=128, vocab=32768):
    from nanorlhf_b200.models.nezavik import NezavikForCausalLM
    from nanorlhf_b200.models.qwen2 import Qwen2Config, Qwen2ForCausalLM
    from nanorlhf_b200.sampler.hybrid_sampler import HybridSampler
    from nanorlhf_b200.sampler.native_sampler import NativeSampler
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, vocab - 2, (batch, prompt_len), generator=g).tolist()
    res = {"width": width, "layers": n_layers, "batch": batch, "prompt_len": prompt_len, "new_tokens": new}
    # ---- Nezavik on the step engine ----
    ncfg = nezavik_config(width, n_layers, vocab)
    nez = NezavikForCausalLM.from_config(ncfg, torch.bfloat16, dev, seed=0, rank=64)
    eng = HybridSampler(nez, dtype="bf16", max_num_seqs=batch, prefill_token_budget=16384)
    pre, step = _gen_times(lambda p, mt: eng.generate(p, 1, 1.0, 1.0, mt, None, vocab - 1, 1), prompts, new)
    res["nezavik"] = {"params_m": round(sum(p.numel() for p in nez.parameters()) / 1e6, 1),
                      "prefill_tok_s": round(batch * prompt_len / pre), "decode_tok_s": round(batch / step),
                      "decode_ms_per_step": round(step * 1e3, 3)}
    eng.release()
    del eng, nez
    torch.cuda.empty_cache()
    # ---- Qwen2 of the same width / depth on the whole-prompt engine ----
    H = width // 128
    qcfg = Qwen2Config(vocab_size=vocab, hidden_size=width, intermediate_size=(8 * width // 3 + 127) // 128 * 128, num_hidden_layers=n_layers,
                       num_attention_heads=H, num_key_value_heads=max(1, H // 4), head_dim=128, tie_word_embeddings=False,
                       max_position_embeddings=8192)
    qw = Qwen2ForCausalLM.from_config(qcfg, torch.bfloat16, dev, seed=0)
    qe = NativeSampler(qw, rollout_dtype="bf16", kv_cache_dtype="bf16", max_num_seqs=max(batch, 128), kv_cache_gb=8.0)
    qe.sync_weights(force=True)
    pre, step = _gen_times(lambda p, mt: qe.generate(p, 1, 1.0, 1.0, mt, None, vocab - 1, 1), prompts, new)
    res["qwen2"] = {"params_m": round(sum(p.numel() for p in qw.parameters()) / 1e6, 1),
                    "prefill_tok_s": round(batch * prompt_len / pre), "decode_tok_s": round(batch / step),
                    "decode_ms_per_step": round(step * 1e3, 3)}
    qe.release()
    del qe, qw
    torch.cuda.empty_cache()
    return res


def kernels(width=2048, batch=16, prompt_len=2048, window=1024, decode_batch=256, ctx=2048):
    """Each kernel of the step engine on its own: seconds, algorithmic bytes / FLOPs, fraction of the roofline."""
    from nanorlhf_b200 import _C
    from nanorlhf_b200.ops import hybrid as hy, native
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    hbm, flops_peak, which = _peaks()
    dev = torch.device("cuda:0")
    out = {"roofline": which, "width": width}
    H, Hkv, D = width // 128, max(1, width // 512), 128

    def plan_for(B, n_new, n_old):
        s = _C.StepScheduler((n_old + n_new + 15) // 16 * B + 8, 16, B)
        sids = [s.open() for _ in range(B)]
        if n_old:
            s.plan(sids, [n_old] * B)
        data, E, T, MB = s.plan(sids, [n_new] * B)
        return StepPlan(torch.from_numpy(data).to(dev), E, T, MB), s

    fp32_peak = 148 * 128 * 2 * 1.9e9              # FMA lanes x 2 x clock: the float32 scans cannot use the tensor cores

    def report(name, sec, bytes_, flops=0.0, like=None, fp32=False):
        floor = max(bytes_ / hbm, flops / (fp32_peak if fp32 else flops_peak))
        out[name] = {"us": round(sec * 1e6, 1), "gb_s": round(bytes_ / sec / 1e9, 1), "tflop_s": round(flops / sec / 1e12, 2),
                     "roofline_frac": round(floor / sec, 3)}
        if like:
            out[name]["like"] = like

    for phase, B, n_new, n_old in (("prefill", batch, prompt_len, 0), ("decode", decode_batch, 1, ctx - 1)):
        plan, sched = plan_for(B, n_new, n_old)
        T = plan.T
        f32 = dict(dtype=torch.float32, device=dev)
        # -- depth-weighted stream + norm (layer 8 of a deep model: 9 results read) vs plain fused add + RMS norm
        nres = 9
        results = torch.randn(nres + 1, T, width, **f32)
        o, xp, xc = torch.randn(T, width, **f32), torch.randn(T, width, **f32), torch.empty(T, width, **f32)
        h = torch.empty(T, width, dtype=torch.bfloat16, device=dev)
        dw, gain = torch.rand(nres + 1, **f32), torch.ones(1, **f32)
        sec = _time(lambda: hy.stream_norm(results, nres, o, xp, dw, gain, 1e-6, xc, h, T))
        report(f"{phase}.stream_norm(depth 9)", sec, T * width * (4.0 * (nres + 2) + 4 * 2 + 2))
        xb, rb, wb = torch.randn(T, width, device=dev).bfloat16(), torch.randn(T, width, device=dev).bfloat16(), torch.ones(width, device=dev).bfloat16()
        sec = _time(lambda: native.add_rmsnorm(xb, rb, wb, 1e-6))
        report(f"{phase}.qwen2.add_rmsnorm", sec, T * width * 2.0 * 4)
        # -- sliding-window attention vs the transformer path's attention
        kc = torch.randn(sched.num_free_blocks() + plan.max_blocks * B + 8, Hkv, 16, D, device=dev).bfloat16()
        vc = torch.randn_like(kc)
        q = torch.randn(T, H * D, **f32)
        k, v = torch.randn(T, Hkv * D, **f32), torch.randn(T, Hkv * D, **f32)
        qw_, kw_ = torch.ones(D, **f32), torch.ones(D, **f32)
        ao = torch.empty(T, H * D, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.qknorm_kv_write(q, k, v, qw_, kw_, 1e-6, kc, vc, plan))
        report(f"{phase}.qknorm_kv_write", sec, T * (H + 2 * Hkv) * D * 4.0 + T * H * D * 4.0 + T * 2 * Hkv * D * 2.0)
        for impl in ("auto", "tile", "mma"):
            sec = _time(lambda: hy.window_attention(q, kc, vc, plan, window, D ** -0.5, 1.0, ao, impl=impl), iters=3, warm=1)
            name = f"{phase}.window_attention(w={window})" + ("" if impl == "auto" else f"[{impl}]")
            if phase == "prefill":
                keys = sum(min(p + 1, window) for p in range(n_new)) * B
                report(name, sec, T * H * D * 6.0 + T * 2 * Hkv * D * 2.0, flops=4.0 * keys * H * D)
            else:
                keys = min(ctx, window)
                report(name, sec, B * keys * 2 * Hkv * D * 2.0 + T * H * D * 6.0, flops=4.0 * B * keys * H * D)
        if phase == "prefill":
            from nanorlhf_b200.ops.attention import attention_varlen
            qb = torch.randn(T, H, D, device=dev).bfloat16()
            kb, vb = torch.randn(T, Hkv, D, device=dev).bfloat16(), torch.randn(T, Hkv, D, device=dev).bfloat16()
            cu = torch.arange(0, T + 1, n_new, dtype=torch.int32, device=dev)
            sec = _time(lambda: attention_varlen(qb, kb, vb, cu, n_new, causal=True))
            report("prefill.qwen2.attention_fwd(causal, full)", sec, T * (2 * H + 2 * Hkv) * D * 2.0, flops=4.0 * B * n_new * (n_new + 1) / 2 * H * D)
        else:
            qb = torch.randn(B, H, D, device=dev).bfloat16()
            ctxl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
            sec = _time(lambda: native.paged_decode(qb, kc, vc, plan.block_table.contiguous(), ctxl, D ** -0.5, 1))
            report("decode.qwen2.paged_decode(full ctx)", sec, B * ctx * 2 * Hkv * D * 2.0, flops=4.0 * B * ctx * H * D)
        del kc, vc
        # -- recurrent mixers (no like kernel in the transformer path)
        Hs, P, N = width // 64, 64, 128
        ch = Hs * P + 2 * N
        raw, conv_w, conv_b = torch.randn(T, ch, **f32), torch.randn(ch, 4, **f32), torch.randn(ch, **f32)
        cst, xbc = torch.zeros(B, 3, ch, **f32), torch.empty(T, ch, **f32)
        sec = _time(lambda: hy.causal_conv(raw, conv_w, conv_b, cst, xbc, plan))
        report(f"{phase}.causal_conv", sec, T * ch * 8.0 + B * 3 * ch * 8.0)
        st = torch.zeros(B, Hs, N, P, **f32)
        dt, y = torch.randn(T, Hs, **f32), torch.empty(T, Hs * P, **f32)
        vec = torch.zeros(Hs, **f32)
        for impl in ("auto", "rows"):
            sec = _time(lambda: hy.ssd_scan(xbc, Hs * P, Hs * P + N, dt, vec, vec, vec, st, y, plan, 1, impl=impl), iters=3, warm=1)
            report(f"{phase}.ssd_scan" + ("" if impl == "auto" else f"[{impl}]"), sec,
                   T * (ch + Hs + Hs * P) * 4.0 + 2 * st.numel() * 4.0, flops=6.0 * T * Hs * N * P, fp32=True)
        Hd, Dk, Dv = width // 128, 128, 128
        qkv = torch.randn(T, 3 * Hd * Dk, **f32)
        beta, dec = torch.rand(T, Hd, **f32), torch.rand(T, Hd, **f32)
        std, od = torch.zeros(B, Hd, Dk, Dv, **f32), torch.empty(T, Hd * Dv, **f32)
        for impl in ("auto", "rows"):
            sec = _time(lambda: hy.delta_scan(qkv, Hd * Dk, 2 * Hd * Dk, beta, dec, std, od, plan, Hd, False, impl=impl), iters=3, warm=1)
            report(f"{phase}.delta_scan" + ("" if impl == "auto" else f"[{impl}]"), sec,
                   T * (4 * Hd * Dk + 2 * Hd) * 4.0 + 2 * std.numel() * 4.0, flops=8.0 * T * Hd * Dk * Dv, fp32=True)
        gate, nw = torch.randn(T, Hd * Dv, **f32), torch.ones(Dv, **f32)
        go = torch.empty(T, Hd * Dv, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.gated_part_rmsnorm(od, gate, nw, Dv, "silu", False, 1e-6, 1.0, go))
        report(f"{phase}.gated_part_rmsnorm", sec, T * Hd * Dv * 10.0)
        up = torch.randn(T, 4 * width, **f32)
        ub = torch.empty(T, 4 * width, dtype=torch.bfloat16, device=dev)
        sec = _time(lambda: hy.act_cols(up, ub, "relu2"))
        report(f"{phase}.relu2", sec, T * 4 * width * 6.0)
        gu = torch.randn(T, 8 * width, device=dev).bfloat16()
        sec = _time(lambda: native.ext().swiglu(gu))
        report(f"{phase}.qwen2.swiglu", sec, T * 4 * width * 6.0)
    return out


def main(quick: bool = False, small: bool = False, model: str = "nezavik"):
    from nanorlhf_b200.ops import native
    global SMALL
    native.load()
    if model == "lukarax":
        SMALL = small
        if small:
            print(json.dumps({"bench": "serve-lukarax-small",
                              "kernels": kernels_lukarax(width=1024, batch=8, prompt_len=1024, decode_batch=64, ctx=1024)}))
            return None
        res = {"bench": "serve-lukarax", "kernels": kernels_lukarax(), "end_to_end": []}
        for width, layers, batch, plen in ((1024, 8, 32, 1024), (2048, 8, 16, 2048)) if not quick else ((1024, 4, 8, 512),):
            res["end_to_end"].append(end_to_end_lukarax(width, layers, batch, plen))
        res["gpu_launches"] = native.launches()
        print(json.dumps(res))
        return res
    if model == "damilix":
        SMALL = small
        if small:
            print(json.dumps({"bench": "serve-damilix-small",
                              "kernels": kernels_damilix(width=1024, batch=8, prompt_len=1024, decode_batch=64, ctx=1024)}))
            return None
        res = {"bench": "serve-damilix", "kernels": kernels_damilix(), "end_to_end": []}
        for width, layers, batch, plen in ((1024, 8, 32, 1024), (2048, 8, 16, 2048)) if not quick else ((1024, 4, 8, 512),):
            res["end_to_end"].append(end_to_end_damilix(width, layers, batch, plen))
        res["gpu_launches"] = native.launches()
        print(json.dumps(res))
        return res
    if model == "vilosun":
        SMALL = small
        if small:
            print(json.dumps({"bench": "serve-vilosun-small",
                              "kernels": kernels_vilosun(width=1024, batch=8, prompt_len=1024, decode_batch=64, ctx=1024)}))
            return None
        res = {"bench": "serve-vilosun", "kernels": kernels_vilosun(), "end_to_end": []}
        for width, layers, batch, plen in ((1024, 8, 32, 1024), (2048, 8, 16, 2048)) if not quick else ((1024, 4, 8, 512),):
            res["end_to_end"].append(end_to_end_vilosun(width, layers, batch, plen))
        res["gpu_launches"] = native.launches()
        print(json.dumps(res))
        return res
    if small:                                  # kernels only, on a case of a few hundred MB
        SMALL = True
        print(json.dumps({"bench": "serve-small", "kernels": kernels(width=1024, batch=8, prompt_len=1024, decode_batch=64, ctx=1024)}))
        return None
    res = {"bench": "serve", "kernels": kernels(), "end_to_end": []}
    for width, layers, batch, plen in ((1024, 8, 32, 1024), (2048, 8, 16, 2048)) if not quick else ((1024, 4, 8, 512),):
        res["end_to_end"].append(end_to_end(width, layers, batch, plen))
    res["gpu_launches"] = native.launches()
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main(quick="--quick" in sys.argv, small="--small" in sys.argv,
         model="lukarax" if "--lukarax" in sys.argv else "damilix" if "--damilix" in sys.argv else "vilosun" if "--vilosun" in sys.argv else "nezavik")
