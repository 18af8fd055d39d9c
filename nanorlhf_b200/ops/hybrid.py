"""Op layer of hybrid (attention + recurrent-state) decoders: thin, launch-counting wrappers over the sm_100a kernels of
``csrc/stream_ops.cu``, ``csrc/recurrent.cu``, ``csrc/attention_window.cu`` / ``attention_window_mma.cu`` /
``attention_latent_mma.cu`` and ``csrc/moe.cu``
(with the grouped form of ``csrc/gemm_tc.cu``).

All of them take the step plan of ``_C.StepScheduler.plan`` (entries = runs of consecutive tokens of one sequence) and
work on packed ``[tokens, ...]`` tensors; recurrent state and convolution taps live in per-sequence slots, keys and values
in 16-token pages.  There is no PyTorch fallback: these ops exist on CUDA only.
"""
from __future__ import annotations

from . import native


def _ext():
    return native.ext()


def embed_pos(embed, pos_table, tok, pos, out):
    native._count()
    _ext().embed_pos(embed, pos_table, tok, pos, out)
    return out


def stream_norm(results, i, o, xprev, dw, gain, eps, xcur, h, T):
    """Close layer ``i - 1`` (``results[i] = xprev + o``), form ``x = sum_j dw[j] results[j]`` and ``h = rmsnorm(x) * gain``."""
    native._count()
    _ext().stream_norm(results, i, o, xprev, dw, gain, eps, xcur, h, T)


def act_cols(x, out, act: str = "copy"):
    native._count()
    _ext().act_cols(x, out, {"copy": 0, "relu2": 1}[act])


def gated_part_rmsnorm(y, gate, w, part, gate_act, gate_first, eps, scale, out):
    native._count()
    _ext().gated_part_rmsnorm(y, gate, w, part, {"silu": 0, "sigmoid": 1}[gate_act], gate_first, eps, scale, out)


def causal_conv(x, w, bias, state, out, plan, in_bias=None, act: str = "silu"):
    """``in_bias``: bias of the projection that made ``x`` (part of the convolved signal and of the carried taps); ``bias``: added
    after the convolution; ``act``: "silu" or "none"."""
    native._count(2)
    _ext().causal_conv(x, w, bias, state, out, plan.cu, plan.tok_entry, plan.start, plan.state_slot, in_bias,
                       {"none": 0, "silu": 1}[act])


SCAN_IMPLS = {"auto": 0, "column": 1, "rows": 2, "shared": 3}


def ssd_scan(xbc, col_b, col_c, dt_raw, dt_bias, A_log, D, state, y, plan, groups, impl: str = "auto"):
    native._count()
    _ext().ssd_scan(xbc, col_b, col_c, dt_raw, dt_bias, A_log, D, state, y, plan.cu, plan.start, plan.state_slot, groups,
                    SCAN_IMPLS[impl])


def delta_prep(qkv, col_k, b_raw, a_raw, dt_bias, A_log, beta, decay, kv_heads, dim, per_channel):
    native._count()
    _ext().delta_prep(qkv, col_k, b_raw, a_raw, dt_bias, A_log, beta, decay, kv_heads, dim, per_channel)


def delta_scan(qkv, col_k, col_v, beta, decay, state, o, plan, kv_heads, per_channel, impl: str = "auto"):
    """``beta`` None: plain accumulation ``S = diag(decay) S + k v^T`` (gated linear attention) instead of the delta rule."""
    native._count()
    _ext().delta_scan(qkv, col_k, col_v, beta, decay, state, o, plan.cu, plan.start, plan.state_slot, kv_heads, per_channel,
                      SCAN_IMPLS[impl])


def qknorm_kv_write(q, k, v, qw, kw, eps, k_cache, v_cache, plan):
    native._count()
    _ext().qknorm_kv_write(q, k, v, qw, kw, eps, k_cache, v_cache, plan.kv_slot)


WINDOW_IMPLS = {"auto": 0, "tile": 1, "simple": 2, "mma": 3}


def window_attention(q, k_cache, v_cache, plan, window, scale, out_scale, out, impl: str = "auto", chunked: bool = False,
                     head_scale=None, head_slope=None, gate=None, head_sink=None, value_size: int = 0, softcap: float = 0.0,
                     keep_first: int = 0, dist_bias=None, v_div: int = 1):
    """``impl``: "auto" (tensor cores for prompt portions over bf16 pages, the scalar tile kernel otherwise) or one kernel by
    name; a kernel that does not fit the shapes raises.  ``chunked``: keys of the query's own chunk of ``window`` positions
    instead of the last ``window`` keys.  ``head_scale`` / ``head_slope`` [heads]: per-head score multiplier and linear distance
    penalty; ``gate`` [T, heads]: the head's output is multiplied by sigmoid(gate); ``head_sink`` [heads]: the softmax denominator
    also holds exp(sink).  ``value_size`` > 0 (with ``v_cache is k_cache``): the values are the first ``value_size`` columns of the
    key rows (latent attention: one cached row per token serves as key and value of every head); ``q`` may then be head-major
    [heads, T, >= D], the layout a batched GEMM leaves.  ``softcap`` > 0: the scaled score becomes softcap * tanh(score / softcap);
    ``keep_first`` > 0: the first positions of a sequence stay visible behind the window; ``dist_bias`` [distances, heads]: row
    min(distance, distances - 1) is added to the score (after scale and cap); ``v_div`` > 1: that many neighbouring key heads read
    one value head (several score maps over the same values).  ``out`` may be float32 over bf16 pages: the result is then not
    rounded (for results that are combined further)."""
    native._count()
    _ext().window_attention(q, k_cache, v_cache, plan.block_table, plan.tok_entry, plan.pos, window, scale, out_scale, out,
                            WINDOW_IMPLS[impl], chunked, head_scale, head_slope, gate, head_sink, value_size > 0, value_size,
                            q.shape[0] if q.dim() == 3 else 0, softcap, keep_first, dist_bias, v_div)


def kv_write_blend(k, v, v_other, lam, k_cache, v_cache, plan):
    """Keys and values into their pages; ``v <- (1 - lam) v + lam v_other`` first (in place) when ``v_other`` is given."""
    native._count()
    _ext().kv_write_blend(k, v, v_other, lam, k_cache, v_cache, plan.kv_slot)


def embed_hashed(embed, pair, plan, prev_state, scale, mul_prev, mul_cur, buckets, out):
    """x0 = embed[tok] * scale + pair[(prev * mul_prev + tok * mul_cur) % buckets] (row ``buckets`` at a sequence's start)."""
    native._count(2 if pair is not None else 1)
    _ext().embed_hashed(embed, pair, plan.tokens, plan.cu, plan.tok_entry, plan.start, plan.state_slot, prev_state, scale, mul_prev,
                        mul_cur, buckets, out)
    return out


def group_norm_residual(x, o, gate, gate_bias, w_post, w_pre, groups, eps, h):
    """``x += groupnorm(o * sigmoid(gate + gate_bias)) * w_post`` (when ``o`` is given), then ``h = groupnorm(x) * w_pre``."""
    native._count()
    _ext().group_norm_residual(x, o, gate, gate_bias, w_post, w_pre, groups, eps, h)


def moe_route(router, router_bias, top, gu=None, ff=0, act=None, ids=None, wts=None):
    """Top-k routing (softmax over the chosen logits); with ``gu`` / ``act`` also the dense-form expert activations."""
    native._count()
    _ext().moe_route(router, router_bias, top, gu, ff, act, ids, wts)


def interleave_gate_up(gate, up):
    """Rows of one expert's gate and up matrices [ff, W] interleaved per 32 features ([32 gate | 32 up] ...): the layout the
    grouped GEMM's SwiGLU epilogue expects (``ff % 32 == 0``)."""
    import torch
    ff, W = gate.shape
    return torch.stack([gate.view(ff // 32, 32, W), up.view(ff // 32, 32, W)], 1).reshape(2 * ff, W)


def moe_grouped_ffn(h, ids, wts, w_gate_up, w_down, experts, ff, out, fused_act: bool = False, identity: int = 0):
    """Expert feed-forwards of a routed batch on the grouped tcgen05 GEMM.  ``h`` bf16 [T, W]; ``ids`` / ``wts`` [T, top] from
    ``moe_route``; ``w_gate_up`` bf16 [experts * 2 ff, W] (per expert its gate rows, then its up rows; ``fused_act``: interleaved
    per 32 features by ``interleave_gate_up``, the SwiGLU is then formed in the GEMM's epilogue); ``w_down`` bf16
    [experts * W, ff]; ``out`` float [T, W] = sum_k wts[t, k] * expert_k(h[t]).  No launch depends on the routing.
    ``identity``: ids ``experts .. experts + identity - 1`` name experts without matrices; their pairs carry weight 0 here and are
    skipped (the caller adds their share of the input)."""
    import torch
    T, W = h.shape
    R = ids.numel()
    ext = _ext()
    native._count(5 if fused_act else 6)
    slot_of, row_token, _seg, tiles, num_tiles = ext.moe_plan(ids, experts + identity, 128, experts)
    xp = torch.empty(R, W, dtype=h.dtype, device=h.device)
    ext.gather_rows(h, row_token, xp)
    act = torch.empty(R, ff, dtype=h.dtype, device=h.device)
    if fused_act:
        ext.gemm_tc_grouped(xp, w_gate_up, None, tiles, num_tiles, 0, act)
    else:
        gu = torch.empty(R, 2 * ff, dtype=torch.float32, device=h.device)
        ext.gemm_tc_grouped(xp, w_gate_up, gu, tiles, num_tiles)
        ext.swiglu_rows(gu, act)
    y = torch.empty(R, W, dtype=torch.float32, device=h.device)
    ext.gemm_tc_grouped(act, w_down, y, tiles, num_tiles)
    ext.moe_combine(y, slot_of, wts, out)
    return out


def embed_norm(embed, tok, w, eps, x, h):
    """x = embed[tok] / rms * w (float); h = x in the GEMM operand type."""
    native._count()
    _ext().embed_norm(embed, tok, w, eps, x, h)


def post_norm_residual(x, o, self_w, w_post, w_pre, eps, h):
    """Boundary of a stream that norms only what a sublayer returns: ``x += rmsnorm(o + self_w[:, None] * x) * w_post`` (``self_w``
    None: no such term), then ``h = rmsnorm(x) * w_pre`` or, without ``w_pre``, ``h = x`` (operand type)."""
    native._count()
    _ext().post_norm_residual(x, o, self_w, w_post, w_pre, eps, h)


def side_gate(u, table, col0, tok, out, dim):
    """out[:, :dim] = gelu_tanh(u[:, :dim]) * table[tok, col0:col0 + dim]; further columns of ``out`` are zeroed."""
    native._count()
    _ext().side_gate(u, table, col0, tok, out, dim)


def swiglu_cols(gu, row_gate, out):
    """out = silu(gu[:, :C]) * gu[:, C:] (``* sigmoid(row_gate)`` [T, 1] when given)."""
    native._count()
    _ext().swiglu_cols(gu, row_gate, out)


def moe_route_all(router, correction, n_real, top, scale, gu=None, ff=0, act=None, ids=None, wts=None, self_w=None, groups: int = 1,
                  keep: int = 1):
    """Routing by a softmax over all router outputs (the last ``E - n_real`` are identity experts), choice by score + correction,
    weights = chosen scores / their sum * scale; ``self_w`` [T] receives the identity experts' weights.  ``groups`` > 1: the outputs
    form that many equal groups of neighbours and only the ``keep`` groups with the largest choice score can be chosen from."""
    native._count()
    _ext().moe_route_all(router, correction, n_real, top, scale, groups, keep, gu, ff, act, ids, wts, self_w)


def gla_prep(qkv, a_raw, a_bias, tau, decay, heads, dim):
    """q (first heads * dim columns of ``qkv``) times dim^-1/2 in place; decay = sigmoid(a_raw + a_bias)^(1 / tau)."""
    native._count()
    _ext().gla_prep(qkv, a_raw, a_bias, tau, decay, heads, dim)


def latent_kv_write(q, heads, dim, rot_dim, dkv, norm_w, eps, freq, rot_dims, mult, interleaved, plan, cache, qa, qn=None):
    """Latent attention, write side: RMS-normed latent + rotated shared key part into the token's cache row, the heads' rotated
    query parts into ``qa`` ([T, heads * (rank + rot_dim)] or head-major [heads, T, rank + rot_dim]) behind the absorbed columns;
    ``qn`` (bf16 [heads, T, dim]) receives the unrotated query columns as the operand of the GEMM that absorbs them."""
    native._count()
    _ext().latent_kv_write(q, heads, dim, rot_dim, dkv, norm_w, eps, freq, rot_dims, mult, interleaved, plan.pos, plan.kv_slot, cache, qa, qn)


def rotary_frequencies(dims: int, base: float, scaling=None):
    """(frequencies [dims / 2] as float64 list, cos / sin multiplier).  ``scaling`` {"factor", "original", "fast", "slow"}: frequencies
    that turn more than ``fast`` times within ``original`` positions keep their value, those that turn less than ``slow`` times
    are divided by ``factor``, linear in the pair index between; cos and sin are then multiplied by 0.1 ln(factor) + 1."""
    import math
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):                                    # the (real-valued) pair index that turns `turns` times in `orig` positions
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def embed_streams(embed, tok, scale, xs):
    """xs[t, s] = embed[tok[t]] * scale for every residual stream s (xs float [T, S, W])."""
    native._count()
    _ext().embed_streams(embed, tok, scale, xs)


def hyper_boundary(xs, o, o_bias, self_w, mix, outw, inw, ln_w, ln_b, eps, h):
    """Boundary between sublayers over several mixed residual streams.  With ``o`` (the closing sublayer's result, plus ``o_bias`` [W]
    and ``self_w[t] * h[t]``, h still being that sublayer's input): ``x_t <- sum_s mix[s, t] x_s + outw[t] y`` for all streams at once.
    With ``h``: ``u = sum_s inw[s] x_s`` (``inw`` None: the plain sum) and ``h = layernorm(u) * ln_w + ln_b`` in the operand type."""
    native._count()
    _ext().hyper_boundary(xs, o, o_bias, self_w, mix, outw, inw, ln_w, ln_b, eps, h)


MLSTM_IMPLS = {"auto": 0, "column": 1, "global": 2}


def mlstm_scan(qkv, col_q, col_k, col_v, col_i, col_f, i_bias, f_bias, cap, q_scale, state, mstate, o, m_out, plan, impl: str = "auto"):
    """Matrix memory with exponential gates: ``state`` [slots, heads, D, >= Dv + 1] holds S and, as column Dv, the normaliser n;
    ``mstate`` [slots, heads] the running maximum.  ``o`` [T, heads, Dv + 1] receives S^T q (numerator | n . q), ``m_out`` [T, heads]
    the maximum after every token."""
    native._count()
    _ext().mlstm_scan(qkv, col_q, col_k, col_v, col_i, col_f, i_bias, f_bias, cap, q_scale, state, mstate, o, m_out, plan.cu, plan.start,
                      plan.state_slot, MLSTM_IMPLS[impl])


def mlstm_out(o, m, gate, w, eps, scale, out, heads):
    """y = o[:Dv] / (max(|o[Dv]|, exp(-m)) + 1e-6); out = scale * y / rms_head(y) * w * sigmoid(gate)."""
    native._count()
    _ext().mlstm_out(o, m, gate, w, eps, scale, out, heads)


def rot_kv_write(q, q_bias, k, k_bias, v, freq, rot_dims, mult, interleaved, unit_norm, q_norm_w, k_norm_w, eps, plan, k_cache, v_cache):
    """Biased, rotated and (``unit_norm``) RMS-normed queries in place and keys into their pages; values into their pages (``v`` None:
    the values are the keys as projected).  ``k`` None: queries only."""
    native._count()
    _ext().rot_kv_write(q, q_bias, k, k_bias, v, freq, rot_dims, mult, interleaved, unit_norm, q_norm_w, k_norm_w, eps, plan.pos,
                        plan.kv_slot, k_cache, v_cache)


def diff_combine(a, lam, post, eps, gate, out_scale, out, heads, kv_heads):
    """Two score maps over the same values: o = a_1 - lam a_2 per head, RMS-normed, times ``post`` and sigmoid(gate)."""
    native._count()
    _ext().diff_combine(a, lam, post, eps, gate, out_scale, out, heads, kv_heads)


def distance_bias_table(rel, bias_max: int):
    """Expand a bucketed distance bias ``rel`` [B, heads] into one row per distance 0 .. bias_max: the first B / 2 buckets hold one
    distance each, the others grow logarithmically up to ``bias_max``, from where on the last bucket holds."""
    import math

    import torch
    B = rel.shape[0]
    half = B // 2
    rows = []
    for n in range(bias_max + 1):
        if n < half:
            rows.append(n)
        elif bias_max <= half:
            rows.append(B - 1)
        else:
            rows.append(min(B - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (B - half)))))
    return rel.float()[torch.tensor(rows, device=rel.device)].contiguous()
