// Tensor validation + stream forwarding for the hybrid-decoder kernels; the launch API is hybrid_kernels.h.
#include "bindings_hybrid.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "gemm_tc.h"
#include "hybrid_kernels.h"
#include "tma_host.h"

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void check(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }

inline const float* f32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kFloat32, name, " must be a CUDA float tensor");
  TORCH_CHECK(t.dim() == 0 || t.stride(-1) == 1, name, " must have unit inner stride");
  return t.data_ptr<float>();
}
inline float* f32w(Tensor& t, const char* name) { return const_cast<float*>(f32(t, name)); }
inline const int* i32(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous(), name, " must be a contiguous CUDA int32 tensor");
  return t.data_ptr<int>();
}
// typed operand: float or bf16 with unit inner stride; returns is-float
inline int typed(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && (t.scalar_type() == torch::kFloat32 || t.scalar_type() == torch::kBFloat16), name,
              " must be a CUDA float or bf16 tensor");
  TORCH_CHECK(t.stride(-1) == 1, name, " must have unit inner stride");
  return t.scalar_type() == torch::kFloat32 ? 1 : 0;
}

void embed_pos(const Tensor& embed, const Tensor& pos_table, const Tensor& tok, const Tensor& pos, Tensor out) {
  c10::cuda::CUDAGuard guard(out.device());
  const int wf = typed(embed, "embed");
  TORCH_CHECK(typed(pos_table, "pos_table") == wf && embed.is_contiguous() && pos_table.is_contiguous(), "embed_pos: tables");
  const int T = static_cast<int>(tok.numel()), W = static_cast<int>(embed.size(1));
  TORCH_CHECK(out.is_contiguous() && out.size(0) >= T && out.size(1) == W && pos_table.size(1) == W, "embed_pos: shapes");
  check(nrl_embed_pos(embed.data_ptr(), pos_table.data_ptr(), wf, i32(tok, "tok"), i32(pos, "pos"), f32w(out, "out"), T, W, cur_stream()),
        "embed_pos");
}

void stream_norm(Tensor results, int64_t i, const c10::optional<Tensor>& o, const c10::optional<Tensor>& xprev,
                 const c10::optional<Tensor>& dw, const Tensor& g, double eps, Tensor xcur, Tensor h, int64_t T) {
  c10::cuda::CUDAGuard guard(h.device());
  TORCH_CHECK(results.dim() == 3 && results.stride(2) == 1 && results.stride(1) == results.size(2), "stream_norm: results [n, cap, W]");
  const int W = static_cast<int>(results.size(2));
  TORCH_CHECK(i >= 0 && i < results.size(0) && T <= results.size(1), "stream_norm: index");
  TORCH_CHECK(xcur.is_contiguous() && xcur.size(-1) == W && h.is_contiguous() && h.size(-1) == W, "stream_norm: outputs");
  TORCH_CHECK(o.has_value() == xprev.has_value(), "stream_norm: o and xprev go together");
  if (o.has_value()) TORCH_CHECK(o->is_contiguous() && xprev->is_contiguous() && o->size(-1) == W, "stream_norm: o / xprev");
  if (dw.has_value()) TORCH_CHECK(dw->numel() == i + 1, "stream_norm: one depth weight per result");
  check(nrl_stream_norm(f32w(results, "results"), results.stride(0), static_cast<int>(i), o.has_value() ? f32(*o, "o") : nullptr,
                        xprev.has_value() ? f32(*xprev, "xprev") : nullptr, dw.has_value() ? f32(*dw, "dw") : nullptr, f32(g, "g"),
                        static_cast<float>(eps), f32w(xcur, "xcur"), h.data_ptr(), typed(h, "h"), static_cast<int>(T), W, cur_stream()),
        "stream_norm");
}

void act_cols(const Tensor& in, Tensor out, int64_t act) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(in.dim() == 2 && out.dim() == 2 && in.size(0) == out.size(0) && in.size(1) == out.size(1), "act_cols: shapes");
  check(nrl_act_cols(f32(in, "in"), in.stride(0), out.data_ptr(), out.stride(0), typed(out, "out"), static_cast<int>(act),
                     static_cast<int>(in.size(0)), static_cast<int>(in.size(1)), cur_stream()),
        "act_cols");
}

void gated_part_rmsnorm(const Tensor& y, const Tensor& gate, const Tensor& w, int64_t part, int64_t gate_act, bool gate_first,
                        double eps, double scale, Tensor out) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(y.dim() == 2 && gate.dim() == 2 && out.dim() == 2 && gate.size(1) == y.size(1) && out.size(1) == y.size(1) &&
                  gate.size(0) == y.size(0) && out.size(0) == y.size(0), "gated_part_rmsnorm: shapes");
  const bool shared = w.numel() == part;
  TORCH_CHECK(shared || w.numel() == y.size(1), "gated_part_rmsnorm: weight of one part or of all columns");
  check(nrl_gated_part_rmsnorm(f32(y, "y"), y.stride(0), f32(gate, "gate"), gate.stride(0), f32(w, "w"), shared ? 1 : 0,
                               static_cast<int>(part), static_cast<int>(gate_act), gate_first ? 1 : 0, static_cast<float>(eps),
                               static_cast<float>(scale), out.data_ptr(), out.stride(0), typed(out, "out"),
                               static_cast<int>(y.size(0)), static_cast<int>(y.size(1)), cur_stream()),
        "gated_part_rmsnorm");
}

void causal_conv(const Tensor& in, const Tensor& w, const c10::optional<Tensor>& bias, Tensor state, Tensor out, const Tensor& cu,
                 const Tensor& tok_entry, const Tensor& start, const Tensor& state_slot, const c10::optional<Tensor>& in_bias,
                 int64_t act) {
  c10::cuda::CUDAGuard guard(out.device());
  const int T = static_cast<int>(in.size(0)), C = static_cast<int>(in.size(1)), taps = static_cast<int>(w.size(1));
  const int E = static_cast<int>(start.numel());
  TORCH_CHECK(in.dim() == 2 && out.dim() == 2 && out.size(0) == T && out.size(1) == C && w.is_contiguous() && w.size(0) == C,
              "causal_conv: shapes");
  TORCH_CHECK(state.is_contiguous() && state.dim() == 3 && state.size(1) == taps - 1 && state.size(2) == C, "causal_conv: state [slots, taps-1, C]");
  TORCH_CHECK(cu.numel() == E + 1 && tok_entry.numel() >= T && state_slot.numel() == E, "causal_conv: plan");
  if (bias.has_value()) TORCH_CHECK(bias->numel() == C, "causal_conv: bias");
  if (in_bias.has_value()) TORCH_CHECK(in_bias->numel() == C, "causal_conv: in_bias");
  const float* ib = in_bias.has_value() ? f32(*in_bias, "in_bias") : nullptr;
  check(nrl_causal_conv(f32(in, "in"), in.stride(0), ib, static_cast<int>(act), f32(w, "w"),
                        bias.has_value() ? f32(*bias, "bias") : nullptr, f32(state, "state"),
                        f32w(out, "out"), out.stride(0), i32(cu, "cu"), i32(tok_entry, "tok_entry"), i32(start, "start"),
                        i32(state_slot, "state_slot"), T, E, C, taps, cur_stream()),
        "causal_conv");
  check(nrl_causal_conv_carry(f32(in, "in"), in.stride(0), ib, f32w(state, "state"), i32(cu, "cu"), i32(start, "start"),
                              i32(state_slot, "state_slot"), E, C, taps, cur_stream()),
        "causal_conv_carry");
}

void ssd_scan(const Tensor& xbc, int64_t col_b, int64_t col_c, const Tensor& dt_raw, const Tensor& dt_bias, const Tensor& A_log,
              const Tensor& Dskip, Tensor state, Tensor y, const Tensor& cu, const Tensor& start, const Tensor& state_slot, int64_t groups,
              int64_t impl) {
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(state.dim() == 4 && state.is_contiguous(), "ssd_scan: state [slots, heads, N, P]");
  const int heads = static_cast<int>(state.size(1)), N = static_cast<int>(state.size(2)), P = static_cast<int>(state.size(3));
  const int E = static_cast<int>(start.numel());
  TORCH_CHECK(xbc.dim() == 2 && dt_raw.dim() == 2 && dt_raw.size(1) == heads && y.is_contiguous() && y.size(-1) == heads * P &&
                  y.size(0) >= xbc.size(0), "ssd_scan: shapes");
  TORCH_CHECK(col_b >= heads * P && col_c + groups * N <= xbc.size(1) && dt_bias.numel() == heads && A_log.numel() == heads &&
                  Dskip.numel() == heads, "ssd_scan: columns / per-head vectors");
  check(nrl_ssd_scan(f32(xbc, "xbc"), xbc.stride(0), static_cast<int>(col_b), static_cast<int>(col_c), f32(dt_raw, "dt_raw"),
                     dt_raw.stride(0), f32(dt_bias, "dt_bias"), f32(A_log, "A_log"), f32(Dskip, "D"), f32w(state, "state"), f32w(y, "y"),
                     i32(cu, "cu"), i32(start, "start"), i32(state_slot, "state_slot"), E, heads, static_cast<int>(groups), N, P,
                     static_cast<int>(impl), cur_stream()),
        "ssd_scan");
}

void delta_prep(Tensor qkv, int64_t col_k, const Tensor& b_raw, const Tensor& a_raw, const Tensor& dt_bias, const Tensor& A_log,
                Tensor beta, Tensor decay, int64_t kv_heads, int64_t D, bool per_channel) {
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = static_cast<int>(qkv.size(0)), heads = static_cast<int>(A_log.numel());
  TORCH_CHECK(dt_bias.numel() == (per_channel ? static_cast<int64_t>(heads) * D : heads), "delta_prep: dt_bias per head or per head and key channel");
  TORCH_CHECK(b_raw.dim() == 2 && b_raw.size(1) == heads && a_raw.dim() == 2 && a_raw.size(1) == dt_bias.numel() && beta.is_contiguous() &&
                  decay.is_contiguous() && beta.numel() >= static_cast<int64_t>(T) * heads &&
                  decay.numel() >= static_cast<int64_t>(T) * dt_bias.numel(), "delta_prep: shapes");
  check(nrl_delta_prep(f32w(qkv, "qkv"), qkv.stride(0), static_cast<int>(col_k), f32(b_raw, "b_raw"), b_raw.stride(0), f32(a_raw, "a_raw"),
                       a_raw.stride(0), f32(dt_bias, "dt_bias"), f32(A_log, "A_log"), f32w(beta, "beta"), f32w(decay, "decay"), T, heads,
                       static_cast<int>(kv_heads), static_cast<int>(D), per_channel ? 1 : 0, cur_stream()),
        "delta_prep");
}

void delta_scan(const Tensor& qkv, int64_t col_k, int64_t col_v, const c10::optional<Tensor>& beta, const Tensor& decay, Tensor state, Tensor o,
                const Tensor& cu, const Tensor& start, const Tensor& state_slot, int64_t kv_heads, bool per_channel, int64_t impl) {
  c10::cuda::CUDAGuard guard(o.device());
  TORCH_CHECK(state.dim() == 4 && state.is_contiguous(), "delta_scan: state [slots, heads, D, Dv]");
  const int heads = static_cast<int>(state.size(1)), D = static_cast<int>(state.size(2)), Dv = static_cast<int>(state.size(3));
  const int E = static_cast<int>(start.numel());
  TORCH_CHECK(qkv.dim() == 2 && col_v + heads * Dv <= qkv.size(1) && o.is_contiguous() && o.size(-1) == heads * Dv, "delta_scan: shapes");
  check(nrl_delta_scan(f32(qkv, "qkv"), qkv.stride(0), static_cast<int>(col_k), static_cast<int>(col_v), beta.has_value() ? f32(*beta, "beta") : nullptr,
                       f32(decay, "decay"), f32w(state, "state"), f32w(o, "o"), i32(cu, "cu"), i32(start, "start"),
                       i32(state_slot, "state_slot"), E, heads, static_cast<int>(kv_heads), D, Dv, per_channel ? 1 : 0,
                       static_cast<int>(impl), cur_stream()),
        "delta_scan");
}

void qknorm_kv_write(Tensor q, const Tensor& k, const Tensor& v, const Tensor& qw, const Tensor& kw, double eps, Tensor k_cache,
                     Tensor v_cache, const Tensor& kv_slot) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(), "qknorm_kv_write: caches");
  const int Hkv = static_cast<int>(k_cache.size(1)), page = static_cast<int>(k_cache.size(2)), D = static_cast<int>(k_cache.size(3));
  const int Dv = static_cast<int>(v_cache.size(3));
  const int T = static_cast<int>(q.size(0)), Hq = static_cast<int>(q.size(1) / D);
  TORCH_CHECK(q.size(1) == static_cast<int64_t>(Hq) * D && k.size(1) == static_cast<int64_t>(Hkv) * D &&
                  v.size(1) == static_cast<int64_t>(Hkv) * Dv && qw.numel() == D && kw.numel() == D && kv_slot.numel() >= T,
              "qknorm_kv_write: shapes");
  const int cf = typed(k_cache, "k_cache");
  TORCH_CHECK(typed(v_cache, "v_cache") == cf, "qknorm_kv_write: cache types differ");
  check(nrl_qknorm_kv_write(f32w(q, "q"), q.stride(0), f32(k, "k"), k.stride(0), f32(v, "v"), v.stride(0), f32(qw, "qw"), f32(kw, "kw"),
                            static_cast<float>(eps), k_cache.data_ptr(), v_cache.data_ptr(), cf, i32(kv_slot, "kv_slot"), T, Hq, Hkv, D,
                            Dv, page, cur_stream()),
        "qknorm_kv_write");
}

void window_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_table, const Tensor& tok_entry,
                      const Tensor& pos, int64_t window, double scale, double out_scale, Tensor out, int64_t impl, bool chunked,
                      const c10::optional<Tensor>& head_scale, const c10::optional<Tensor>& head_slope,
                      const c10::optional<Tensor>& gate, const c10::optional<Tensor>& head_sink, bool kv_shared, int64_t value_size,
                      int64_t heads, double softcap, int64_t keep_first, const c10::optional<Tensor>& dist_bias, int64_t v_div) {
  const bool single_token = block_table.size(0) == (q.dim() == 3 ? q.size(1) : q.size(0));
  c10::cuda::CUDAGuard guard(q.device());
  const int Hkv = static_cast<int>(k_cache.size(1)), page = static_cast<int>(k_cache.size(2)), D = static_cast<int>(k_cache.size(3));
  // kv_shared: the values are the first `value_size` columns of the key rows (one cache tensor, passed twice)
  const int Dv = kv_shared ? static_cast<int>(value_size) : static_cast<int>(v_cache.size(3));
  // q [T, Hq * D], or head-major [Hq, T, D'] (D' >= D columns per row, `heads` = Hq given): the layout a batched GEMM leaves
  const bool head_major = q.dim() == 3;
  const int T = static_cast<int>(head_major ? q.size(1) : q.size(0)), Hq = static_cast<int>(head_major ? q.size(0) : q.size(1) / D);
  TORCH_CHECK(block_table.dim() == 2 && out.dim() == 2 && out.size(0) == T && out.size(1) == static_cast<int64_t>(Hq) * Dv,
              "window_attention: shapes");
  NrlAttnMods md = {chunked ? 1 : 0, nullptr, nullptr, nullptr, 0, nullptr, 0, 0};
  if (head_major) {
    TORCH_CHECK(kv_shared && heads == Hq && q.size(2) >= D && q.stride(2) == 1 && q.stride(1) >= D, "window_attention: head-major queries [Hq, T, >= D] go with shared rows");
    md.q_head_stride = q.stride(0);
  }
  if (kv_shared) {
    TORCH_CHECK(v_cache.data_ptr() == k_cache.data_ptr() && Dv >= 1 && Dv <= D, "window_attention: shared rows need one cache and value_size <= D");
    md.kv_shared = 1;
  }
  if (head_sink.has_value()) {
    TORCH_CHECK(head_sink->numel() == Hq && head_sink->is_contiguous(), "window_attention: head_sink [Hq]");
    md.head_sink = f32(*head_sink, "head_sink");
  }
  if (head_scale.has_value()) {
    TORCH_CHECK(head_scale->numel() == Hq && head_scale->is_contiguous(), "window_attention: head_scale [Hq]");
    md.head_scale = f32(*head_scale, "head_scale");
  }
  if (head_slope.has_value()) {
    TORCH_CHECK(head_slope->numel() == Hq && head_slope->is_contiguous(), "window_attention: head_slope [Hq]");
    md.head_slope = f32(*head_slope, "head_slope");
  }
  if (gate.has_value()) {
    TORCH_CHECK(gate->dim() == 2 && gate->size(0) == T && gate->size(1) == Hq, "window_attention: gate [T, Hq]");
    md.gate = f32(*gate, "gate");
    md.gate_stride = gate->stride(0);
  }
  md.softcap = static_cast<float>(softcap);
  md.keep_first = static_cast<int>(keep_first);
  if (dist_bias.has_value()) {
    TORCH_CHECK(dist_bias->dim() == 2 && dist_bias->size(1) == Hq && dist_bias->size(0) >= 1 && dist_bias->is_contiguous(),
                "window_attention: dist_bias [distances, Hq]");
    md.dist_bias = f32(*dist_bias, "dist_bias");
    md.dist_max = static_cast<int>(dist_bias->size(0)) - 1;
  }
  if (v_div > 1) {
    TORCH_CHECK(!kv_shared && Hkv % v_div == 0 && v_cache.size(1) * v_div == Hkv, "window_attention: v_div key heads share one value head");
    md.v_div = static_cast<int>(v_div);
  } else {
    TORCH_CHECK(kv_shared || v_cache.size(1) == Hkv, "window_attention: key and value heads differ");
  }
  // a float result over bf16 pages (results that are combined further before they are rounded)
  const bool float_out = out.scalar_type() == at::kFloat && k_cache.scalar_type() == at::kBFloat16;
  if (float_out) {
    TORCH_CHECK(!kv_shared, "window_attention: a float result over bf16 pages is not available with shared key / value rows");
    md.out_float = out.data_ptr<float>();
    md.out_float_stride = out.stride(0);
  }
  // steps of single tokens on bf16 pages: cut the key walk into parts so that few sequences still fill the GPU
  int nsplit = 0;
  Tensor part;
  if (single_token && (impl == 0 || impl == 3) && k_cache.scalar_type() == at::kBFloat16 &&
      nrl_window_attention_mma_fits(out.data_ptr(), out.stride(0), Hq, Hkv, D, Dv, page) && !md.kv_shared) {
    nsplit = nrl_window_attention_splits(T, Hq, Hkv, static_cast<int>(window), static_cast<int>(block_table.size(1)), page);
    if (nsplit >= 1) part = at::empty({T, Hq, 4 * nsplit, Dv + 2}, q.options().dtype(at::kFloat));
  }
  if (single_token && (impl == 0 || impl == 3) && k_cache.scalar_type() == at::kBFloat16 && md.kv_shared && Hkv == 1 &&
      window >= (1 << 30) && nrl_latent_attention_mma_fits(out.data_ptr(), out.stride(0), D, Dv, page)) {
    nsplit = nrl_latent_attention_splits(T, Hq, Dv, static_cast<int>(block_table.size(1)));
    part = at::empty({T, Hq, 4 * nsplit, Dv + 2}, q.options().dtype(at::kFloat));
  }
  check(nrl_window_attention(f32(q, "q"), head_major ? q.stride(1) : q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), typed(k_cache, "k_cache"),
                             i32(block_table, "block_table"), static_cast<int>(block_table.size(1)), i32(tok_entry, "tok_entry"),
                             i32(pos, "pos"), static_cast<int>(window), static_cast<float>(scale), static_cast<float>(out_scale),
                             out.data_ptr(), out.stride(0), float_out ? 0 : typed(out, "out"), T, Hq, Hkv, D, Dv, page, single_token ? 1 : 0, static_cast<int>(impl),
                             nsplit, nsplit >= 1 ? part.data_ptr<float>() : nullptr, &md, cur_stream()),
        "window_attention");
}

void embed_streams(const Tensor& embed, const Tensor& tok, double scale, Tensor xs) {
  c10::cuda::CUDAGuard guard(xs.device());
  const int T = static_cast<int>(tok.numel());
  TORCH_CHECK(embed.dim() == 2 && embed.is_contiguous() && xs.dim() == 3 && xs.is_contiguous() && xs.size(0) == T && xs.size(2) == embed.size(1),
              "embed_streams: embed [V, W], xs [T, S, W]");
  check(nrl_embed_streams(embed.data_ptr(), typed(embed, "embed"), i32(tok, "tok"), static_cast<float>(scale), f32w(xs, "xs"), T,
                          static_cast<int>(xs.size(1)), static_cast<int>(xs.size(2)), cur_stream()),
        "embed_streams");
}

void hyper_boundary(Tensor xs, const c10::optional<Tensor>& o, const c10::optional<Tensor>& o_bias, const c10::optional<Tensor>& self_w,
                    const c10::optional<Tensor>& mix, const c10::optional<Tensor>& outw, const c10::optional<Tensor>& inw,
                    const c10::optional<Tensor>& ln_w, const c10::optional<Tensor>& ln_b, double eps, c10::optional<Tensor> h) {
  c10::cuda::CUDAGuard guard(xs.device());
  TORCH_CHECK(xs.dim() == 3 && xs.is_contiguous(), "hyper_boundary: xs [T, S, W] contiguous");
  const int T = static_cast<int>(xs.size(0)), S = static_cast<int>(xs.size(1)), W = static_cast<int>(xs.size(2));
  if (o.has_value()) TORCH_CHECK(o->is_contiguous() && o->dim() == 2 && o->size(0) == T && o->size(1) == W, "hyper_boundary: o [T, W]");
  if (o_bias.has_value()) TORCH_CHECK(o_bias->numel() == W && o_bias->is_contiguous(), "hyper_boundary: o_bias [W]");
  if (self_w.has_value()) TORCH_CHECK(self_w->numel() == T && self_w->is_contiguous() && h.has_value(), "hyper_boundary: self_w [T] goes with h");
  if (mix.has_value()) TORCH_CHECK(mix->numel() == S * S && mix->is_contiguous(), "hyper_boundary: mix [S, S]");
  if (outw.has_value()) TORCH_CHECK(outw->numel() == S && outw->is_contiguous(), "hyper_boundary: outw [S]");
  if (inw.has_value()) TORCH_CHECK(inw->numel() == S && inw->is_contiguous(), "hyper_boundary: inw [S]");
  if (h.has_value())
    TORCH_CHECK(h->is_contiguous() && h->dim() == 2 && h->size(0) == T && h->size(1) == W && ln_w.has_value() && ln_w->numel() == W &&
                    ln_w->is_contiguous() && (!ln_b.has_value() || (ln_b->numel() == W && ln_b->is_contiguous())),
                "hyper_boundary: h [T, W] goes with ln_w [W] (and ln_b [W])");
  auto opt = [](const c10::optional<Tensor>& t, const char* n) { return t.has_value() ? f32(*t, n) : nullptr; };
  check(nrl_hyper_boundary(f32w(xs, "xs"), S, opt(o, "o"), opt(o_bias, "o_bias"), opt(self_w, "self_w"), opt(mix, "mix"), opt(outw, "outw"),
                           opt(inw, "inw"), opt(ln_w, "ln_w"), opt(ln_b, "ln_b"), static_cast<float>(eps),
                           h.has_value() ? h->data_ptr() : nullptr, h.has_value() ? typed(*h, "h") : 1, T, W, cur_stream()),
        "hyper_boundary");
}

void mlstm_scan(const Tensor& qkv, int64_t col_q, int64_t col_k, int64_t col_v, int64_t col_i, int64_t col_f,
                const c10::optional<Tensor>& i_bias, const c10::optional<Tensor>& f_bias, double cap, double q_scale, Tensor state,
                Tensor mstate, Tensor o, Tensor m_out, const Tensor& cu, const Tensor& start, const Tensor& state_slot, int64_t impl) {
  c10::cuda::CUDAGuard guard(qkv.device());
  TORCH_CHECK(state.dim() == 4 && state.is_contiguous() && mstate.dim() == 2 && mstate.is_contiguous() && mstate.size(0) == state.size(0) &&
                  mstate.size(1) == state.size(1), "mlstm_scan: state [slots, heads, D, >= Dv + 1], mstate [slots, heads]");
  const int T = static_cast<int>(qkv.size(0)), heads = static_cast<int>(state.size(1)), D = static_cast<int>(state.size(2)),
            Cs = static_cast<int>(state.size(3)), E = static_cast<int>(start.numel());
  TORCH_CHECK(o.dim() == 2 && o.size(0) == T && o.size(1) % heads == 0, "mlstm_scan: o [T, heads * (Dv + 1)]");
  const int Dv = static_cast<int>(o.size(1) / heads) - 1;
  TORCH_CHECK(Dv >= 1 && Cs >= Dv + 1, "mlstm_scan: the state's rows hold at least Dv + 1 columns");
  const int64_t wd = qkv.size(1);
  TORCH_CHECK(qkv.dim() == 2 && Dv >= 1 && col_q >= 0 && col_q + heads * D <= wd && col_k >= 0 && col_k + heads * D <= wd && col_v >= 0 &&
                  col_v + heads * Dv <= wd && col_i >= 0 && col_i + heads <= wd && col_f >= 0 && col_f + heads <= wd, "mlstm_scan: columns");
  TORCH_CHECK(o.is_contiguous() && o.numel() == static_cast<int64_t>(T) * heads * (Dv + 1) && m_out.is_contiguous() &&
                  m_out.numel() == static_cast<int64_t>(T) * heads && cu.numel() == E + 1 && state_slot.numel() == E, "mlstm_scan: outputs / plan");
  if (i_bias.has_value()) TORCH_CHECK(i_bias->numel() == heads && i_bias->is_contiguous(), "mlstm_scan: i_bias [heads]");
  if (f_bias.has_value()) TORCH_CHECK(f_bias->numel() == heads && f_bias->is_contiguous(), "mlstm_scan: f_bias [heads]");
  check(nrl_mlstm_scan(f32(qkv, "qkv"), qkv.stride(0), static_cast<int>(col_q), static_cast<int>(col_k), static_cast<int>(col_v),
                       static_cast<int>(col_i), static_cast<int>(col_f), i_bias.has_value() ? f32(*i_bias, "i_bias") : nullptr,
                       f_bias.has_value() ? f32(*f_bias, "f_bias") : nullptr, static_cast<float>(cap), static_cast<float>(q_scale),
                       f32w(state, "state"), f32w(mstate, "mstate"), f32w(o, "o"), f32w(m_out, "m_out"), i32(cu, "cu"), i32(start, "start"),
                       i32(state_slot, "state_slot"), E, heads, D, Dv, Cs, T == E ? 1 : 0, static_cast<int>(impl), cur_stream()),
        "mlstm_scan");
}

void mlstm_out(const Tensor& o, const Tensor& m, const Tensor& gate, const Tensor& w, double eps, double scale, Tensor out, int64_t heads) {
  c10::cuda::CUDAGuard guard(o.device());
  const int T = static_cast<int>(m.numel() / heads);
  const int Dv = static_cast<int>(o.numel() / (static_cast<int64_t>(T > 0 ? T : 1) * heads)) - 1;
  TORCH_CHECK(o.is_contiguous() && m.is_contiguous() && (T == 0 || o.numel() == static_cast<int64_t>(T) * heads * (Dv + 1)), "mlstm_out: o / m");
  TORCH_CHECK(gate.dim() == 2 && gate.size(0) == T && gate.size(1) == heads * Dv && w.numel() == heads * Dv && w.is_contiguous() &&
                  out.dim() == 2 && out.size(0) == T && out.size(1) == heads * Dv, "mlstm_out: gate / w / out [.., heads * Dv]");
  check(nrl_mlstm_out(f32(o, "o"), f32(m, "m"), f32(gate, "gate"), gate.stride(0), f32(w, "w"), static_cast<float>(eps),
                      static_cast<float>(scale), out.data_ptr(), out.stride(0), typed(out, "out"), T, static_cast<int>(heads), Dv, cur_stream()),
        "mlstm_out");
}

void rot_kv_write(Tensor q, const c10::optional<Tensor>& q_bias, const c10::optional<Tensor>& k, const c10::optional<Tensor>& k_bias,
                  const c10::optional<Tensor>& v, const c10::optional<Tensor>& freq, int64_t rdims, double mult, bool interleaved,
                  bool unit_norm, const c10::optional<Tensor>& q_norm_w, const c10::optional<Tensor>& k_norm_w, double eps, const Tensor& pos,
                  const Tensor& kv_slot, Tensor k_cache, Tensor v_cache) {
  c10::cuda::CUDAGuard guard(q.device());
  const int cf = typed(k_cache, "k_cache");
  TORCH_CHECK(typed(v_cache, "v_cache") == cf && k_cache.dim() == 4 && v_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(),
              "rot_kv_write: caches [pages, heads, page, size] of one type");
  const int T = static_cast<int>(q.size(0)), Hk = static_cast<int>(k_cache.size(1)), page = static_cast<int>(k_cache.size(2)),
            D = static_cast<int>(k_cache.size(3)), Hv = static_cast<int>(v_cache.size(1)), Dv = static_cast<int>(v_cache.size(3));
  TORCH_CHECK(q.dim() == 2 && q.size(1) % D == 0, "rot_kv_write: q [T, Hq * D]");
  const int Hq = static_cast<int>(q.size(1)) / D;
  if (k.has_value()) TORCH_CHECK(k->dim() == 2 && k->size(0) == T && k->size(1) == static_cast<int64_t>(Hk) * D, "rot_kv_write: k [T, Hk * D]");
  if (v.has_value()) TORCH_CHECK(k.has_value() && v->dim() == 2 && v->size(0) == T && v->size(1) == static_cast<int64_t>(Hv) * Dv, "rot_kv_write: v [T, Hv * Dv]");
  if (q_bias.has_value()) TORCH_CHECK(q_bias->numel() == static_cast<int64_t>(Hq) * D && q_bias->is_contiguous(), "rot_kv_write: q_bias");
  if (k_bias.has_value()) TORCH_CHECK(k_bias->numel() == static_cast<int64_t>(Hk) * D && k_bias->is_contiguous(), "rot_kv_write: k_bias");
  if (q_norm_w.has_value()) TORCH_CHECK(q_norm_w->numel() == D && q_norm_w->is_contiguous(), "rot_kv_write: q_norm_w [D]");
  if (k_norm_w.has_value()) TORCH_CHECK(k_norm_w->numel() == D && k_norm_w->is_contiguous(), "rot_kv_write: k_norm_w [D]");
  if (rdims > 0)
    TORCH_CHECK(freq.has_value() && freq->is_cuda() && freq->scalar_type() == torch::kFloat64 && freq->is_contiguous() && freq->numel() == rdims / 2,
                "rot_kv_write: freq double [rdims / 2]");
  check(nrl_rot_kv_write(f32w(q, "q"), q.stride(0), q_bias.has_value() ? f32(*q_bias, "q_bias") : nullptr, k.has_value() ? f32(*k, "k") : nullptr,
                         k.has_value() ? k->stride(0) : 0, k_bias.has_value() ? f32(*k_bias, "k_bias") : nullptr,
                         v.has_value() ? f32(*v, "v") : nullptr, v.has_value() ? v->stride(0) : 0,
                         rdims > 0 ? freq->data_ptr<double>() : nullptr, static_cast<int>(rdims), static_cast<float>(mult), interleaved ? 1 : 0,
                         unit_norm ? 1 : 0, q_norm_w.has_value() ? f32(*q_norm_w, "q_norm_w") : nullptr,
                         k_norm_w.has_value() ? f32(*k_norm_w, "k_norm_w") : nullptr, static_cast<float>(eps), i32(pos, "pos"),
                         i32(kv_slot, "kv_slot"), k_cache.data_ptr(), v_cache.data_ptr(), cf, page, T, Hq, Hk, Hv, D, Dv, cur_stream()),
        "rot_kv_write");
}

void diff_combine(const Tensor& a, double lambda, double post, double eps, const c10::optional<Tensor>& gate, double out_scale, Tensor out,
                  int64_t heads, int64_t kv_heads) {
  c10::cuda::CUDAGuard guard(a.device());
  const int T = static_cast<int>(a.size(0));
  TORCH_CHECK(a.dim() == 2 && out.dim() == 2 && out.size(0) == T && a.size(1) == 2 * out.size(1) && out.size(1) % heads == 0,
              "diff_combine: a [T, 2 H Dv], out [T, H Dv]");
  const int Dv = static_cast<int>(out.size(1) / heads);
  if (gate.has_value()) TORCH_CHECK(gate->dim() == 2 && gate->size(0) == T && gate->size(1) == out.size(1), "diff_combine: gate [T, H Dv]");
  check(nrl_diff_combine(a.data_ptr(), a.stride(0), typed(a, "a"), static_cast<float>(lambda), static_cast<float>(post), static_cast<float>(eps),
                         gate.has_value() ? f32(*gate, "gate") : nullptr, gate.has_value() ? gate->stride(0) : 0, static_cast<float>(out_scale),
                         out.data_ptr(), out.stride(0), typed(out, "out"), T, static_cast<int>(heads), static_cast<int>(kv_heads), Dv,
                         cur_stream()),
        "diff_combine");
}

void kv_write_blend(const Tensor& k, Tensor v, const c10::optional<Tensor>& v_other, const c10::optional<Tensor>& lambda, Tensor k_cache,
                    Tensor v_cache, const Tensor& kv_slot) {
  c10::cuda::CUDAGuard guard(k.device());
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(), "kv_write_blend: caches");
  const int Hkv = static_cast<int>(k_cache.size(1)), page = static_cast<int>(k_cache.size(2)), D = static_cast<int>(k_cache.size(3));
  const int Dv = static_cast<int>(v_cache.size(3));
  const int T = static_cast<int>(k.size(0));
  TORCH_CHECK(k.dim() == 2 && v.dim() == 2 && v.size(0) == T && k.size(1) == static_cast<int64_t>(Hkv) * D &&
                  v.size(1) == static_cast<int64_t>(Hkv) * Dv && kv_slot.numel() >= T, "kv_write_blend: shapes");
  TORCH_CHECK(v_other.has_value() == lambda.has_value(), "kv_write_blend: v_other and lambda go together");
  if (v_other.has_value())
    TORCH_CHECK(v_other->dim() == 2 && v_other->size(0) == T && v_other->size(1) == v.size(1) && lambda->numel() == 1,
                "kv_write_blend: v_other like v, lambda one number");
  const int cf = typed(k_cache, "k_cache");
  TORCH_CHECK(typed(v_cache, "v_cache") == cf, "kv_write_blend: cache types differ");
  check(nrl_kv_write_blend(f32(k, "k"), k.stride(0), f32w(v, "v"), v.stride(0), v_other.has_value() ? f32(*v_other, "v_other") : nullptr,
                           v_other.has_value() ? v_other->stride(0) : 0, lambda.has_value() ? f32(*lambda, "lambda") : nullptr,
                           k_cache.data_ptr(), v_cache.data_ptr(), cf, i32(kv_slot, "kv_slot"), T, Hkv, D, Dv, page, cur_stream()),
        "kv_write_blend");
}

void embed_hashed(const Tensor& embed, const c10::optional<Tensor>& pair, const Tensor& tok, const Tensor& cu, const Tensor& tok_entry,
                  const Tensor& start, const Tensor& state_slot, const c10::optional<Tensor>& prev_state, double scale, int64_t mul_prev,
                  int64_t mul_cur, int64_t buckets, Tensor out) {
  c10::cuda::CUDAGuard guard(out.device());
  const int wf = typed(embed, "embed");
  const int T = static_cast<int>(tok.numel()), W = static_cast<int>(embed.size(1)), E = static_cast<int>(start.numel());
  TORCH_CHECK(embed.is_contiguous() && out.is_contiguous() && out.size(0) >= T && out.size(1) == W, "embed_hashed: shapes");
  TORCH_CHECK(pair.has_value() == prev_state.has_value(), "embed_hashed: the pair table needs the per-slot previous tokens");
  if (pair.has_value()) {
    TORCH_CHECK(typed(*pair, "pair") == wf && pair->is_contiguous() && pair->size(1) == W && pair->size(0) == buckets + 1 && buckets > 0,
                "embed_hashed: pair table [buckets + 1, W]");
    TORCH_CHECK(prev_state->scalar_type() == torch::kInt32 && prev_state->is_contiguous(), "embed_hashed: prev_state int32 [slots]");
  }
  check(nrl_embed_hashed(embed.data_ptr(), pair.has_value() ? pair->data_ptr() : nullptr, wf, i32(tok, "tok"), i32(cu, "cu"),
                         i32(tok_entry, "tok_entry"), i32(start, "start"), i32(state_slot, "state_slot"),
                         prev_state.has_value() ? prev_state->data_ptr<int>() : nullptr, static_cast<float>(scale), mul_prev, mul_cur,
                         buckets, f32w(out, "out"), T, E, W, cur_stream()),
        "embed_hashed");
}

void group_norm_residual(Tensor x, const c10::optional<Tensor>& o, const c10::optional<Tensor>& gate, const c10::optional<Tensor>& gate_bias,
                         const c10::optional<Tensor>& w_post, const c10::optional<Tensor>& w_pre, int64_t groups, double eps,
                         const c10::optional<Tensor>& h) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous(), "group_norm_residual: x [T, W] contiguous");
  const int T = static_cast<int>(x.size(0)), W = static_cast<int>(x.size(1));
  if (o.has_value()) TORCH_CHECK(o->is_contiguous() && o->size(0) == T && o->size(1) == W && w_post.has_value() && w_post->numel() == W, "group_norm_residual: o / w_post");
  if (gate.has_value()) TORCH_CHECK(gate->dim() == 2 && gate->size(0) == T && gate->size(1) == W, "group_norm_residual: gate [T, W]");
  if (gate_bias.has_value()) TORCH_CHECK(gate_bias->numel() == W, "group_norm_residual: gate_bias [W]");
  if (h.has_value()) TORCH_CHECK(h->is_contiguous() && h->size(0) == T && h->size(1) == W && w_pre.has_value() && w_pre->numel() == W, "group_norm_residual: h / w_pre");
  check(nrl_group_norm_residual(f32w(x, "x"), o.has_value() ? f32(*o, "o") : nullptr, gate.has_value() ? f32(*gate, "gate") : nullptr,
                                gate.has_value() ? gate->stride(0) : 0, gate_bias.has_value() ? f32(*gate_bias, "gate_bias") : nullptr,
                                w_post.has_value() ? f32(*w_post, "w_post") : nullptr, w_pre.has_value() ? f32(*w_pre, "w_pre") : nullptr,
                                static_cast<int>(groups), static_cast<float>(eps), h.has_value() ? h->data_ptr() : nullptr,
                                h.has_value() ? typed(*h, "h") : 1, T, W, cur_stream()),
        "group_norm_residual");
}

void moe_route(const Tensor& router, const c10::optional<Tensor>& router_bias, int64_t top, const c10::optional<Tensor>& gu, int64_t ff,
               const c10::optional<Tensor>& act, const c10::optional<Tensor>& ids, const c10::optional<Tensor>& wts) {
  c10::cuda::CUDAGuard guard(router.device());
  TORCH_CHECK(router.dim() == 2, "moe_route: router [T, E]");
  const int T = static_cast<int>(router.size(0)), E = static_cast<int>(router.size(1));
  if (router_bias.has_value()) TORCH_CHECK(router_bias->numel() == E, "moe_route: router_bias [E]");
  TORCH_CHECK(act.has_value() == gu.has_value(), "moe_route: gu and act go together");
  if (act.has_value())
    TORCH_CHECK(gu->dim() == 2 && gu->size(0) == T && gu->size(1) == static_cast<int64_t>(E) * 2 * ff && act->dim() == 2 &&
                    act->size(0) == T && act->size(1) == static_cast<int64_t>(E) * ff, "moe_route: gu [T, E*2ff], act [T, E*ff]");
  if (ids.has_value()) TORCH_CHECK(ids->scalar_type() == torch::kInt32 && ids->is_contiguous() && ids->numel() == static_cast<int64_t>(T) * top, "moe_route: ids int32 [T, top]");
  if (wts.has_value()) TORCH_CHECK(ids.has_value() && wts->is_contiguous() && wts->numel() == static_cast<int64_t>(T) * top, "moe_route: wts float [T, top]");
  Tensor wt = wts.has_value() ? *wts : Tensor();
  check(nrl_moe_route(f32(router, "router"), router.stride(0), router_bias.has_value() ? f32(*router_bias, "router_bias") : nullptr, E,
                      static_cast<int>(top), gu.has_value() ? f32(*gu, "gu") : nullptr, gu.has_value() ? gu->stride(0) : 0,
                      static_cast<int>(ff), act.has_value() ? act->data_ptr() : nullptr, act.has_value() ? act->stride(0) : 0,
                      act.has_value() ? typed(*act, "act") : 1, ids.has_value() ? ids->data_ptr<int>() : nullptr,
                      wts.has_value() ? f32w(wt, "wts") : nullptr, T, cur_stream()),
        "moe_route");
}

// ---- stream with the norm on the sublayer's output, token-side input, softmax-over-all routing ----
void embed_norm(const Tensor& embed, const Tensor& tok, const Tensor& w, double eps, Tensor x, Tensor h) {
  c10::cuda::CUDAGuard guard(x.device());
  const int T = static_cast<int>(tok.numel()), W = static_cast<int>(embed.size(1));
  TORCH_CHECK(embed.dim() == 2 && embed.is_contiguous() && x.is_contiguous() && h.is_contiguous() && x.size(0) >= T && x.size(1) == W &&
                  h.size(0) >= T && h.size(1) == W && w.numel() == W, "embed_norm: shapes");
  check(nrl_embed_norm(embed.data_ptr(), typed(embed, "embed"), i32(tok, "tok"), f32(w, "w"), static_cast<float>(eps), f32w(x, "x"),
                       h.data_ptr(), typed(h, "h"), T, W, cur_stream()),
        "embed_norm");
}

void post_norm_residual(Tensor x, const Tensor& o, const c10::optional<Tensor>& self_w, const Tensor& w_post,
                        const c10::optional<Tensor>& w_pre, double eps, const c10::optional<Tensor>& h) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous(), "post_norm_residual: x [T, W] contiguous");
  const int T = static_cast<int>(x.size(0)), W = static_cast<int>(x.size(1));
  TORCH_CHECK(o.is_contiguous() && o.dim() == 2 && o.size(0) == T && o.size(1) == W && w_post.numel() == W, "post_norm_residual: o / w_post");
  if (self_w.has_value()) TORCH_CHECK(self_w->is_contiguous() && self_w->numel() == T, "post_norm_residual: self_w [T]");
  if (w_pre.has_value()) TORCH_CHECK(w_pre->numel() == W && h.has_value(), "post_norm_residual: w_pre [W] goes with h");
  if (h.has_value()) TORCH_CHECK(h->is_contiguous() && h->size(0) == T && h->size(1) == W, "post_norm_residual: h [T, W]");
  check(nrl_post_norm_residual(f32w(x, "x"), f32(o, "o"), self_w.has_value() ? f32(*self_w, "self_w") : nullptr, f32(w_post, "w_post"),
                               w_pre.has_value() ? f32(*w_pre, "w_pre") : nullptr, static_cast<float>(eps),
                               h.has_value() ? h->data_ptr() : nullptr, h.has_value() ? typed(*h, "h") : 1, T, W, cur_stream()),
        "post_norm_residual");
}

void side_gate(const Tensor& u, const Tensor& table, int64_t col0, const Tensor& tok, Tensor out, int64_t C) {
  c10::cuda::CUDAGuard guard(u.device());
  const int T = static_cast<int>(u.size(0));
  TORCH_CHECK(u.dim() == 2 && u.size(1) >= C && table.dim() == 2 && col0 >= 0 && col0 + C <= table.size(1) && out.dim() == 2 &&
                  out.size(0) == T && out.size(1) >= C && tok.numel() >= T, "side_gate: shapes");
  f32(u, "u");
  check(nrl_side_gate(u.data_ptr<float>(), u.stride(0), table.data_ptr(), table.stride(0), typed(table, "table"), static_cast<int>(col0),
                      i32(tok, "tok"), out.data_ptr(), out.stride(0), typed(out, "out"), T, static_cast<int>(C),
                      static_cast<int>(out.size(1)), cur_stream()),
        "side_gate");
}

void swiglu_cols(const Tensor& in, const c10::optional<Tensor>& rgate, Tensor out) {
  c10::cuda::CUDAGuard guard(in.device());
  TORCH_CHECK(in.dim() == 2 && out.dim() == 2 && in.size(0) == out.size(0) && in.size(1) == 2 * out.size(1), "swiglu_cols: in [T, 2 C], out [T, C]");
  if (rgate.has_value()) TORCH_CHECK(rgate->dim() == 2 && rgate->size(0) == in.size(0) && rgate->size(1) == 1, "swiglu_cols: rgate [T, 1]");
  check(nrl_swiglu_cols(f32(in, "in"), in.stride(0), rgate.has_value() ? f32(*rgate, "rgate") : nullptr,
                        rgate.has_value() ? rgate->stride(0) : 0, out.data_ptr(), out.stride(0), typed(out, "out"),
                        static_cast<int>(in.size(0)), static_cast<int>(out.size(1)), cur_stream()),
        "swiglu_cols");
}

void moe_route_all(const Tensor& router, const c10::optional<Tensor>& correction, int64_t n_real, int64_t top, double route_scale,
                   int64_t groups, int64_t keep, const c10::optional<Tensor>& gu, int64_t ff, const c10::optional<Tensor>& act, const c10::optional<Tensor>& ids,
                   const c10::optional<Tensor>& wts, const c10::optional<Tensor>& self_w) {
  c10::cuda::CUDAGuard guard(router.device());
  TORCH_CHECK(router.dim() == 2, "moe_route_all: router [T, E]");
  const int T = static_cast<int>(router.size(0)), E = static_cast<int>(router.size(1));
  if (correction.has_value()) TORCH_CHECK(correction->numel() == E, "moe_route_all: correction [E]");
  TORCH_CHECK(act.has_value() == gu.has_value(), "moe_route_all: gu and act go together");
  if (act.has_value())
    TORCH_CHECK(gu->dim() == 2 && gu->size(0) == T && gu->size(1) == n_real * 2 * ff && act->dim() == 2 && act->size(0) == T &&
                    act->size(1) == n_real * ff, "moe_route_all: gu [T, n_real*2ff], act [T, n_real*ff]");
  if (ids.has_value()) TORCH_CHECK(ids->scalar_type() == torch::kInt32 && ids->is_contiguous() && ids->numel() == static_cast<int64_t>(T) * top, "moe_route_all: ids int32 [T, top]");
  if (wts.has_value()) TORCH_CHECK(wts->is_contiguous() && wts->numel() == static_cast<int64_t>(T) * top, "moe_route_all: wts float [T, top]");
  if (self_w.has_value()) TORCH_CHECK(self_w->is_contiguous() && self_w->numel() == T, "moe_route_all: self_w float [T]");
  Tensor wt = wts.has_value() ? *wts : Tensor(), sw = self_w.has_value() ? *self_w : Tensor();
  check(nrl_moe_route_all(f32(router, "router"), router.stride(0), correction.has_value() ? f32(*correction, "correction") : nullptr, E,
                          static_cast<int>(n_real), static_cast<int>(top), static_cast<float>(route_scale), static_cast<int>(groups),
                          static_cast<int>(keep), gu.has_value() ? f32(*gu, "gu") : nullptr, gu.has_value() ? gu->stride(0) : 0, static_cast<int>(ff),
                          act.has_value() ? act->data_ptr() : nullptr, act.has_value() ? act->stride(0) : 0,
                          act.has_value() ? typed(*act, "act") : 1, ids.has_value() ? ids->data_ptr<int>() : nullptr,
                          wts.has_value() ? f32w(wt, "wts") : nullptr, self_w.has_value() ? f32w(sw, "self_w") : nullptr, T, cur_stream()),
        "moe_route_all");
}

void gla_prep(Tensor qkv, const Tensor& a_raw, const c10::optional<Tensor>& a_bias, double tau, Tensor decay, int64_t heads, int64_t D) {
  c10::cuda::CUDAGuard guard(qkv.device());
  const int T = static_cast<int>(qkv.size(0));
  const int64_t n = heads * D;
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) >= n && a_raw.dim() == 2 && a_raw.size(0) == T && a_raw.size(1) == n && decay.is_contiguous() &&
                  decay.numel() == static_cast<int64_t>(T) * n, "gla_prep: shapes");
  if (a_bias.has_value()) TORCH_CHECK(a_bias->numel() == n, "gla_prep: a_bias [heads * D]");
  check(nrl_gla_prep(f32w(qkv, "qkv"), qkv.stride(0), f32(a_raw, "a_raw"), a_raw.stride(0), a_bias.has_value() ? f32(*a_bias, "a_bias") : nullptr,
                     static_cast<float>(tau), f32w(decay, "decay"), T, static_cast<int>(heads), static_cast<int>(D), cur_stream()),
        "gla_prep");
}

void latent_kv_write(const Tensor& q, int64_t H, int64_t dn, int64_t dr, const Tensor& dkv, const Tensor& w, double eps, const Tensor& freq,
                     int64_t rdims, double mult, bool interleaved, const Tensor& pos, const Tensor& kv_slot, Tensor cache, Tensor qa,
                     const c10::optional<Tensor>& qn) {
  c10::cuda::CUDAGuard guard(q.device());
  const int T = static_cast<int>(q.size(0));
  const int64_t rank = w.numel(), D = rank + dr;
  TORCH_CHECK(cache.dim() == 4 && cache.is_contiguous() && cache.size(1) == 1 && cache.size(3) == D, "latent_kv_write: cache [pages, 1, page, rank + dr]");
  TORCH_CHECK(q.dim() == 2 && q.size(1) == H * (dn + dr) && dkv.dim() == 2 && dkv.size(0) == T && dkv.size(1) == D && pos.numel() >= T &&
                  kv_slot.numel() >= T, "latent_kv_write: shapes");
  // qa: [T, H * D], or head-major [H, T, D]
  TORCH_CHECK((qa.dim() == 2 && qa.size(0) == T && qa.size(1) == H * D) ||
                  (qa.dim() == 3 && qa.size(0) == H && qa.size(1) == T && qa.size(2) == D && qa.stride(2) == 1), "latent_kv_write: qa [T, H * D] or [H, T, D]");
  const long sqa = qa.dim() == 3 ? qa.stride(1) : qa.stride(0), sha = qa.dim() == 3 ? qa.stride(0) : D;
  if (qn.has_value())
    TORCH_CHECK(qn->scalar_type() == torch::kBFloat16 && qn->is_contiguous() && qn->numel() == static_cast<int64_t>(H) * T * dn,
                "latent_kv_write: qn bf16 [H, T, dn]");
  TORCH_CHECK(freq.is_cuda() && freq.scalar_type() == torch::kFloat64 && freq.is_contiguous() && freq.numel() == rdims / 2 && rdims % 2 == 0 &&
                  rdims <= dr, "latent_kv_write: freq double [rdims / 2]");
  check(nrl_latent_kv_write(f32(q, "q"), q.stride(0), static_cast<int>(H), static_cast<int>(dn), static_cast<int>(dr), f32(dkv, "dkv"),
                            dkv.stride(0), static_cast<int>(rank), f32(w, "w"), static_cast<float>(eps), freq.data_ptr<double>(),
                            static_cast<int>(rdims), static_cast<float>(mult), interleaved ? 1 : 0, i32(pos, "pos"), i32(kv_slot, "kv_slot"),
                            cache.data_ptr(), typed(cache, "cache"), static_cast<int>(cache.size(2)), f32w(qa, "qa"), sqa, sha,
                            qn.has_value() ? qn->data_ptr() : nullptr, T, cur_stream()),
        "latent_kv_write");
}

// ---- mixture of experts, grouped form ----
std::vector<Tensor> moe_plan(const Tensor& ids, int64_t E, int64_t tile_rows, int64_t n_real) {
  c10::cuda::CUDAGuard guard(ids.device());
  TORCH_CHECK(ids.dim() == 2 && ids.scalar_type() == torch::kInt32 && ids.is_contiguous(), "moe_plan: ids int32 [T, top]");
  const int R = static_cast<int>(ids.numel()), top = static_cast<int>(ids.size(1));
  const int64_t max_tiles = (R + tile_rows - 1) / tile_rows + E;
  auto opt = ids.options();
  Tensor slot_of = at::empty({R}, opt), row_token = at::empty({R}, opt), seg = at::empty({E + 1}, opt);
  Tensor tiles = at::zeros({max_tiles, 3}, opt), num_tiles = at::zeros({1}, opt);
  check(nrl_moe_plan(i32(ids, "ids"), R, top, static_cast<int>(E), static_cast<int>(n_real < 0 ? E : n_real), static_cast<int>(tile_rows), slot_of.data_ptr<int>(),
                     row_token.data_ptr<int>(), seg.data_ptr<int>(), tiles.data_ptr<int>(), num_tiles.data_ptr<int>(), cur_stream()),
        "moe_plan");
  return {slot_of, row_token, seg, tiles, num_tiles};
}

void gather_rows(const Tensor& in, const Tensor& row_token, Tensor out) {
  c10::cuda::CUDAGuard guard(in.device());
  TORCH_CHECK(in.dim() == 2 && out.dim() == 2 && in.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16 &&
                  in.stride(1) == 1 && out.is_contiguous() && out.size(1) == in.size(1) && out.size(0) == row_token.numel(),
              "gather_rows: bf16 in [T, W], out [R, W] contiguous");
  check(nrl_gather_rows16(in.data_ptr(), in.stride(0), i32(row_token, "row_token"), out.data_ptr(), static_cast<int>(out.size(0)),
                          static_cast<int>(in.size(1)), cur_stream()),
        "gather_rows");
}

void swiglu_rows(const Tensor& gu, Tensor act) {
  c10::cuda::CUDAGuard guard(gu.device());
  TORCH_CHECK(gu.dim() == 2 && act.dim() == 2 && act.scalar_type() == torch::kBFloat16 && act.stride(1) == 1 && gu.size(0) == act.size(0) &&
                  gu.size(1) == 2 * act.size(1), "swiglu_rows: gu float [R, 2 ff], act bf16 [R, ff]");
  check(nrl_swiglu_rows(f32(gu, "gu"), gu.stride(0), act.data_ptr(), act.stride(0), static_cast<int>(gu.size(0)),
                        static_cast<int>(act.size(1)), cur_stream()),
        "swiglu_rows");
}

void moe_combine(const Tensor& y, const Tensor& slot_of, const Tensor& wts, Tensor out) {
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.dim() == 2 && out.dim() == 2 && wts.dim() == 2 && wts.is_contiguous() && out.size(0) == wts.size(0) &&
                  out.size(1) == y.size(1) && slot_of.numel() == wts.numel() && y.size(0) == wts.numel(), "moe_combine: shapes");
  check(nrl_moe_combine(f32(y, "y"), y.stride(0), i32(slot_of, "slot_of"), f32(wts, "wts"), static_cast<int>(wts.size(1)),
                        f32w(out, "out"), out.stride(0), static_cast<int>(out.size(0)), static_cast<int>(out.size(1)), cur_stream()),
        "moe_combine");
}

// Rows sorted by expert: a bf16 [R, K], b bf16 [E * N, K]; tiles / num_tiles from moe_plan (128-row tiles).
//   out float [R, N] = a[r] . b[expert(r)]^T,  or
//   act bf16 [R, N / 2] = silu(gate) * up with b's rows interleaved per 32 features ([32 gate rows | 32 up rows], N % 64 == 0).
void gemm_tc_grouped(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& out, const Tensor& tiles, const Tensor& num_tiles,
                     int64_t block_n, const c10::optional<Tensor>& act) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == torch::kBFloat16 && b.scalar_type() == torch::kBFloat16 && a.dim() == 2 &&
                  b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_tc_grouped: bf16 2D operands with unit inner stride");
  TORCH_CHECK((a.stride(0) * 2) % 16 == 0 && (b.stride(0) * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0, "gemm_tc_grouped: 16-byte aligned rows");
  TORCH_CHECK(out.has_value() != act.has_value(), "gemm_tc_grouped: give either the float result or the activation output");
  const int64_t R = a.size(0), K = a.size(1), N = out.has_value() ? out->size(1) : 2 * act->size(1);
  TORCH_CHECK(b.size(1) == K && K % 8 == 0 && N % 8 == 0 && b.size(0) % N == 0, "gemm_tc_grouped: b [E * N, K], K and N multiples of 8");
  TORCH_CHECK(tiles.scalar_type() == torch::kInt32 && tiles.is_contiguous() && tiles.dim() == 2 && tiles.size(1) == 3 &&
                  num_tiles.scalar_type() == torch::kInt32 && num_tiles.numel() == 1, "gemm_tc_grouped: tile table");
  nrl::tc::TcParams p{};
  if (out.has_value()) {
    TORCH_CHECK(out->scalar_type() == torch::kFloat32 && out->dim() == 2 && out->size(0) == R && out->stride(1) == 1 &&
                    out->stride(0) % 4 == 0 && (reinterpret_cast<uintptr_t>(out->data_ptr()) & 15) == 0,
                "gemm_tc_grouped: out float [R, N], 16-byte aligned rows");
    p.out_f32 = out->data_ptr<float>();
    p.out_f32_stride = out->stride(0);
  } else {
    TORCH_CHECK(act->scalar_type() == torch::kBFloat16 && act->dim() == 2 && act->size(0) == R && act->stride(1) == 1 &&
                    act->stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(act->data_ptr()) & 15) == 0 && N % 64 == 0,
                "gemm_tc_grouped: act bf16 [R, N / 2], 16-byte aligned rows, N a multiple of 64");
    p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(act->data_ptr());
    p.out_stride = act->stride(0);
  }
  if (R == 0) return;
  const int bn = block_n > 0 ? static_cast<int>(block_n) : (N <= 64 ? 64 : 128);
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap maps[2];
  maps[0] = nrl::make_tma_2d(a.data_ptr(), a.size(0), a.size(1), a.stride(0) * 2, 128, 64, BF, 2);
  maps[1] = nrl::make_tma_2d(b.data_ptr(), b.size(0), b.size(1), b.stride(0) * 2, bn, 64, BF, 2);
  p.M = static_cast<int>(R); p.N = static_cast<int>(N); p.K = static_cast<int>(K); p.K2 = 0;
  p.alpha = 1.f;
  p.grp_tiles = tiles.data_ptr<int>();
  p.grp_num_tiles = num_tiles.data_ptr<int>();
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  check(nrl_gemm_tc_grouped(maps, &p, bn, static_cast<int>(tiles.size(0)), sms, cur_stream()), "gemm_tc_grouped");
}

}  // namespace

namespace nrl {
void bind_hybrid(pybind11::module_& m) {
  m.def("moe_plan", &moe_plan, "sort (token, choice) pairs by expert: slot_of, row_token, seg, tiles, num_tiles (experts >= n_real get no tiles)",
        pybind11::arg("ids"), pybind11::arg("E"), pybind11::arg("tile_rows"), pybind11::arg("n_real") = -1);
  m.def("gather_rows", &gather_rows, "out[r] = in[row_token[r]] (bf16 rows)");
  m.def("swiglu_rows", &swiglu_rows, "act = silu(gu[:, :ff]) * gu[:, ff:] (float in, bf16 out)");
  m.def("moe_combine", &moe_combine, "out[t] = sum_k wts[t, k] y[slot_of[t, k]]");
  m.def("gemm_tc_grouped", &gemm_tc_grouped, "grouped tcgen05 GEMM over rows sorted by expert: float32 out, or fused SwiGLU bf16 out",
        pybind11::arg("a"), pybind11::arg("b"), pybind11::arg("out"), pybind11::arg("tiles"), pybind11::arg("num_tiles"),
        pybind11::arg("block_n") = 0, pybind11::arg("act") = pybind11::none());
  m.def("embed_norm", &embed_norm, "x = rmsnorm(embed[tok]) * w (float), h = x (typed)");
  m.def("post_norm_residual", &post_norm_residual, "x += rmsnorm(o + self_w x) * w_post; h = w_pre ? rmsnorm(x) * w_pre : x");
  m.def("side_gate", &side_gate, "out = gelu_tanh(u) * table[tok, col0:col0 + C], zero padded");
  m.def("swiglu_cols", &swiglu_cols, "out = silu(in[:, :C]) * in[:, C:] * sigmoid(row gate)");
  m.def("moe_route_all", &moe_route_all, "routing by a softmax over all router outputs, with identity experts");
  m.def("gla_prep", &gla_prep, "q * D^-1/2 in place and per-channel decays sigmoid(z)^(1/tau) of gated linear attention");
  m.def("latent_kv_write", &latent_kv_write, "normed latent + rotated shared key part into the page; rotated query parts into the absorbed queries");
  m.def("embed_pos", &embed_pos, "x0 = embed[tok] + pos_table[pos] (float)");
  m.def("stream_norm", &stream_norm, "close a layer, form the depth-weighted stream and its single-gain RMS norm");
  m.def("act_cols", &act_cols, "typed out = act(float in): 0 copy, 1 relu^2");
  m.def("gated_part_rmsnorm", &gated_part_rmsnorm, "part-wise RMS norm with a silu / sigmoid gate before or after it");
  m.def("causal_conv", &causal_conv, "depthwise causal convolution (+ silu) with taps carried per state slot", pybind11::arg("in"),
        pybind11::arg("w"), pybind11::arg("bias"), pybind11::arg("state"), pybind11::arg("out"), pybind11::arg("cu"),
        pybind11::arg("tok_entry"), pybind11::arg("start"), pybind11::arg("state_slot"), pybind11::arg("in_bias") = pybind11::none(),
        pybind11::arg("act") = 1);
  m.def("ssd_scan", &ssd_scan, "state-space scan with a scalar decay per head, state carried per slot");
  m.def("delta_prep", &delta_prep, "unit q / k, beta and decays of the gated delta rule");
  m.def("delta_scan", &delta_scan, "gated delta rule scan, state carried per slot");
  m.def("qknorm_kv_write", &qknorm_kv_write, "per-head RMS norm of q (in place) and k (into the paged cache), v into the cache");
  m.def("window_attention", &window_attention, "sliding-window attention over the paged cache", pybind11::arg("q"),
        pybind11::arg("k_cache"), pybind11::arg("v_cache"), pybind11::arg("block_table"), pybind11::arg("tok_entry"), pybind11::arg("pos"),
        pybind11::arg("window"), pybind11::arg("scale"), pybind11::arg("out_scale"), pybind11::arg("out"), pybind11::arg("impl") = 0,
        pybind11::arg("chunked") = false, pybind11::arg("head_scale") = pybind11::none(), pybind11::arg("head_slope") = pybind11::none(),
        pybind11::arg("gate") = pybind11::none(), pybind11::arg("head_sink") = pybind11::none(), pybind11::arg("kv_shared") = false,
        pybind11::arg("value_size") = 0, pybind11::arg("heads") = 0, pybind11::arg("softcap") = 0.0, pybind11::arg("keep_first") = 0,
        pybind11::arg("dist_bias") = pybind11::none(), pybind11::arg("v_div") = 1);
  m.def("embed_streams", &embed_streams, "xs[t, s] = embed[tok[t]] * scale for every residual stream");
  m.def("hyper_boundary", &hyper_boundary, "close a sublayer over several mixed residual streams and layer-norm the next one's input");
  m.def("mlstm_scan", &mlstm_scan, "matrix memory with exponential gates and a running maximum, state carried per slot");
  m.def("mlstm_out", &mlstm_out, "normaliser division, per-head RMS norm, weight and sigmoid gate of the matrix memory's read-out");
  m.def("rot_kv_write", &rot_kv_write, "biased, rotated, optionally unit-normed queries (in place) and keys (into pages); values into pages");
  m.def("diff_combine", &diff_combine, "o = a1 - lambda a2 of two score maps, per-head RMS norm, gate");
  m.def("kv_write_blend", &kv_write_blend, "keys and (optionally blended) values of a step's tokens into their pages");
  m.def("embed_hashed", &embed_hashed, "x0 = embed[tok] * scale + pair[hash(previous token, token)] (float), previous tokens carried per slot");
  m.def("group_norm_residual", &group_norm_residual, "x += groupnorm(o * sigmoid(gate)) * w_post; h = groupnorm(x) * w_pre");
  m.def("moe_route", &moe_route, "top-k routing with softmax over the chosen logits; dense-form expert activations");
}
}  // namespace nrl
