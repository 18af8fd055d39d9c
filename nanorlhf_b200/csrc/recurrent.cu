// Recurrent token mixers with state carried per sequence slot: short causal convolution, state-space scan with a scalar
// decay per head, gated delta rule with a decay per head or per key channel.  One launch serves a whole engine step:
// every entry (a run of consecutive tokens of one sequence: a prompt portion or one decoded token) starts from the state
// its slot holds (zero when the sequence is new) and leaves the updated state there.  All arithmetic is float.
// Compiled WITHOUT fast-math.
#include <cuda_bf16.h>

#include "hybrid_kernels.h"

namespace {

constexpr int kMaxTaps = 16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------------------------------------------------
// causal convolution: thread per (token, channel)
// ---------------------------------------------------------------------------------------------------------------------
__global__ void causal_conv_kernel(const float* __restrict__ in, long si, const float* __restrict__ in_bias, int act,
                                   const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state, float* __restrict__ out, long so, const int* __restrict__ cu,
                                   const int* __restrict__ tok_entry, const int* __restrict__ start,
                                   const int* __restrict__ state_slot, long T, int C, int taps) {
  const long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  if (idx >= T * C) return;
  const long t = idx / C;
  const int c = static_cast<int>(idx - t * C);
  const int e = tok_entry[t];
  const long first = cu[e];
  const int local = static_cast<int>(t - first);
  const bool carried = start[e] > 0;
  const float* st = state + static_cast<long>(state_slot[e]) * (taps - 1) * C;
  float acc = bias != nullptr ? bias[c] : 0.f;
  const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = local - (taps - 1 - j);
    float x = 0.f;
    if (src >= 0) x = in[(first + src) * si + c] + ib;
    else if (carried) x = st[static_cast<long>(taps - 1 + src) * C + c];
    acc += w[static_cast<long>(c) * taps + j] * x;
  }
  out[t * so + c] = act ? silu(acc) : acc;
}

// thread per (channel, run of kConvTok consecutive tokens): the last taps-1 inputs slide through registers, so every input is
// read once (plus the history at the start of a run or of a sequence) and the taps' weights once per run
constexpr int kConvTok = 8;

template <int MAXT>
__global__ void causal_conv_run_kernel(const float* __restrict__ in, long si, const float* __restrict__ in_bias, int act,
                                       const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state, float* __restrict__ out, long so, const int* __restrict__ cu,
                                       const int* __restrict__ tok_entry, const int* __restrict__ start,
                                       const int* __restrict__ state_slot, int T, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t_begin = blockIdx.y * kConvTok, t_end = min(T, t_begin + kConvTok);
  float wv[MAXT], hist[MAXT];
#pragma unroll
  for (int j = 0; j < MAXT; ++j) {
    wv[j] = j < taps ? w[static_cast<long>(c) * taps + j] : 0.f;
    hist[j] = 0.f;
  }
  const float b = bias != nullptr ? bias[c] : 0.f;
  const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
  int e_prev = -1;
  for (int t = t_begin; t < t_end; ++t) {
    const int e = tok_entry[t];
    if (e != e_prev) {                                   // first token of the run, or another sequence begins: fetch the history
      const long first = cu[e];
      const int local = static_cast<int>(t - first);
      const bool carried = start[e] > 0;
      const float* st = state + static_cast<long>(state_slot[e]) * (taps - 1) * C;
#pragma unroll
      for (int j = 0; j < MAXT - 1; ++j) {
        if (j < taps - 1) {
          const int src = local - (taps - 1 - j);
          float x = 0.f;
          if (src >= 0) x = in[(first + src) * si + c] + ib;
          else if (carried) x = st[static_cast<long>(taps - 1 + src) * C + c];
          hist[j] = x;
        }
      }
      e_prev = e;
    }
    const float cur = in[static_cast<long>(t) * si + c] + ib;
    float acc = b;
#pragma unroll
    for (int j = 0; j < MAXT - 1; ++j)
      if (j < taps - 1) acc += wv[j] * hist[j];
#pragma unroll
    for (int j = 0; j < MAXT; ++j)
      if (j == taps - 1) acc += wv[j] * cur;
    out[static_cast<long>(t) * so + c] = act ? silu(acc) : acc;
#pragma unroll
    for (int j = 0; j < MAXT - 1; ++j) {
      if (j < taps - 2) hist[j] = hist[j + 1];
      else if (j == taps - 2) hist[j] = cur;
    }
  }
}

// thread per (entry, channel): the slot keeps the last taps-1 inputs of the sequence, oldest first
__global__ void causal_conv_carry_kernel(const float* __restrict__ in, long si, const float* __restrict__ in_bias,
                                         float* __restrict__ state, const int* __restrict__ cu,
                                         const int* __restrict__ start, const int* __restrict__ state_slot, int E, int C, int taps) {
  const long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<long>(E) * C) return;
  const int e = static_cast<int>(idx / C);
  const int c = static_cast<int>(idx - static_cast<long>(e) * C);
  const long first = cu[e];
  const int n = cu[e + 1] - cu[e];
  const bool carried = start[e] > 0;
  float* st = state + static_cast<long>(state_slot[e]) * (taps - 1) * C;
  float keep[kMaxTaps];
  const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j) {
    if (j < taps - 1) {
      const int src = n - (taps - 1) + j;
      float x = 0.f;
      if (src >= 0) x = in[(first + src) * si + c] + ib;
      else if (carried) x = st[static_cast<long>(taps - 1 + src) * C + c];
      keep[j] = x;
    }
  }
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j)
    if (j < taps - 1) st[static_cast<long>(j) * C + c] = keep[j];
}

// ---------------------------------------------------------------------------------------------------------------------
// state-space scan: block per (entry, head); thread (r, p) owns column p of S [N, P] for rows n = r, r + R, ...
// ---------------------------------------------------------------------------------------------------------------------
__global__ void ssd_scan_kernel(const float* __restrict__ xbc, long sx, int col_b, int col_c, const float* __restrict__ dt_raw, long sd,
                                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                                float* __restrict__ state, float* __restrict__ y, const int* __restrict__ cu,
                                const int* __restrict__ start, const int* __restrict__ state_slot, int heads, int groups, int N, int P,
                                int R) {
  extern __shared__ float sm[];
  float* S = sm;                         // [N][P]
  float* vB = S + static_cast<long>(N) * P;   // [N]
  float* vC = vB + N;                    // [N]
  float* vx = vC + N;                    // [P]
  float* red = vx + P;                   // [R][P]
  const int e = blockIdx.x, h = blockIdx.y, g = h / (heads / groups);
  const int tid = threadIdx.x, r = tid / P, p = tid - r * P;
  const bool live = r < R;
  float* gS = state + (static_cast<long>(state_slot[e]) * heads + h) * N * P;
  const bool carried = start[e] > 0;
  for (int i = tid; i < N * P; i += blockDim.x) S[i] = carried ? gS[i] : 0.f;
  const float negA = -expf(A_log[h]), dskip = Dskip[h], bias = dt_bias[h];
  const int t0 = cu[e], t1 = cu[e + 1];
  for (int t = t0; t < t1; ++t) {
    __syncthreads();                                                     // S loaded / previous token's reads done
    const float* row = xbc + static_cast<long>(t) * sx;
    for (int i = tid; i < N; i += blockDim.x) {
      vB[i] = row[col_b + g * N + i];
      vC[i] = row[col_c + g * N + i];
    }
    for (int i = tid; i < P; i += blockDim.x) vx[i] = row[h * P + i];
    const float dt = softplus(dt_raw[static_cast<long>(t) * sd + h] + bias);
    const float a = expf(negA * dt);
    __syncthreads();
    float acc = 0.f;
    if (live) {
      const float xs = dt * vx[p];
      for (int n = r; n < N; n += R) {
        const float sv = a * S[n * P + p] + vB[n] * xs;
        S[n * P + p] = sv;
        acc += sv * vC[n];
      }
      red[r * P + p] = acc;
    }
    __syncthreads();
    if (tid < P) {
      float tot = 0.f;
      for (int q = 0; q < R; ++q) tot += red[q * P + tid];
      y[static_cast<long>(t) * heads * P + h * P + tid] = tot + dskip * vx[tid];
    }
  }
  __syncthreads();
  for (int i = tid; i < N * P; i += blockDim.x) gS[i] = S[i];
}

// ---------------------------------------------------------------------------------------------------------------------
// gated delta rule
// ---------------------------------------------------------------------------------------------------------------------
// block per token: warps normalise the q / k heads, then all threads form beta and the decays
__global__ void delta_prep_kernel(float* __restrict__ qkv, long sq, int col_k, const float* __restrict__ b_raw, long sb,
                                  const float* __restrict__ a_raw, long sa, const float* __restrict__ dt_bias,
                                  const float* __restrict__ A_log, float* __restrict__ beta, float* __restrict__ decay, int heads,
                                  int kv_heads, int D, int per_channel) {
  const long t = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float qscale = 1.f / sqrtf(static_cast<float>(D));
  for (int hh = w; hh < 2 * kv_heads; hh += nw) {
    const bool is_k = hh >= kv_heads;
    float* v = qkv + t * sq + (is_k ? col_k + (hh - kv_heads) * D : hh * D);
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) ss += v[c] * v[c];
    ss = warp_sum(ss);
    const float r = (is_k ? 1.f : qscale) / sqrtf(ss + 1e-6f);
    for (int c = lane; c < D; c += 32) v[c] *= r;
  }
  for (int hh = threadIdx.x; hh < heads; hh += blockDim.x) beta[t * heads + hh] = 1.f / (1.f + expf(-b_raw[t * sb + hh]));
  const int nd = per_channel ? heads * D : heads;
  for (int i = threadIdx.x; i < nd; i += blockDim.x) {
    const int hh = per_channel ? i / D : i;
    decay[t * nd + i] = expf(-expf(A_log[hh]) * softplus(a_raw[t * sa + i] + dt_bias[i]));
  }
}

// Gated linear attention inputs, block per token: q (columns 0 .. heads*D-1 of qkv, in place) times D^-1/2, and the decay of every
// key channel  decay[t, i] = sigmoid(z)^(1 / tau) = exp(-softplus(-z) / tau)  with z = a_raw[t, i] + a_bias[i].
__global__ void gla_prep_kernel(float* __restrict__ qkv, long sq, const float* __restrict__ a_raw, long sa, const float* __restrict__ a_bias,
                                float inv_tau, float* __restrict__ decay, int n, int D) {
  const long t = blockIdx.x;
  const float qscale = 1.f / sqrtf(static_cast<float>(D));
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    qkv[t * sq + i] *= qscale;
    const float z = a_raw[t * sa + i] + (a_bias != nullptr ? a_bias[i] : 0.f);
    decay[t * n + i] = expf(-softplus(-z) * inv_tau);
  }
}

// block per (entry, head); thread (r, v) owns column v of S [D, Dv] for rows d = r, r + R, ...
// One pass over S forms the decayed state, S^T k and S^T q; the read-out of the written state is o = S^T q + u (k . q).
__global__ void delta_scan_kernel(const float* __restrict__ qkv, long sq, int col_k, int col_v, const float* __restrict__ beta,
                                  const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ o,
                                  const int* __restrict__ cu, const int* __restrict__ start, const int* __restrict__ state_slot,
                                  int heads, int kv_heads, int D, int Dv, int per_channel, int R) {
  extern __shared__ float sm[];
  float* S = sm;                              // [D][Dv]
  float* vq = S + static_cast<long>(D) * Dv;  // [D]
  float* vk = vq + D;                         // [D]
  float* vg = vk + D;                         // [D]
  float* red = vg + D;                        // [2][R][Dv]
  float* kq = red + 2 * R * Dv;               // [1]
  const int e = blockIdx.x, h = blockIdx.y, g = h / (heads / kv_heads);
  const int tid = threadIdx.x, r = tid / Dv, v = tid - r * Dv;
  const bool live = r < R;
  float* gS = state + (static_cast<long>(state_slot[e]) * heads + h) * D * Dv;
  const bool carried = start[e] > 0;
  for (int i = tid; i < D * Dv; i += blockDim.x) S[i] = carried ? gS[i] : 0.f;
  const int t0 = cu[e], t1 = cu[e + 1];
  const int nd = per_channel ? heads * D : heads;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    const float* row = qkv + static_cast<long>(t) * sq;
    for (int i = tid; i < D; i += blockDim.x) {
      vq[i] = row[g * D + i];
      vk[i] = row[col_k + g * D + i];
      vg[i] = per_channel ? decay[static_cast<long>(t) * nd + h * D + i] : decay[static_cast<long>(t) * nd + h];
    }
    __syncthreads();
    if (tid < 32) {
      float d = 0.f;
      for (int i = tid; i < D; i += 32) d += vk[i] * vq[i];
      d = warp_sum(d);
      if (tid == 0) kq[0] = d;
    }
    float pk = 0.f, pq = 0.f;
    if (live) {
      for (int d = r; d < D; d += R) {
        const float sv = vg[d] * S[d * Dv + v];
        S[d * Dv + v] = sv;
        pk += sv * vk[d];
        pq += sv * vq[d];
      }
      red[r * Dv + v] = pk;
      red[(R + r) * Dv + v] = pq;
    }
    __syncthreads();
    if (live) {
      float sk = 0.f, sq_ = 0.f;
      for (int q = 0; q < R; ++q) {
        sk += red[q * Dv + v];
        sq_ += red[(R + q) * Dv + v];
      }
      const float vt = row[col_v + h * Dv + v];
      const float u = beta != nullptr ? beta[static_cast<long>(t) * heads + h] * (vt - sk) : vt;   // no beta: plain accumulation
      if (r == 0) o[static_cast<long>(t) * heads * Dv + h * Dv + v] = sq_ + u * kq[0];
      for (int d = r; d < D; d += R) S[d * Dv + v] += vk[d] * u;
    }
  }
  __syncthreads();
  for (int i = tid; i < D * Dv; i += blockDim.x) gS[i] = S[i];
}


// ---------------------------------------------------------------------------------------------------------------------
// Register-resident scans (the usual sizes): thread (r, c) keeps rows r, r + R, ... of column c of the state in RPT
// registers for the whole entry -- one global read of the state at the start, one write at the end, which is all a decoded
// token needs -- and the next token's inputs are fetched into registers while the current token is computed.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kPre = 4;            // prefetch registers per thread

template <int RPT>
__global__ void __launch_bounds__(RPT >= 64 ? 256 : 512)
ssd_scan_reg_kernel(const float* __restrict__ xbc, long sx, int col_b, int col_c, const float* __restrict__ dt_raw, long sd,
                    const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                    float* __restrict__ state, float* __restrict__ y, const int* __restrict__ cu, const int* __restrict__ start,
                    const int* __restrict__ state_slot, int heads, int groups, int N, int P, int R) {
  extern __shared__ float sm[];
  const int L = 2 * N + P;                       // per token: B | C | x
  float* vec = sm;                               // [2][L]
  float* red = sm + 2 * L;                       // [R][P]
  const int e = blockIdx.x, h = blockIdx.y, g = h / (heads / groups);
  const int tid = threadIdx.x, nth = blockDim.x, r = tid / P, p = tid - r * P;
  const bool live = r < R;
  float* gS = state + (static_cast<long>(state_slot[e]) * heads + h) * N * P;
  const bool carried = start[e] > 0;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int n = r + i * R;
    S[i] = (live && n < N && carried) ? gS[n * P + p] : 0.f;
  }
  const float negA = -expf(A_log[h]), dskip = Dskip[h], bias = dt_bias[h];
  const int t0 = cu[e], t1 = cu[e + 1];
  auto src = [&](int t, int idx) -> const float* {
    const float* row = xbc + static_cast<long>(t) * sx;
    return idx < N ? row + col_b + g * N + idx : idx < 2 * N ? row + col_c + g * N + (idx - N) : row + h * P + (idx - 2 * N);
  };
  float pre[kPre], pre_dt;
#pragma unroll
  for (int i = 0; i < kPre; ++i) {
    const int idx = tid + i * nth;
    pre[i] = idx < L ? *src(t0, idx) : 0.f;
  }
  pre_dt = dt_raw[static_cast<long>(t0) * sd + h];
  for (int t = t0; t < t1; ++t) {
    float* v = vec + ((t - t0) & 1) * L;
#pragma unroll
    for (int i = 0; i < kPre; ++i) {
      const int idx = tid + i * nth;
      if (idx < L) v[idx] = pre[i];
    }
    const float dt = softplus(pre_dt + bias);
    __syncthreads();
    if (t + 1 < t1) {
#pragma unroll
      for (int i = 0; i < kPre; ++i) {
        const int idx = tid + i * nth;
        if (idx < L) pre[i] = *src(t + 1, idx);
      }
      pre_dt = dt_raw[static_cast<long>(t + 1) * sd + h];
    }
    const float a = expf(negA * dt);
    const float* vB = v;
    const float* vC = v + N;
    const float* vx = v + 2 * N;
    if (live) {
      const float xs = dt * vx[p];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int n = r + i * R;
        if (n < N) {
          S[i] = a * S[i] + vB[n] * xs;
          acc += S[i] * vC[n];
        }
      }
      red[r * P + p] = acc;
    }
    __syncthreads();
    if (tid < P) {
      float tot = 0.f;
      for (int q = 0; q < R; ++q) tot += red[q * P + tid];
      y[static_cast<long>(t) * heads * P + h * P + tid] = tot + dskip * vx[tid];
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int n = r + i * R;
      if (n < N) gS[n * P + p] = S[i];
    }
  }
}

template <int RPT>
__global__ void __launch_bounds__(RPT >= 64 ? 256 : 512)
delta_scan_reg_kernel(const float* __restrict__ qkv, long sq, int col_k, int col_v, const float* __restrict__ beta,
                      const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ o, const int* __restrict__ cu,
                      const int* __restrict__ start, const int* __restrict__ state_slot, int heads, int kv_heads, int D, int Dv,
                      int per_channel, int R) {
  extern __shared__ float sm[];
  const int L = 3 * D;                           // per token: q | k | decay per row
  float* vec = sm;                               // [2][L]
  float* red = sm + 2 * L;                       // [2][R][Dv]
  float* rkq = red + 2 * R * Dv;                 // [R]
  const int e = blockIdx.x, h = blockIdx.y, g = h / (heads / kv_heads);
  const int tid = threadIdx.x, nth = blockDim.x, r = tid / Dv, c = tid - r * Dv;
  const bool live = r < R;
  float* gS = state + (static_cast<long>(state_slot[e]) * heads + h) * D * Dv;
  const bool carried = start[e] > 0;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int d = r + i * R;
    S[i] = (live && d < D && carried) ? gS[d * Dv + c] : 0.f;
  }
  const int t0 = cu[e], t1 = cu[e + 1];
  const int nd = per_channel ? heads * D : heads;
  auto src = [&](int t, int idx) -> const float* {
    const float* row = qkv + static_cast<long>(t) * sq;
    return idx < D ? row + g * D + idx
           : idx < 2 * D ? row + col_k + g * D + (idx - D)
                         : decay + static_cast<long>(t) * nd + (per_channel ? h * D + (idx - 2 * D) : h);
  };
  float pre[kPre], pre_v = 0.f, pre_beta;
#pragma unroll
  for (int i = 0; i < kPre; ++i) {
    const int idx = tid + i * nth;
    pre[i] = idx < L ? *src(t0, idx) : 0.f;
  }
  if (live) pre_v = qkv[static_cast<long>(t0) * sq + col_v + h * Dv + c];
  pre_beta = beta != nullptr ? beta[static_cast<long>(t0) * heads + h] : 0.f;
  for (int t = t0; t < t1; ++t) {
    float* v = vec + ((t - t0) & 1) * L;
#pragma unroll
    for (int i = 0; i < kPre; ++i) {
      const int idx = tid + i * nth;
      if (idx < L) v[idx] = pre[i];
    }
    const float v_cur = pre_v, b_cur = pre_beta;
    __syncthreads();
    if (t + 1 < t1) {
#pragma unroll
      for (int i = 0; i < kPre; ++i) {
        const int idx = tid + i * nth;
        if (idx < L) pre[i] = *src(t + 1, idx);
      }
      if (live) pre_v = qkv[static_cast<long>(t + 1) * sq + col_v + h * Dv + c];
      pre_beta = beta != nullptr ? beta[static_cast<long>(t + 1) * heads + h] : 0.f;
    }
    const float* vq = v;
    const float* vk = v + D;
    const float* vg = v + 2 * D;
    if (live) {
      float pk = 0.f, pq = 0.f, pkq = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int d = r + i * R;
        if (d < D) {
          const float sv = vg[d] * S[i];
          S[i] = sv;
          pk += sv * vk[d];
          pq += sv * vq[d];
          if (c == 0) pkq += vk[d] * vq[d];
        }
      }
      red[r * Dv + c] = pk;
      red[(R + r) * Dv + c] = pq;
      if (c == 0) rkq[r] = pkq;
    }
    __syncthreads();
    if (live) {
      float sk = 0.f, sq_ = 0.f, kq = 0.f;
      for (int x = 0; x < R; ++x) {
        sk += red[x * Dv + c];
        sq_ += red[(R + x) * Dv + c];
        kq += rkq[x];
      }
      const float u = beta != nullptr ? b_cur * (v_cur - sk) : v_cur;
      if (r == 0) o[static_cast<long>(t) * heads * Dv + h * Dv + c] = sq_ + u * kq;
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int d = r + i * R;
        if (d < D) S[i] += vk[d] * u;
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int d = r + i * R;
      if (d < D) gS[d * Dv + c] = S[i];
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Column-resident scans (state rows <= 128, the usual sizes): thread c keeps the whole column c of the state in ROWS
// registers, so S^T k, S^T q and S^T C are sums inside one thread -- no reduction across threads -- and a token costs one
// barrier: the vectors all columns share (B and C, or q, k and the row decays) are staged in shared memory, double
// buffered, zero padded to ROWS, and fetched from global memory one token ahead.
// ---------------------------------------------------------------------------------------------------------------------
__host__ __device__ constexpr int col_min_threads(int rows) { return rows > 64 ? 64 : 32; }      // so that a thread stages few values per token

// SPLIT (1 or 2) threads share a column: neighbouring lanes hold the upper and the lower half of its rows and add their
// partial sums with one shuffle (more threads in flight and half the registers for 128-row states).  In shared memory a
// staged vector is SPLIT segments of ROWS / SPLIT + 4 floats, so that the two halves read different banks.
template <int ROWS, int SPLIT>
struct ColStage {
  static constexpr int RH = ROWS / SPLIT;                 // rows per thread
  static constexpr int VL = SPLIT * (RH + 4);             // floats per staged vector
  __host__ __device__ static constexpr int at(int d) { return (d / RH) * (RH + 4) + d % RH; }
};

template <int ROWS, int SPLIT>
__global__ void __launch_bounds__(256)
ssd_scan_col_kernel(const float* __restrict__ xbc, long sx, int col_b, int col_c, const float* __restrict__ dt_raw, long sd,
                    const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                    float* __restrict__ state, float* __restrict__ y, const int* __restrict__ cu, const int* __restrict__ start,
                    const int* __restrict__ state_slot, int heads, int groups, int N, int P) {
  using St = ColStage<ROWS, SPLIT>;
  constexpr int RH = St::RH, VL = St::VL, L = 2 * VL + 4;  // per token: B | C | dt, decay
  constexpr int kStagePre = (2 * ROWS + col_min_threads(ROWS) - 1) / col_min_threads(ROWS);
  __shared__ __align__(16) float stage[2 * L];
  const int e = blockIdx.x, h = blockIdx.y, g = h / (heads / groups);
  const int tid = threadIdx.x, nth = blockDim.x, p = tid / SPLIT, half = tid % SPLIT, r0 = half * RH;
  const bool live = p < P;
  float* gS = state + (static_cast<long>(state_slot[e]) * heads + h) * N * P;
  const bool carried = start[e] > 0;
  float S[RH];
#pragma unroll
  for (int i = 0; i < RH; ++i) S[i] = (live && r0 + i < N && carried) ? gS[static_cast<long>(r0 + i) * P + p] : 0.f;
  const float negA = -expf(A_log[h]), dskip = Dskip[h], bias = dt_bias[h];
  const int t0 = cu[e], t1 = cu[e + 1];
  float pre[kStagePre], pre_x, pre_dt;
  auto fetch = [&](int t) {
    const float* row = xbc + static_cast<long>(t) * sx;
#pragma unroll
    for (int i = 0; i < kStagePre; ++i) {
      const int idx = tid + i * nth;
      if (idx < 2 * ROWS) {
        const int n = idx < ROWS ? idx : idx - ROWS;
        pre[i] = n < N ? row[(idx < ROWS ? col_b : col_c) + g * N + n] : 0.f;
      }
    }
    pre_x = live ? row[h * P + p] : 0.f;
    pre_dt = dt_raw[static_cast<long>(t) * sd + h];
  };
  if (t0 < t1) fetch(t0);
  for (int t = t0; t < t1; ++t) {
    float* v = stage + ((t - t0) & 1) * L;
#pragma unroll
    for (int i = 0; i < kStagePre; ++i) {
      const int idx = tid + i * nth;
      if (idx < 2 * ROWS) v[(idx < ROWS ? 0 : VL) + St::at(idx < ROWS ? idx : idx - ROWS)] = pre[i];
    }
    if (tid == 0) {
      const float dt = softplus(pre_dt + bias);
      v[2 * VL] = dt;
      v[2 * VL + 1] = expf(negA * dt);
    }
    const float x_cur = pre_x;
    __syncthreads();
    if (t + 1 < t1) fetch(t + 1);
    const float dt = v[2 * VL], a = v[2 * VL + 1];
    const float xs = dt * x_cur;
    const float4* vB = reinterpret_cast<const float4*>(v + half * (RH + 4));
    const float4* vC = reinterpret_cast<const float4*>(v + VL + half * (RH + 4));
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < RH / 4; ++i) {
      const float4 b = vB[i], c = vC[i];
      S[4 * i] = a * S[4 * i] + b.x * xs;
      S[4 * i + 1] = a * S[4 * i + 1] + b.y * xs;
      S[4 * i + 2] = a * S[4 * i + 2] + b.z * xs;
      S[4 * i + 3] = a * S[4 * i + 3] + b.w * xs;
      acc[0] += S[4 * i] * c.x;
      acc[1] += S[4 * i + 1] * c.y;
      acc[2] += S[4 * i + 2] * c.z;
      acc[3] += S[4 * i + 3] * c.w;
    }
    float tot = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    if (SPLIT == 2) tot += __shfl_xor_sync(0xffffffffu, tot, 1);
    if (live && half == 0) y[static_cast<long>(t) * heads * P + h * P + p] = tot + dskip * x_cur;
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RH; ++i)
      if (r0 + i < N) gS[static_cast<long>(r0 + i) * P + p] = S[i];
  }
}

template <int ROWS, int SPLIT>
__global__ void __launch_bounds__(256)
delta_scan_col_kernel(const float* __restrict__ qkv, long sq, int col_k, int col_v, const float* __restrict__ beta,
                      const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ o, const int* __restrict__ cu,
                      const int* __restrict__ start, const int* __restrict__ state_slot, int heads, int kv_heads, int D, int Dv,
                      int per_channel) {
  using St = ColStage<ROWS, SPLIT>;
  constexpr int RH = St::RH, VL = St::VL, L = 3 * VL;      // per token: q | k | row decays
  constexpr int kStagePre = (3 * ROWS + col_min_threads(ROWS) - 1) / col_min_threads(ROWS);
  __shared__ __align__(16) float stage[2 * L];
  const int e = blockIdx.x, h = blockIdx.y, g = h / (heads / kv_heads);
  const int tid = threadIdx.x, nth = blockDim.x, c = tid / SPLIT, half = tid % SPLIT, r0 = half * RH;
  const bool live = c < Dv;
  float* gS = state + (static_cast<long>(state_slot[e]) * heads + h) * D * Dv;
  const bool carried = start[e] > 0;
  float S[RH];
#pragma unroll
  for (int i = 0; i < RH; ++i) S[i] = (live && r0 + i < D && carried) ? gS[static_cast<long>(r0 + i) * Dv + c] : 0.f;
  const int t0 = cu[e], t1 = cu[e + 1];
  const int nd = per_channel ? heads * D : heads;
  float pre[kStagePre], pre_v, pre_beta;
  auto fetch = [&](int t) {
    const float* row = qkv + static_cast<long>(t) * sq;
#pragma unroll
    for (int i = 0; i < kStagePre; ++i) {
      const int idx = tid + i * nth;
      if (idx < 3 * ROWS) {
        const int part = idx / ROWS, d = idx - part * ROWS;
        float x = 0.f;
        if (d < D) {
          if (part == 0) x = row[g * D + d];
          else if (part == 1) x = row[col_k + g * D + d];
          else x = decay[static_cast<long>(t) * nd + (per_channel ? h * D + d : h)];
        }
        pre[i] = x;
      }
    }
    pre_v = live ? row[col_v + h * Dv + c] : 0.f;
    pre_beta = beta != nullptr ? beta[static_cast<long>(t) * heads + h] : 0.f;
  };
  if (t0 < t1) fetch(t0);
  for (int t = t0; t < t1; ++t) {
    float* v = stage + ((t - t0) & 1) * L;
#pragma unroll
    for (int i = 0; i < kStagePre; ++i) {
      const int idx = tid + i * nth;
      if (idx < 3 * ROWS) v[(idx / ROWS) * VL + St::at(idx % ROWS)] = pre[i];
    }
    const float v_cur = pre_v, b_cur = pre_beta;
    __syncthreads();
    if (t + 1 < t1) fetch(t + 1);
    const float4* vq = reinterpret_cast<const float4*>(v + half * (RH + 4));
    const float4* vk = reinterpret_cast<const float4*>(v + VL + half * (RH + 4));
    const float4* vg = reinterpret_cast<const float4*>(v + 2 * VL + half * (RH + 4));
    float pk[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < RH / 4; ++i) {                         // S <- g S;  S^T k
      const float4 gg = vg[i], kk = vk[i];
      S[4 * i] *= gg.x;
      S[4 * i + 1] *= gg.y;
      S[4 * i + 2] *= gg.z;
      S[4 * i + 3] *= gg.w;
      pk[0] += S[4 * i] * kk.x;
      pk[1] += S[4 * i + 1] * kk.y;
      pk[2] += S[4 * i + 2] * kk.z;
      pk[3] += S[4 * i + 3] * kk.w;
    }
    float sk = (pk[0] + pk[1]) + (pk[2] + pk[3]);
    if (SPLIT == 2) sk += __shfl_xor_sync(0xffffffffu, sk, 1);
    const float u = beta != nullptr ? b_cur * (v_cur - sk) : v_cur;
    float po[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < RH / 4; ++i) {                         // S <- S + k u^T;  o = S^T q sees this token's write
      const float4 kk = vk[i], qq = vq[i];
      S[4 * i] += kk.x * u;
      S[4 * i + 1] += kk.y * u;
      S[4 * i + 2] += kk.z * u;
      S[4 * i + 3] += kk.w * u;
      po[0] += S[4 * i] * qq.x;
      po[1] += S[4 * i + 1] * qq.y;
      po[2] += S[4 * i + 2] * qq.z;
      po[3] += S[4 * i + 3] * qq.w;
    }
    float so_ = (po[0] + po[1]) + (po[2] + po[3]);
    if (SPLIT == 2) so_ += __shfl_xor_sync(0xffffffffu, so_, 1);
    if (live && half == 0) o[static_cast<long>(t) * heads * Dv + h * Dv + c] = so_;
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RH; ++i)
      if (r0 + i < D) gS[static_cast<long>(r0 + i) * Dv + c] = S[i];
  }
}

// template sizes and block size of the column-resident kernels for a state of `rows` x `cols`; false when they do not fit
bool pick_col_layout(int cols, int rows, int* rows_t, int* split_out, int* threads_out) {
  if (rows > 128 || cols < 1 || cols > 256) return false;
  const int rt = rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128;
  const int split = rt == 128 && cols <= 128 ? 2 : 1;      // 128 rows: two threads per column when the block allows
  int threads = ((cols * split + 31) / 32) * 32;
  if (threads < col_min_threads(rt)) threads = col_min_threads(rt);
  *rows_t = rt;
  *split_out = split;
  *threads_out = threads;
  return true;
}

// rows per thread / row groups for a state of `rows` x `cols`: as many row groups as 512 threads allow (256 when a thread
// holds 64 rows), at most 64 rows per thread, and enough threads to fetch a token's inputs with kPre loads each
bool pick_reg_layout(int cols, int rows, int per_token, int* R_out, int* rpt_out, int* threads_out) {
  if (cols > 512) return false;
  int R = 512 / cols;
  if (R > rows) R = rows;
  if (R < 1) return false;
  int need = (rows + R - 1) / R;
  if (need > 32) {
    R = 256 / cols;
    if (R > rows) R = rows;
    if (R < 1) return false;
    need = (rows + R - 1) / R;
    if (need > 64) return false;
    if (need <= 32) need = 33;                      // stays in the 64-row variant, whose blocks have 256 threads
  }
  const int rpt = need <= 4 ? 4 : need <= 8 ? 8 : need <= 16 ? 16 : need <= 32 ? 32 : 64;
  int threads = ((cols * R + 31) / 32) * 32;
  const int for_loads = (((per_token + kPre - 1) / kPre + 31) / 32) * 32;
  if (threads < for_loads) threads = for_loads;
  if (threads > (rpt == 64 ? 256 : 512)) return false;
  *R_out = R; *rpt_out = rpt; *threads_out = threads;
  return true;
}

int pick_rows(int cols, int rows) {
  // threads = cols * R <= 512, R <= rows
  int R = 512 / cols;
  if (R < 1) R = 1;
  if (R > rows) R = rows;
  if (R > 16) R = 16;
  return R;
}

// ---------------------------------------------------------------------------------------------------------------------
// Matrix memory with exponential gates and a running maximum (mLSTM).  Per head, with log gates i and f of the token and the
// carried maximum m (0 for a new sequence):  m' = max(f + m, i);  S = exp(f + m - m') S + exp(i - m') k v^T  and the
// normaliser n likewise with k alone.  n is kept as one more column of the state (a value that is always 1), so the state
// of a head is [D, Dv + 1] and its read-out S^T q gives the numerator in columns 0 .. Dv-1 and n . q in column Dv; the division
// is left to nrl_mlstm_out.  The raw gates are capped (cap * tanh(z / cap), cap > 0) and the forget gate goes through
// log-sigmoid.  Block per (entry, head): thread c keeps column c of the state in ROWS registers; one more warp forms the
// gates of the next token while the columns work on the current one (the recurrence of m is one dependent chain per head).
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float logsigmoid_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

struct MlstmGate {
  float a, b, m;
};
__device__ __forceinline__ MlstmGate mlstm_gate(float i_raw, float f_raw, float cap, float m_prev) {
  const float ig = cap > 0.f ? cap * tanhf(i_raw / cap) : i_raw;
  const float fg = logsigmoid_(cap > 0.f ? cap * tanhf(f_raw / cap) : f_raw);
  MlstmGate g;
  g.m = fmaxf(fg + m_prev, ig);
  g.a = expf(fg + m_prev - g.m);
  g.b = expf(ig - g.m);
  return g;
}

// SPLIT (1 or 2) threads share a column as in the other column-resident scans (ColStage): neighbouring lanes hold the upper and
// the lower half of its rows and add their partial sums with one shuffle.
template <int ROWS, int SPLIT>
__global__ void __launch_bounds__(ROWS >= 128 ? 320 : ROWS >= 64 ? 256 : 544)      // 128 rows: 168 registers, two blocks of 192 threads per SM
mlstm_scan_col_kernel(const float* __restrict__ qkv, long sq, int col_q, int col_k, int col_v, int col_i, int col_f,
                      const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                      float* __restrict__ state, float* __restrict__ mstate, float* __restrict__ o, float* __restrict__ m_out,
                      const int* __restrict__ cu, const int* __restrict__ start, const int* __restrict__ state_slot, int heads, int D,
                      int Dv, int Cs) {
  using St = ColStage<ROWS, SPLIT>;
  constexpr int RH = St::RH, VL = St::VL, L = 2 * VL + 4;  // per token: q | k | a, b
  constexpr int kStagePre = (2 * ROWS + 63) / 64;          // a block has at least 64 threads
  __shared__ __align__(16) float stage[2 * L];
  const int e = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, nth = blockDim.x, ncol = nth - 32, C = Dv + 1;        // ncol threads own columns, the last warp the gates
  const int c = tid / SPLIT, half = tid % SPLIT, r0 = half * RH;
  const bool gate_lane = tid == ncol, col_thread = tid < ncol, live = col_thread && c < C;
  const long slot = state_slot[e];
  float* gS = state + (slot * heads + h) * D * Cs;       // rows of Cs >= Dv + 1 floats
  const bool carried = start[e] > 0;
  float S[RH];
#pragma unroll
  for (int i = 0; i < RH; ++i) S[i] = (live && r0 + i < D && carried) ? gS[static_cast<long>(r0 + i) * Cs + c] : 0.f;
  const int t0 = cu[e], t1 = cu[e + 1];
  const float ib = i_bias != nullptr ? i_bias[h] : 0.f, fb = f_bias != nullptr ? f_bias[h] : 0.f;
  float m_run = carried ? mstate[slot * heads + h] : 0.f;
  MlstmGate gt = {0.f, 0.f, 0.f};
  float pre[kStagePre], pre_v = 0.f;
  auto fetch = [&](int t) {
    const float* row = qkv + static_cast<long>(t) * sq;
#pragma unroll
    for (int i = 0; i < kStagePre; ++i) {
      const int idx = tid + i * nth;
      if (idx < 2 * ROWS) {
        const int d = idx < ROWS ? idx : idx - ROWS;
        pre[i] = d < D ? (idx < ROWS ? row[col_q + h * D + d] * q_scale : row[col_k + h * D + d]) : 0.f;
      }
    }
    if (col_thread) pre_v = c < Dv ? row[col_v + h * Dv + c] : 1.f;
    if (gate_lane) {
      gt = mlstm_gate(row[col_i + h] + ib, row[col_f + h] + fb, cap, m_run);
      m_run = gt.m;
    }
  };
  if (t0 < t1) fetch(t0);
  for (int t = t0; t < t1; ++t) {
    float* v = stage + ((t - t0) & 1) * L;
#pragma unroll
    for (int i = 0; i < kStagePre; ++i) {
      const int idx = tid + i * nth;
      if (idx < 2 * ROWS) v[(idx < ROWS ? 0 : VL) + St::at(idx < ROWS ? idx : idx - ROWS)] = pre[i];
    }
    if (gate_lane) {
      v[2 * VL] = gt.a;
      v[2 * VL + 1] = gt.b;
      m_out[static_cast<long>(t) * heads + h] = gt.m;
    }
    const float v_cur = pre_v;
    __syncthreads();
    if (t + 1 < t1) fetch(t + 1);
    if (col_thread) {
      const float a = v[2 * VL], bv = v[2 * VL + 1] * v_cur;
      const float4* vq = reinterpret_cast<const float4*>(v + half * (RH + 4));
      const float4* vk = reinterpret_cast<const float4*>(v + VL + half * (RH + 4));
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < RH / 4; ++i) {
        const float4 kk = vk[i], qq = vq[i];
        S[4 * i] = a * S[4 * i] + kk.x * bv;
        S[4 * i + 1] = a * S[4 * i + 1] + kk.y * bv;
        S[4 * i + 2] = a * S[4 * i + 2] + kk.z * bv;
        S[4 * i + 3] = a * S[4 * i + 3] + kk.w * bv;
        acc[0] += S[4 * i] * qq.x;
        acc[1] += S[4 * i + 1] * qq.y;
        acc[2] += S[4 * i + 2] * qq.z;
        acc[3] += S[4 * i + 3] * qq.w;
      }
      float tot = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      if (SPLIT == 2) tot += __shfl_xor_sync(0xffffffffu, tot, 1);
      if (live && half == 0) o[(static_cast<long>(t) * heads + h) * C + c] = tot;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RH; ++i)
      if (r0 + i < D) gS[static_cast<long>(r0 + i) * Cs + c] = S[i];
  }
  if (gate_lane && t0 < t1) mstate[slot * heads + h] = m_run;
}

// Any size: the state stays in global memory, thread per column, every thread forms the gates itself.
__global__ void mlstm_scan_kernel(const float* __restrict__ qkv, long sq, int col_q, int col_k, int col_v, int col_i, int col_f,
                                  const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                                  float* __restrict__ state, float* __restrict__ mstate, float* __restrict__ o, float* __restrict__ m_out,
                                  const int* __restrict__ cu, const int* __restrict__ start, const int* __restrict__ state_slot, int heads,
                                  int D, int Dv, int Cs) {
  const int e = blockIdx.x, h = blockIdx.y, C = Dv + 1;
  const long slot = state_slot[e];
  float* gS = state + (slot * heads + h) * D * Cs;
  const bool carried = start[e] > 0;
  const float ib = i_bias != nullptr ? i_bias[h] : 0.f, fb = f_bias != nullptr ? f_bias[h] : 0.f;
  const float m0 = carried ? mstate[slot * heads + h] : 0.f;
  __syncthreads();                                         // every thread has read the carried maximum before thread 0 replaces it
  const int t0 = cu[e], t1 = cu[e + 1];
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float m_run = m0;
    for (int t = t0; t < t1; ++t) {
      const float* row = qkv + static_cast<long>(t) * sq;
      const MlstmGate gt = mlstm_gate(row[col_i + h] + ib, row[col_f + h] + fb, cap, m_run);
      m_run = gt.m;
      const float bv = gt.b * (c < Dv ? row[col_v + h * Dv + c] : 1.f);
      float acc = 0.f;
      for (int d = 0; d < D; ++d) {
        const float old = (carried || t > t0) ? gS[static_cast<long>(d) * Cs + c] : 0.f;
        const float sv = gt.a * old + row[col_k + h * D + d] * bv;
        gS[static_cast<long>(d) * Cs + c] = sv;
        acc += sv * (row[col_q + h * D + d] * q_scale);
      }
      o[(static_cast<long>(t) * heads + h) * C + c] = acc;
      if (c == 0) m_out[static_cast<long>(t) * heads + h] = gt.m;
    }
    if (c == 0 && t0 < t1) mstate[slot * heads + h] = m_run;
  }
}

// warp per (token, head): y = o[:Dv] / (max(|o[Dv]|, exp(-m)) + 1e-6); out = scale * y / rms(y) * w * sigmoid(gate)
template <typename OT>
__global__ void mlstm_out_kernel(const float* __restrict__ o, const float* __restrict__ m, const float* __restrict__ gate, long sg,
                                 const float* __restrict__ w, float eps, float scale, OT* __restrict__ out, long so, long T, int heads,
                                 int Dv) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * heads) return;
  const long t = wid / heads;
  const int h = static_cast<int>(wid - t * heads);
  const float* row = o + wid * (Dv + 1);
  const float inv = 1.f / (fmaxf(fabsf(row[Dv]), expf(-m[wid])) + 1e-6f);
  float ss = 0.f;
  for (int c = lane; c < Dv; c += 32) {
    const float y = row[c] * inv;
    ss += y * y;
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / static_cast<float>(Dv) + eps);
  for (int c = lane; c < Dv; c += 32) {
    const long col = static_cast<long>(h) * Dv + c;
    const float g = gate[t * sg + col];
    const float val = scale * (row[c] * inv * r * w[col] * (1.f / (1.f + expf(-g))));
    if constexpr (sizeof(OT) == 4) out[t * so + col] = val;
    else out[t * so + col] = __float2bfloat16_rn(val);
  }
}

}  // namespace

extern "C" {

cudaError_t nrl_causal_conv(const float* in, long si, const float* in_bias, int act, const float* w, const float* bias,
                            const float* state, float* out, long so, const int* cu, const int* tok_entry, const int* start,
                            const int* state_slot, int T, int E, int C, int taps, cudaStream_t s) {
  if (T <= 0 || C <= 0) return cudaSuccess;
  if (taps < 1 || taps > kMaxTaps) return cudaErrorInvalidValue;
  if (T >= 2 * kConvTok && T >= 2 * E && (T + kConvTok - 1) / kConvTok <= 65535) {     // prompt portions: runs of tokens per thread
    const dim3 grid((C + 127) / 128, (T + kConvTok - 1) / kConvTok);
    if (taps <= 4)
      causal_conv_run_kernel<4><<<grid, 128, 0, s>>>(in, si, in_bias, act, w, bias, state, out, so, cu, tok_entry, start, state_slot, T, C, taps);
    else
      causal_conv_run_kernel<kMaxTaps><<<grid, 128, 0, s>>>(in, si, in_bias, act, w, bias, state, out, so, cu, tok_entry, start, state_slot, T, C, taps);
    return cudaGetLastError();
  }
  const long n = static_cast<long>(T) * C;
  causal_conv_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(in, si, in_bias, act, w, bias, state, out, so, cu,
                                                                           tok_entry, start, state_slot, T, C, taps);
  return cudaGetLastError();
}

cudaError_t nrl_causal_conv_carry(const float* in, long si, const float* in_bias, float* state, const int* cu, const int* start,
                                  const int* state_slot, int E, int C, int taps, cudaStream_t s) {
  if (E <= 0 || C <= 0 || taps <= 1) return cudaSuccess;
  if (taps > kMaxTaps) return cudaErrorInvalidValue;
  const long n = static_cast<long>(E) * C;
  causal_conv_carry_kernel<<<static_cast<unsigned>((n + 127) / 128), 128, 0, s>>>(in, si, in_bias, state, cu, start, state_slot, E, C, taps);
  return cudaGetLastError();
}

cudaError_t nrl_ssd_scan(const float* xbc, long sx, int col_b, int col_c, const float* dt_raw, long sd, const float* dt_bias,
                         const float* A_log, const float* Dskip, float* state, float* y, const int* cu, const int* start,
                         const int* state_slot, int E, int heads, int groups, int N, int P, int impl, cudaStream_t s) {
  if (E <= 0) return cudaSuccess;
  if (P > 512 || heads % groups != 0 || impl < 0 || impl > 3) return cudaErrorInvalidValue;
  if (impl == 0 || impl == 1) {
    int rt, split, threads;
    if (pick_col_layout(P, N, &rt, &split, &threads)) {
#define NRL_SSDC(R_, S_)                                                                                                           \
  if (rt == R_ && split == S_) {                                                                                                   \
    ssd_scan_col_kernel<R_, S_><<<dim3(E, heads), threads, 0, s>>>(xbc, sx, col_b, col_c, dt_raw, sd, dt_bias, A_log, Dskip, state, y, \
                                                                   cu, start, state_slot, heads, groups, N, P);                    \
    return cudaGetLastError();                                                                                                     \
  }
      NRL_SSDC(16, 1) NRL_SSDC(32, 1) NRL_SSDC(64, 1) NRL_SSDC(128, 1) NRL_SSDC(128, 2)
#undef NRL_SSDC
    }
    if (impl == 1) return cudaErrorInvalidValue;
  }
  if (impl != 3) {
    int R, rpt, threads;
    const size_t smem_reg = sizeof(float) * (2 * (2 * static_cast<size_t>(N) + P) + 512);
    if (pick_reg_layout(P, N, 2 * N + P, &R, &rpt, &threads) && smem_reg <= 48 * 1024) {
      const size_t smem = sizeof(float) * (2 * (2 * static_cast<size_t>(N) + P) + static_cast<size_t>(R) * P);
#define NRL_SSD(RPT_)                                                                                                              \
  if (rpt == RPT_) {                                                                                                               \
    ssd_scan_reg_kernel<RPT_><<<dim3(E, heads), threads, smem, s>>>(xbc, sx, col_b, col_c, dt_raw, sd, dt_bias, A_log, Dskip, state, y, \
                                                                    cu, start, state_slot, heads, groups, N, P, R);                \
    return cudaGetLastError();                                                                                                     \
  }
      NRL_SSD(4) NRL_SSD(8) NRL_SSD(16) NRL_SSD(32) NRL_SSD(64)
#undef NRL_SSD
    }
    if (impl == 2) return cudaErrorInvalidValue;
  }
  const int R = pick_rows(P, N);
  const int threads = ((P * R + 31) / 32) * 32;
  const size_t smem = sizeof(float) * (static_cast<size_t>(N) * P + 2 * N + P + static_cast<size_t>(R) * P);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(ssd_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    configured = 200 * 1024;
  }
  ssd_scan_kernel<<<dim3(E, heads), threads, smem, s>>>(xbc, sx, col_b, col_c, dt_raw, sd, dt_bias, A_log, Dskip, state, y, cu, start,
                                                        state_slot, heads, groups, N, P, R);
  return cudaGetLastError();
}

cudaError_t nrl_delta_prep(float* qkv, long sq, int col_k, const float* b_raw, long sb, const float* a_raw, long sa,
                           const float* dt_bias, const float* A_log, float* beta, float* decay, int T, int heads, int kv_heads, int D,
                           int per_channel, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  delta_prep_kernel<<<T, 128, 0, s>>>(qkv, sq, col_k, b_raw, sb, a_raw, sa, dt_bias, A_log, beta, decay, heads, kv_heads, D,
                                      per_channel);
  return cudaGetLastError();
}

cudaError_t nrl_gla_prep(float* qkv, long sq, const float* a_raw, long sa, const float* a_bias, float tau, float* decay, int T,
                         int heads, int D, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (!(tau > 0.f)) return cudaErrorInvalidValue;
  gla_prep_kernel<<<T, 128, 0, s>>>(qkv, sq, a_raw, sa, a_bias, 1.f / tau, decay, heads * D, D);
  return cudaGetLastError();
}

cudaError_t nrl_delta_scan(const float* qkv, long sq, int col_k, int col_v, const float* beta, const float* decay, float* state,
                           float* o, const int* cu, const int* start, const int* state_slot, int E, int heads, int kv_heads, int D,
                           int Dv, int per_channel, int impl, cudaStream_t s) {
  if (E <= 0) return cudaSuccess;
  if (Dv > 512 || heads % kv_heads != 0 || impl < 0 || impl > 3) return cudaErrorInvalidValue;
  if (impl == 0 || impl == 1) {
    int rt, split, threads;
    if (pick_col_layout(Dv, D, &rt, &split, &threads)) {
#define NRL_DELTAC(R_, S_)                                                                                                         \
  if (rt == R_ && split == S_) {                                                                                                   \
    delta_scan_col_kernel<R_, S_><<<dim3(E, heads), threads, 0, s>>>(qkv, sq, col_k, col_v, beta, decay, state, o, cu, start,        \
                                                                     state_slot, heads, kv_heads, D, Dv, per_channel);             \
    return cudaGetLastError();                                                                                                     \
  }
      NRL_DELTAC(16, 1) NRL_DELTAC(32, 1) NRL_DELTAC(64, 1) NRL_DELTAC(128, 1) NRL_DELTAC(128, 2)
#undef NRL_DELTAC
    }
    if (impl == 1) return cudaErrorInvalidValue;
  }
  if (impl != 3) {
    int R, rpt, threads;
    const size_t smem_reg = sizeof(float) * (6 * static_cast<size_t>(D) + 2 * 512 + 64);
    if (pick_reg_layout(Dv, D, 3 * D, &R, &rpt, &threads) && smem_reg <= 48 * 1024) {
      const size_t smem = sizeof(float) * (6 * static_cast<size_t>(D) + 2 * static_cast<size_t>(R) * Dv + R);
#define NRL_DELTA(RPT_)                                                                                                            \
  if (rpt == RPT_) {                                                                                                               \
    delta_scan_reg_kernel<RPT_><<<dim3(E, heads), threads, smem, s>>>(qkv, sq, col_k, col_v, beta, decay, state, o, cu, start,       \
                                                                      state_slot, heads, kv_heads, D, Dv, per_channel, R);         \
    return cudaGetLastError();                                                                                                     \
  }
      NRL_DELTA(4) NRL_DELTA(8) NRL_DELTA(16) NRL_DELTA(32) NRL_DELTA(64)
#undef NRL_DELTA
    }
    if (impl == 2) return cudaErrorInvalidValue;
  }
  const int R = pick_rows(Dv, D);
  const int threads = ((Dv * R + 31) / 32) * 32;
  const size_t smem = sizeof(float) * (static_cast<size_t>(D) * Dv + 3 * D + 2 * static_cast<size_t>(R) * Dv + 1);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    configured = 200 * 1024;
  }
  delta_scan_kernel<<<dim3(E, heads), threads, smem, s>>>(qkv, sq, col_k, col_v, beta, decay, state, o, cu, start, state_slot, heads,
                                                          kv_heads, D, Dv, per_channel, R);
  return cudaGetLastError();
}

cudaError_t nrl_mlstm_scan(const float* qkv, long sq, int col_q, int col_k, int col_v, int col_i, int col_f, const float* i_bias,
                           const float* f_bias, float cap, float q_scale, float* state, float* mstate, float* o, float* m_out,
                           const int* cu, const int* start, const int* state_slot, int E, int heads, int D, int Dv, int Cs,
                           int single_token, int impl, cudaStream_t s) {
  if (E <= 0) return cudaSuccess;
  if (D < 1 || Dv < 1 || Cs < Dv + 1 || impl < 0 || impl > 2) return cudaErrorInvalidValue;
  // Steps of single tokens only move the state: two threads per column of a 128-row state put more loads in flight.  Entries
  // that hold runs of tokens are bound by the token loop, where one thread per column keeps its rows in registers without spills.
  const int rt = D <= 16 ? 16 : D <= 32 ? 32 : D <= 64 ? 64 : 128;
  const int split = single_token && rt == 128 && (((Dv + 1) * 2 + 31) / 32) * 32 + 32 <= 320 ? 2 : 1;
  const int ncol = (((Dv + 1) * split + 31) / 32) * 32;
  if (impl != 2 && D <= 128 && ncol + 32 <= (rt >= 128 ? 320 : rt >= 64 ? 256 : 544)) {
#define NRL_ML(R_, S_)                                                                                                             \
  mlstm_scan_col_kernel<R_, S_><<<dim3(E, heads), ncol + 32, 0, s>>>(qkv, sq, col_q, col_k, col_v, col_i, col_f, i_bias, f_bias, cap,  \
                                                                     q_scale, state, mstate, o, m_out, cu, start, state_slot, heads, D, Dv, Cs)
    if (rt == 16) NRL_ML(16, 1);
    else if (rt == 32) NRL_ML(32, 1);
    else if (rt == 64) NRL_ML(64, 1);
    else if (split == 2) NRL_ML(128, 2);
    else NRL_ML(128, 1);
#undef NRL_ML
    return cudaGetLastError();
  }
  if (impl == 1) return cudaErrorInvalidValue;
  const int th = Dv + 1 >= 256 ? 256 : ((Dv + 1 + 31) / 32) * 32;
  mlstm_scan_kernel<<<dim3(E, heads), th, 0, s>>>(qkv, sq, col_q, col_k, col_v, col_i, col_f, i_bias, f_bias, cap, q_scale, state, mstate,
                                                  o, m_out, cu, start, state_slot, heads, D, Dv, Cs);
  return cudaGetLastError();
}

cudaError_t nrl_mlstm_out(const float* o, const float* m, const float* gate, long sg, const float* w, float eps, float scale, void* out,
                          long so, int out_f32, int T, int heads, int Dv, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const long warps = static_cast<long>(T) * heads;
  const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
  if (out_f32) mlstm_out_kernel<float><<<blocks, 128, 0, s>>>(o, m, gate, sg, w, eps, scale, static_cast<float*>(out), so, T, heads, Dv);
  else mlstm_out_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(o, m, gate, sg, w, eps, scale, static_cast<__nv_bfloat16*>(out), so, T, heads, Dv);
  return cudaGetLastError();
}

}  // extern "C"
