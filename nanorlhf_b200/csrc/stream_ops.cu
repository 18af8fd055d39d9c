// Residual-stream and normalisation kernels of hybrid decoders (float stream, typed GEMM operands):
// learned-position and hashed-pair embeddings, depth-weighted stream + single-gain RMS norm, sandwich (pre + post) group norms
// with a gated residual, part-wise gated RMS norm, column activations, mixture-of-experts routing.
// Compiled WITHOUT fast-math: the float32 serving mode must stay within float rounding of a plain evaluation.
#include <cuda_bf16.h>

#include <cstdint>

#include "hybrid_kernels.h"

namespace {

__device__ __forceinline__ float ld(const float* p, long i) { return p[i]; }
__device__ __forceinline__ float ld(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st(float* p, long i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__nv_bfloat16* p, long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void st4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 u;
  u.x = *reinterpret_cast<const unsigned*>(&a);
  u.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}
// V consecutive floats (V = 1 or 4; 4 needs 16-byte alignment)
template <int V>
__device__ __forceinline__ void ldv(const float* p, float (&v)[V]) {
  if constexpr (V == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  } else {
    v[0] = p[0];
  }
}
template <int V, typename OT>
__device__ __forceinline__ void stv(OT* p, const float (&v)[V]) {
  if constexpr (V == 4) st4(p, v);
  else st(p, 0, v[0]);
}

// sum over the block; every thread gets the result.  red: >= 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}

template <typename WT>
__global__ void embed_pos_kernel(const WT* __restrict__ embed, const WT* __restrict__ ptab, const int* __restrict__ tok,
                                 const int* __restrict__ pos, float* __restrict__ out, int W) {
  const long t = blockIdx.x;
  const long a = static_cast<long>(tok[t]) * W, b = static_cast<long>(pos[t]) * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) out[t * W + c] = ld(embed, a + c) + ld(ptab, b + c);
}

template <typename HT, int V>        // V columns per thread and pass (4: 128-bit accesses, needs W % 4 == 0)
__global__ void stream_norm_kernel(float* __restrict__ results, long stride_r, int i, const float* __restrict__ o,
                                   const float* __restrict__ xprev, const float* __restrict__ dw, const float* __restrict__ g,
                                   float eps, float* __restrict__ xcur, HT* __restrict__ h, int W) {
  __shared__ float red[32];
  const long row = static_cast<long>(blockIdx.x) * W;
  float ss = 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float last[V], x[V];
    if (o != nullptr) {
      float a[V], b[V];
      ldv<V>(xprev + row + c, a);
      ldv<V>(o + row + c, b);
#pragma unroll
      for (int k = 0; k < V; ++k) last[k] = a[k] + b[k];
      stv<V>(results + i * stride_r + row + c, last);
    } else {
      ldv<V>(results + i * stride_r + row + c, last);
    }
    if (dw != nullptr) {
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] = 0.f;
      for (int j = 0; j < i; ++j) {
        float r[V];
        ldv<V>(results + j * stride_r + row + c, r);
        const float wj = dw[j];
#pragma unroll
        for (int k = 0; k < V; ++k) x[k] += wj * r[k];
      }
      const float wi = dw[i];
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] += wi * last[k];
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) x[k] = last[k];
    }
    stv<V>(xcur + row + c, x);
#pragma unroll
    for (int k = 0; k < V; ++k) ss += x[k] * x[k];
  }
  ss = block_sum(ss, red);
  const float r = g[0] / sqrtf(ss / static_cast<float>(W) + eps);
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float x[V];
    ldv<V>(xcur + row + c, x);
#pragma unroll
    for (int k = 0; k < V; ++k) x[k] *= r;
    stv<V>(h + row + c, x);
  }
}

// x[t] = embed[tok[t]] * scale + pair[row], row = (prev * mul_prev + tok * mul_cur) mod buckets, or row `buckets` for the first
// token of a sequence.  prev comes from the step's own tokens or, for the first token of an entry, from the sequence's slot.
template <typename WT>
__global__ void embed_hashed_kernel(const WT* __restrict__ embed, const WT* __restrict__ pair, const int* __restrict__ tok,
                                    const int* __restrict__ cu, const int* __restrict__ tok_entry, const int* __restrict__ start,
                                    const int* __restrict__ state_slot, const int* __restrict__ prev_state, float scale,
                                    long mul_prev, long mul_cur, long buckets, float* __restrict__ out, int W) {
  const long t = blockIdx.x;
  const int cur = tok[t];
  const long a = static_cast<long>(cur) * W;
  long b = -1;
  if (pair != nullptr) {
    const int e = tok_entry[t];
    long row = buckets;
    if (t > cu[e]) row = (static_cast<long>(tok[t - 1]) * mul_prev + static_cast<long>(cur) * mul_cur) % buckets;
    else if (start[e] > 0) row = (static_cast<long>(prev_state[state_slot[e]]) * mul_prev + static_cast<long>(cur) * mul_cur) % buckets;
    b = row * W;
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = ld(embed, a + c) * scale;
    if (b >= 0) v += ld(pair, b + c);
    out[t * W + c] = v;
  }
}

__global__ void token_carry_kernel(const int* __restrict__ tok, const int* __restrict__ cu, const int* __restrict__ state_slot,
                                   int* __restrict__ prev_state, int E) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < E) prev_state[state_slot[e]] = tok[cu[e + 1] - 1];
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }

// Sublayer boundary of a sandwich-normed stream, one block per token; the vector is cut into `groups` equal parts and each
// part has its own root mean square:
//   if (o)  y = o * sigmoid(gate + gate_bias)  (gate == nullptr: y = o);  x += y / rms_part(y) * w_post
//   if (h)  h = x / rms_part(x) * w_pre
template <typename HT>
__global__ void group_norm_residual_kernel(float* __restrict__ x, const float* __restrict__ o, const float* __restrict__ gate, long sg,
                                           const float* __restrict__ gate_bias, const float* __restrict__ w_post,
                                           const float* __restrict__ w_pre, int groups, float eps, HT* __restrict__ h, int W) {
  __shared__ float red[32];
  const long row = static_cast<long>(blockIdx.x) * W;
  const int part = W / groups;
  const float inv = 1.f / static_cast<float>(part);
  for (int g = 0; g < groups; ++g) {
    const int c0 = g * part, c1 = c0 + part;
    if (o != nullptr) {
      float ss = 0.f;
      for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float y = o[row + c];
        if (gate != nullptr) y *= sigmoidf_(gate[blockIdx.x * sg + c] + (gate_bias != nullptr ? gate_bias[c] : 0.f));
        ss += y * y;
      }
      ss = block_sum(ss, red);
      const float r = 1.f / sqrtf(ss * inv + eps);
      for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        float y = o[row + c];
        if (gate != nullptr) y *= sigmoidf_(gate[blockIdx.x * sg + c] + (gate_bias != nullptr ? gate_bias[c] : 0.f));
        x[row + c] += y * r * w_post[c];
      }
    }
    if (h != nullptr) {
      float ss = 0.f;
      for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {       // a thread re-reads the columns it wrote itself
        const float v = x[row + c];
        ss += v * v;
      }
      ss = block_sum(ss, red);
      const float r = 1.f / sqrtf(ss * inv + eps);
      for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) st(h, row + c, x[row + c] * r * w_pre[c]);
    }
  }
}

// The same boundary with 128-bit accesses and the group's values held in registers between the passes (NV float4 per thread):
// o, the gate and x are read once, x and h written once.  Needs W / groups % 4 == 0 and 16-byte aligned rows.
template <typename HT, int NV>
__global__ void group_norm_residual_vec_kernel(float* __restrict__ x, const float* __restrict__ o, const float* __restrict__ gate,
                                               long sg, const float* __restrict__ gate_bias, const float* __restrict__ w_post,
                                               const float* __restrict__ w_pre, int groups, float eps, HT* __restrict__ h, int W) {
  __shared__ float red[32];
  const long row = static_cast<long>(blockIdx.x) * W;
  const int part = W / groups, part4 = part >> 2;
  const float inv = 1.f / static_cast<float>(part);
  for (int g = 0; g < groups; ++g) {
    const int c0 = g * part;
    float v[NV][4];
    if (o != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i4 = threadIdx.x + k * blockDim.x;
        v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.f;
        if (i4 < part4) {
          const int c = c0 + i4 * 4;
          ldv<4>(o + row + c, v[k]);
          if (gate != nullptr) {
            float gv[4], gb[4] = {0.f, 0.f, 0.f, 0.f};
            ldv<4>(gate + blockIdx.x * sg + c, gv);
            if (gate_bias != nullptr) ldv<4>(gate_bias + c, gb);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[k][e] *= sigmoidf_(gv[e] + gb[e]);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) ss += v[k][e] * v[k][e];
        }
      }
      ss = block_sum(ss, red);
      const float r = 1.f / sqrtf(ss * inv + eps);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i4 = threadIdx.x + k * blockDim.x;
        if (i4 < part4) {
          const int c = c0 + i4 * 4;
          float xv[4], wv[4];
          ldv<4>(x + row + c, xv);
          ldv<4>(w_post + c, wv);
#pragma unroll
          for (int e = 0; e < 4; ++e) v[k][e] = xv[e] + v[k][e] * r * wv[e];
          st4(x + row + c, v[k]);
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i4 = threadIdx.x + k * blockDim.x;
        v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.f;
        if (i4 < part4) ldv<4>(x + row + c0 + i4 * 4, v[k]);
      }
    }
    if (h != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k)
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += v[k][e] * v[k][e];
      ss = block_sum(ss, red);
      const float r = 1.f / sqrtf(ss * inv + eps);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int i4 = threadIdx.x + k * blockDim.x;
        if (i4 < part4) {
          const int c = c0 + i4 * 4;
          float wv[4], hv[4];
          ldv<4>(w_pre + c, wv);
#pragma unroll
          for (int e = 0; e < 4; ++e) hv[e] = v[k][e] * r * wv[e];
          st4(h + row + c, hv);
        }
      }
    }
  }
}

// Mixture-of-experts routing and (dense form) expert activations, one block per token.
//   z = router[t, :E] + router_bias;  the `top` largest (ties: lowest index) get softmax(z over the chosen) as weights
//   ids [T, top] int, wts [T, top] float (if not null)
//   act != nullptr:  act[t, e*ff + c] = weight_e * silu(gu[t, e*2ff + c]) * gu[t, e*2ff + ff + c], 0 for experts not chosen
template <typename OT>
__global__ void moe_route_kernel(const float* __restrict__ router, long sr, const float* __restrict__ router_bias, int E, int top,
                                 const float* __restrict__ gu, long sgu, int ff, OT* __restrict__ act, long sa, int* __restrict__ ids,
                                 float* __restrict__ wts) {
  extern __shared__ float smf[];
  float* z = smf;                 // [E]
  float* wsel = z + E;            // [E]: weight, 0 = not chosen
  const long t = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    z[e] = router[t * sr + e] + (router_bias != nullptr ? router_bias[e] : 0.f);
    wsel[e] = 0.f;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float zmax = 0.f, denom = 0.f;
    for (int k = 0; k < top; ++k) {
      float best = -INFINITY;
      int bi = E;
      for (int e = lane; e < E; e += 32) {
        const float v = z[e];
        if (v > best || (v == best && e < bi)) { best = v; bi = e; }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (k == 0) zmax = best;
      const float p = expf(best - zmax);
      denom += p;
      __syncwarp();
      if (lane == 0) {
        wsel[bi] = p;
        z[bi] = -INFINITY;            // taken
        if (ids != nullptr) ids[t * top + k] = bi;
      }
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32) wsel[e] = wsel[e] / denom;
    __syncwarp();
    if (wts != nullptr)
      for (int k = lane; k < top; k += 32) wts[t * top + k] = wsel[ids[t * top + k]];
  }
  __syncthreads();
  if (act == nullptr) return;
  const long n = static_cast<long>(E) * ff;
  for (long idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int e = static_cast<int>(idx / ff), c = static_cast<int>(idx - static_cast<long>(e) * ff);
    const float w = wsel[e];
    float v = 0.f;
    if (w != 0.f) {
      const float gt = gu[t * sgu + static_cast<long>(e) * 2 * ff + c], up = gu[t * sgu + static_cast<long>(e) * 2 * ff + ff + c];
      v = w * (gt * sigmoidf_(gt) * up);
    }
    st(act, t * sa + idx, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Stream with the norm on the sublayer's OUTPUT only: sublayers read x itself, x += rms_norm(sublayer(x)) * w.
// ---------------------------------------------------------------------------------------------------------------------
// x[t] = e / sqrt(mean(e^2) + eps) * w with e = embed[tok[t]];  h = x (typed).  One block per token.
template <typename WT, typename HT>
__global__ void embed_norm_kernel(const WT* __restrict__ embed, const int* __restrict__ tok, const float* __restrict__ w, float eps,
                                  float* __restrict__ x, HT* __restrict__ h, int W) {
  __shared__ float red[32];
  const long t = blockIdx.x, a = static_cast<long>(tok[t]) * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = ld(embed, a + c);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss / static_cast<float>(W) + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = ld(embed, a + c) * r * w[c];
    x[t * W + c] = v;
    st(h, t * W + c, v);
  }
}

// Sublayer boundary, one block per token, the row staged in shared memory (o and x are read once, x and h written once):
//   y = o + self_w[t] * x   (self_w == nullptr: y = o);   x += y / sqrt(mean(y^2) + eps) * w_post
//   h = w_pre ? x / sqrt(mean(x^2) + eps) * w_pre : x                                 (typed)
template <typename HT, int V>
__global__ void post_norm_residual_kernel(float* __restrict__ x, const float* __restrict__ o, const float* __restrict__ self_w,
                                          const float* __restrict__ w_post, const float* __restrict__ w_pre, float eps,
                                          HT* __restrict__ h, int W) {
  extern __shared__ __align__(16) float rowbuf[];       // [W]: y, then the new x
  __shared__ float red[32];
  const long row = static_cast<long>(blockIdx.x) * W;
  const float sw = self_w != nullptr ? self_w[blockIdx.x] : 0.f;
  const float inv = 1.f / static_cast<float>(W);
  float ss = 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float y[V], xv[V];
    ldv<V>(o + row + c, y);
    if (self_w != nullptr) {
      ldv<V>(x + row + c, xv);
#pragma unroll
      for (int e = 0; e < V; ++e) y[e] += sw * xv[e];
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      ss += y[e] * y[e];
      rowbuf[c + e] = y[e];
    }
  }
  ss = block_sum(ss, red);
  const float r = 1.f / sqrtf(ss * inv + eps);
  float s2 = 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {       // a thread re-reads the columns it staged itself
    float xv[V], wv[V];
    ldv<V>(x + row + c, xv);
    ldv<V>(w_post + c, wv);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      xv[e] += rowbuf[c + e] * r * wv[e];
      rowbuf[c + e] = xv[e];
      s2 += xv[e] * xv[e];
    }
    stv<V>(x + row + c, xv);
    if (h != nullptr && w_pre == nullptr) stv<V>(h + row + c, xv);
  }
  if (h == nullptr || w_pre == nullptr) return;
  s2 = block_sum(s2, red);
  const float r2 = 1.f / sqrtf(s2 * inv + eps);
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float hv[V], wv[V];
    ldv<V>(w_pre + c, wv);
#pragma unroll
    for (int e = 0; e < V; ++e) hv[e] = rowbuf[c + e] * r2 * wv[e];
    stv<V>(h + row + c, hv);
  }
}

__device__ __forceinline__ float gelu_tanh_(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// Gated token-side input: out[t, c] (typed, row stride so; columns C..Cpad-1 zero) = gelu_tanh(u[t, c]) * table[tok[t], col0 + c]
template <typename WT, typename OT>
__global__ void side_gate_kernel(const float* __restrict__ u, long su, const WT* __restrict__ table, long st_, int col0,
                                 const int* __restrict__ tok, OT* __restrict__ out, long so, long T, int C, int Cpad) {
  const long n = T * Cpad;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / Cpad;
    const int c = static_cast<int>(idx - t * Cpad);
    float v = 0.f;
    if (c < C) v = gelu_tanh_(u[t * su + c]) * ld(table, static_cast<long>(tok[t]) * st_ + col0 + c);
    st(out, t * so + c, v);
  }
}

// out[t, c] (typed) = silu(in[t, c]) * in[t, C + c] * (rgate ? sigmoid(rgate[t * srg]) : 1):  SwiGLU over [gate | up] columns with an
// optional sigmoid gate per row
template <typename OT>
__global__ void swiglu_cols_kernel(const float* __restrict__ in, long si, const float* __restrict__ rgate, long srg, OT* __restrict__ out,
                                   long so, long T, int C) {
  const long n = T * C;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / C;
    const int c = static_cast<int>(idx - t * C);
    const float g = in[t * si + c], up = in[t * si + C + c];
    float v = g * sigmoidf_(g) * up;
    if (rgate != nullptr) v *= sigmoidf_(rgate[t * srg]);
    st(out, t * so + c, v);
  }
}

// the same, four columns per thread (128-bit loads, 64- / 128-bit stores)
template <typename OT>
__global__ void swiglu_cols_vec4_kernel(const float* __restrict__ in, long si, const float* __restrict__ rgate, long srg,
                                        OT* __restrict__ out, long so, long T, int C4) {
  const long n = T * C4;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / C4;
    const int c = static_cast<int>(idx - t * C4) * 4;
    float g[4], up[4], v[4];
    ldv<4>(in + t * si + c, g);
    ldv<4>(in + t * si + 4 * C4 + c, up);
    const float rg = rgate != nullptr ? sigmoidf_(rgate[t * srg]) : 1.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = g[i] * sigmoidf_(g[i]) * up[i] * rg;
    st4(out + t * so + c, v);
  }
}

// Routing by a softmax over ALL router outputs, one warp per token.  E outputs, of which the last E - n_real are identity
// experts (their result is the expert's input).  s = softmax(z);  the `top` largest s + correction are chosen (ties: lowest
// index);  weight = s / (sum of the chosen s + 1e-20) * route_scale.
//   ids [T, top] int;  wts [T, top] float: the weight, 0 for a chosen identity expert;  self_w [T]: the identity experts' weights, summed
//   act != nullptr (dense form):  act[t, e*ff + c] = weight_e * silu(gu[t, e*2ff + c]) * gu[t, e*2ff + ff + c] for e < n_real, 0 if not chosen
template <typename OT>
__global__ void moe_route_all_kernel(const float* __restrict__ router, long sr, const float* __restrict__ correction, int E, int n_real,
                                     int top, float route_scale, int groups, int keep, const float* __restrict__ gu, long sgu, int ff,
                                     OT* __restrict__ act, long sa, int* __restrict__ ids, float* __restrict__ wts,
                                     float* __restrict__ self_w) {
  extern __shared__ float smf[];
  float* sc = smf;                // [E] softmax scores
  float* ch = sc + E;             // [E] choice scores, -inf once taken
  float* wsel = ch + E;           // [E] weight, 0 = not chosen
  __shared__ int chosen[64];
  const long t = blockIdx.x;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, router[t * sr + e]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float den = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = expf(router[t * sr + e] - mx);
      sc[e] = p;
      den += p;
    }
    den = warp_sum(den);
    for (int e = lane; e < E; e += 32) {
      const float p = sc[e] / den;
      sc[e] = p;
      ch[e] = p + (correction != nullptr ? correction[e] : 0.f);
      wsel[e] = 0.f;
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
      // Only the `keep` groups of neighbours with the largest choice score stay eligible (ties: the lower group).  A group is
      // dropped when at least `keep` others come before it; its experts count as -inf.  Every lane walks the same groups.
      const int gsz = E / groups;
      for (int g = lane; g < groups; g += 32) {
        float b = -INFINITY;
        for (int e = g * gsz; e < (g + 1) * gsz; ++e) b = fmaxf(b, ch[e]);
        wsel[g] = b;                                          // borrowed: groups <= E
      }
      __syncwarp();
      unsigned drop = 0u;                                     // bit i: group lane + 32 i is dropped (groups <= 1024)
      for (int g = lane, i = 0; g < groups; g += 32, ++i) {
        const float mine = wsel[g];
        int before = 0;
        for (int o = 0; o < groups; ++o) {
          const float v = wsel[o];
          before += (v > mine || (v == mine && o < g)) ? 1 : 0;
        }
        if (before >= keep) drop |= 1u << i;
      }
      __syncwarp();
      for (int g = lane, i = 0; g < groups; g += 32, ++i) {
        wsel[g] = 0.f;
        if (drop >> i & 1u)
          for (int e = g * gsz; e < (g + 1) * gsz; ++e) ch[e] = -INFINITY;
      }
      __syncwarp();
    }
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      float best = -INFINITY;
      int bi = E;
      for (int e = lane; e < E; e += 32) {
        const float v = ch[e];
        if (v > best || (v == best && e < bi)) { best = v; bi = e; }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      sum += sc[bi];
      __syncwarp();
      if (lane == 0) {
        ch[bi] = -INFINITY;
        chosen[k] = bi;
      }
      __syncwarp();
    }
    const float norm = route_scale / (sum + 1e-20f);
    float idw = 0.f;
    for (int k = 0; k < top; ++k) {                         // every lane walks the chosen in order: same sums on all lanes
      const int e = chosen[k];
      const float w = sc[e] * norm;
      if (e >= n_real) idw += w;
      if (lane == 0) {
        if (e < n_real) wsel[e] = w;
        if (ids != nullptr) ids[t * top + k] = e;
        if (wts != nullptr) wts[t * top + k] = e < n_real ? w : 0.f;
      }
    }
    if (lane == 0 && self_w != nullptr) self_w[t] = idw;
  }
  __syncthreads();
  if (act == nullptr) return;
  const long n = static_cast<long>(n_real) * ff;
  for (long idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int e = static_cast<int>(idx / ff), c = static_cast<int>(idx - static_cast<long>(e) * ff);
    const float w = wsel[e];
    float v = 0.f;
    if (w != 0.f) {
      const float gt = gu[t * sgu + static_cast<long>(e) * 2 * ff + c], up = gu[t * sgu + static_cast<long>(e) * 2 * ff + ff + c];
      v = w * (gt * sigmoidf_(gt) * up);
    }
    st(act, t * sa + idx, v);
  }
}

template <typename OT>
__global__ void act_cols_kernel(const float* __restrict__ in, long si, OT* __restrict__ out, long so, int act, long T, int C) {
  const long n = T * C;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / C;
    const int c = static_cast<int>(idx - t * C);
    float v = in[t * si + c];
    if (act == 1) {
      v = fmaxf(v, 0.f);
      v = v * v;
    }
    st(out, t * so + c, v);
  }
}

// four columns per thread: 128-bit loads, 64- / 128-bit stores
template <typename OT>
__global__ void act_cols_vec4_kernel(const float* __restrict__ in, long si, OT* __restrict__ out, long so, int act, long T, int C4) {
  const long n = T * C4;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / C4;
    const int c = static_cast<int>(idx - t * C4) * 4;
    float v[4];
    ldv<4>(in + t * si + c, v);
    if (act == 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = fmaxf(v[i], 0.f);
        v[i] = v[i] * v[i];
      }
    }
    st4(out + t * so + c, v);
  }
}

__device__ __forceinline__ float gate_fn(float z, int act) {
  const float sg = 1.f / (1.f + expf(-z));
  return act == 0 ? z * sg : sg;
}

// one warp per (token, part); V columns per lane and pass
template <typename OT, int V>
__global__ void gated_part_rmsnorm_kernel(const float* __restrict__ y, long sy, const float* __restrict__ gate, long sg,
                                          const float* __restrict__ w, int shared_w, int part, int gate_act, int gate_first,
                                          float eps, float scale, OT* __restrict__ out, long so, long T, int nparts) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * nparts) return;
  const long t = wid / nparts;
  const int p = static_cast<int>(wid - t * nparts);
  const float* yr = y + t * sy + static_cast<long>(p) * part;
  const float* gr = gate + t * sg + static_cast<long>(p) * part;
  float ss = 0.f;
  for (int c = lane * V; c < part; c += 32 * V) {
    float v[V], gv[V];
    ldv<V>(yr + c, v);
    if (gate_first) ldv<V>(gr + c, gv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if (gate_first) v[i] *= gate_fn(gv[i], gate_act);
      ss += v[i] * v[i];
    }
  }
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / static_cast<float>(part) + eps);
  for (int c = lane * V; c < part; c += 32 * V) {
    float v[V], gv[V], wv[V];
    ldv<V>(yr + c, v);
    ldv<V>(gr + c, gv);
    ldv<V>(w + (shared_w ? c : p * part + c), wv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float gg = gate_fn(gv[i], gate_act);
      v[i] = scale * (gate_first ? (v[i] * gg) * r * wv[i] : v[i] * r * wv[i] * gg);
    }
    stv<V>(out + t * so + static_cast<long>(p) * part + c, v);
  }
}

// one block per (token, part): wide parts (a warp alone would walk them serially)
template <typename OT, int V>
__global__ void gated_part_rmsnorm_block_kernel(const float* __restrict__ y, long sy, const float* __restrict__ gate, long sg,
                                                const float* __restrict__ w, int shared_w, int part, int gate_act, int gate_first,
                                                float eps, float scale, OT* __restrict__ out, long so, int nparts) {
  __shared__ float red[8];
  const long t = blockIdx.x / nparts;
  const int p = static_cast<int>(blockIdx.x - t * nparts);
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* yr = y + t * sy + static_cast<long>(p) * part;
  const float* gr = gate + t * sg + static_cast<long>(p) * part;
  float ss = 0.f;
  for (int c = threadIdx.x * V; c < part; c += blockDim.x * V) {
    float v[V], gv[V];
    ldv<V>(yr + c, v);
    if (gate_first) ldv<V>(gr + c, gv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if (gate_first) v[i] *= gate_fn(gv[i], gate_act);
      ss += v[i] * v[i];
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[wi] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < nw; ++i) tot += red[i];
  const float r = 1.f / sqrtf(tot / static_cast<float>(part) + eps);
  for (int c = threadIdx.x * V; c < part; c += blockDim.x * V) {
    float v[V], gv[V], wv[V];
    ldv<V>(yr + c, v);
    ldv<V>(gr + c, gv);
    ldv<V>(w + (shared_w ? c : p * part + c), wv);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float gg = gate_fn(gv[i], gate_act);
      v[i] = scale * (gate_first ? (v[i] * gg) * r * wv[i] : v[i] * r * wv[i] * gg);
    }
    stv<V>(out + t * so + static_cast<long>(p) * part + c, v);
  }
}

}  // namespace

namespace {
template <typename OT, int V>
cudaError_t launch_gated_norm(const float* y, long sy, const float* gate, long sg, const float* w, int shared_w, int part, int gate_act,
                              int gate_first, float eps, float scale, OT* out, long so, int T, int nparts, cudaStream_t s) {
  const long warps = static_cast<long>(T) * nparts;
  if (part >= 256) {
    const int th = part >= 1024 * V / 4 ? 256 : 128;
    gated_part_rmsnorm_block_kernel<OT, V><<<static_cast<unsigned>(warps), th, 0, s>>>(y, sy, gate, sg, w, shared_w, part, gate_act,
                                                                                      gate_first, eps, scale, out, so, nparts);
  } else {
    gated_part_rmsnorm_kernel<OT, V><<<static_cast<unsigned>((warps + 3) / 4), 128, 0, s>>>(y, sy, gate, sg, w, shared_w, part, gate_act,
                                                                                            gate_first, eps, scale, out, so, T, nparts);
  }
  return cudaGetLastError();
}
}  // namespace


namespace {
inline bool aligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }
// ---------------------------------------------------------------------------------------------------------------------
// Several residual streams mixed by learned weights (hyper-connections), with a layer norm (weight and bias) in front of every
// sublayer.  xs float [T, S, W].
// ---------------------------------------------------------------------------------------------------------------------
// xs[t, s, :] = embed[tok[t]] * scale for every stream s
template <typename WT>
__global__ void embed_streams_kernel(const WT* __restrict__ embed, const int* __restrict__ tok, float scale, float* __restrict__ xs,
                                     int S, int W) {
  const long t = blockIdx.x;
  const WT* row = embed + static_cast<long>(tok[t]) * W;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = ld(row, c) * scale;
    for (int s = 0; s < S; ++s) xs[(t * S + s) * W + c] = v;
  }
}

constexpr int kMaxStreams = 8;

// Block per token.  Closes a sublayer whose result is o (+ o_bias + self_w[t] * h, h being the sublayer's own input, still in
// place) -- x_t <- sum_s mix[s, t] x_s + outw[t] y, all streams from the old ones -- and opens the next one:
// u = sum_s inw[s] x_s (inw null: the plain sum), h = (u - mean) / sqrt(var + eps) * ln_w + ln_b.
// SM: the stream count rounded up (loops are unrolled over it); V: columns per access (4 needs W % 4 == 0 and aligned rows).
template <typename HT, int SM, int V>
__global__ void hyper_boundary_kernel(float* __restrict__ xs, int S, const float* __restrict__ o, const float* __restrict__ o_bias,
                                      const float* __restrict__ self_w, const float* __restrict__ mix, const float* __restrict__ outw,
                                      const float* __restrict__ inw, const float* __restrict__ ln_w, const float* __restrict__ ln_b,
                                      float eps, HT* __restrict__ h, int W) {
  extern __shared__ __align__(16) float rowbuf[];       // [W]: u
  __shared__ float red[32];
  __shared__ float smix[kMaxStreams * kMaxStreams], sout[kMaxStreams], sin_[kMaxStreams];
  const long t = blockIdx.x;
  if (threadIdx.x < S * S) smix[threadIdx.x] = (o != nullptr && mix != nullptr) ? mix[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    sout[threadIdx.x] = (o != nullptr && outw != nullptr) ? outw[threadIdx.x] : 1.f;
    sin_[threadIdx.x] = inw != nullptr ? inw[threadIdx.x] : 1.f;
  }
  __syncthreads();
  const float sw = (o != nullptr && self_w != nullptr) ? self_w[t] : 0.f;
  float* xt = xs + t * S * W;
  float sum = 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float xv[SM][V], u[V];
#pragma unroll
    for (int s = 0; s < SM; ++s)
      if (s < S) ldv<V>(xt + static_cast<long>(s) * W + c, xv[s]);
#pragma unroll
    for (int e = 0; e < V; ++e) u[e] = 0.f;
    if (o != nullptr) {
      float y[V];
      ldv<V>(o + t * W + c, y);
      if (o_bias != nullptr) {
        float b[V];
        ldv<V>(o_bias + c, b);
#pragma unroll
        for (int e = 0; e < V; ++e) y[e] += b[e];
      }
      if (self_w != nullptr) {
#pragma unroll
        for (int e = 0; e < V; ++e) y[e] += sw * ld(h, t * W + c + e);
      }
#pragma unroll
      for (int to = 0; to < SM; ++to) {
        if (to < S) {
          float a[V];
#pragma unroll
          for (int e = 0; e < V; ++e) a[e] = 0.f;
#pragma unroll
          for (int s = 0; s < SM; ++s) {
            if (s < S) {
              const float m = smix[s * S + to];
#pragma unroll
              for (int e = 0; e < V; ++e) a[e] += m * xv[s][e];
            }
          }
          const float ow = sout[to], iw = sin_[to];
#pragma unroll
          for (int e = 0; e < V; ++e) {
            a[e] += ow * y[e];
            u[e] += iw * a[e];
          }
          stv<V>(xt + static_cast<long>(to) * W + c, a);
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < SM; ++s) {
        if (s < S) {
          const float iw = sin_[s];
#pragma unroll
          for (int e = 0; e < V; ++e) u[e] += iw * xv[s][e];
        }
      }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) {
      rowbuf[c + e] = u[e];
      sum += u[e];
    }
  }
  if (h == nullptr) return;
  const float inv = 1.f / static_cast<float>(W);
  const float mean = block_sum(sum, red) * inv;
  float ss = 0.f;
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {     // a thread re-reads the columns it staged itself
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float d = rowbuf[c + e] - mean;
      ss += d * d;
    }
  }
  const float r = 1.f / sqrtf(block_sum(ss, red) * inv + eps);
  for (int c = threadIdx.x * V; c < W; c += blockDim.x * V) {
    float hv[V], wv[V], bv[V];
    ldv<V>(ln_w + c, wv);
    if (ln_b != nullptr) ldv<V>(ln_b + c, bv);
#pragma unroll
    for (int e = 0; e < V; ++e) hv[e] = (rowbuf[c + e] - mean) * r * wv[e] + (ln_b != nullptr ? bv[e] : 0.f);
    stv<V>(h + t * W + c, hv);
  }
}

}  // namespace

extern "C" {

cudaError_t nrl_embed_pos(const void* embed, const void* pos_table, int w_f32, const int* tok, const int* pos, float* out, int T,
                          int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const int th = W >= 256 ? 256 : 128;
  if (w_f32)
    embed_pos_kernel<float><<<T, th, 0, s>>>(static_cast<const float*>(embed), static_cast<const float*>(pos_table), tok, pos, out, W);
  else
    embed_pos_kernel<__nv_bfloat16><<<T, th, 0, s>>>(static_cast<const __nv_bfloat16*>(embed),
                                                    static_cast<const __nv_bfloat16*>(pos_table), tok, pos, out, W);
  return cudaGetLastError();
}

cudaError_t nrl_embed_hashed(const void* embed, const void* pair, int w_f32, const int* tok, const int* cu, const int* tok_entry,
                             const int* start, const int* state_slot, int* prev_state, float scale, long mul_prev, long mul_cur,
                             long buckets, float* out, int T, int E, int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const int th = W >= 256 ? 256 : 128;
  if (w_f32)
    embed_hashed_kernel<float><<<T, th, 0, s>>>(static_cast<const float*>(embed), static_cast<const float*>(pair), tok, cu, tok_entry,
                                                start, state_slot, prev_state, scale, mul_prev, mul_cur, buckets, out, W);
  else
    embed_hashed_kernel<__nv_bfloat16><<<T, th, 0, s>>>(static_cast<const __nv_bfloat16*>(embed),
                                                        static_cast<const __nv_bfloat16*>(pair), tok, cu, tok_entry, start, state_slot,
                                                        prev_state, scale, mul_prev, mul_cur, buckets, out, W);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || prev_state == nullptr) return e;
  token_carry_kernel<<<(E + 127) / 128, 128, 0, s>>>(tok, cu, state_slot, prev_state, E);
  return cudaGetLastError();
}

cudaError_t nrl_group_norm_residual(float* x, const float* o, const float* gate, long sg, const float* gate_bias, const float* w_post,
                                    const float* w_pre, int groups, float eps, void* h, int h_f32, int T, int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (groups < 1 || W % groups != 0 || (o != nullptr && w_post == nullptr) || (h != nullptr && w_pre == nullptr)) return cudaErrorInvalidValue;
  const int part = W / groups;
  const bool vec = part % 4 == 0 && sg % 4 == 0 && aligned(x, 16) && (o == nullptr || aligned(o, 16)) && (gate == nullptr || aligned(gate, 16)) &&
                   (gate_bias == nullptr || aligned(gate_bias, 16)) && (w_post == nullptr || aligned(w_post, 16)) &&
                   (w_pre == nullptr || aligned(w_pre, 16)) && (h == nullptr || aligned(h, h_f32 ? 16 : 8)) && part <= 8 * 4 * 256;
  if (vec) {
    const int part4 = part / 4;
    int tv = part4 <= 32 ? 32 : part4 <= 64 ? 64 : part4 <= 256 ? 128 : 256;      // up to 2 float4 per thread before the block grows
    const int nv = (part4 + tv - 1) / tv;
#define NRL_GNR(HT_, NV_)                                                                                                          \
  group_norm_residual_vec_kernel<HT_, NV_><<<T, tv, 0, s>>>(x, o, gate, sg, gate_bias, w_post, w_pre, groups, eps, static_cast<HT_*>(h), W)
#define NRL_GNR_NV(HT_)                                                                                                            \
  do {                                                                                                                             \
    if (nv <= 1) NRL_GNR(HT_, 1);                                                                                                  \
    else if (nv <= 2) NRL_GNR(HT_, 2);                                                                                             \
    else if (nv <= 4) NRL_GNR(HT_, 4);                                                                                             \
    else NRL_GNR(HT_, 8);                                                                                                          \
  } while (0)
    if (h_f32) NRL_GNR_NV(float);
    else NRL_GNR_NV(__nv_bfloat16);
#undef NRL_GNR_NV
#undef NRL_GNR
    return cudaGetLastError();
  }
  const int th = part >= 1024 ? 256 : part >= 128 ? 128 : 64;
  if (h_f32)
    group_norm_residual_kernel<float><<<T, th, 0, s>>>(x, o, gate, sg, gate_bias, w_post, w_pre, groups, eps, static_cast<float*>(h), W);
  else
    group_norm_residual_kernel<__nv_bfloat16><<<T, th, 0, s>>>(x, o, gate, sg, gate_bias, w_post, w_pre, groups, eps,
                                                               static_cast<__nv_bfloat16*>(h), W);
  return cudaGetLastError();
}

cudaError_t nrl_moe_route(const float* router, long sr, const float* router_bias, int E, int top, const float* gu, long sgu, int ff,
                          void* act, long sa, int act_f32, int* ids, float* wts, int T, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (E < 1 || top < 1 || top > E || E > 4096 || (wts != nullptr && ids == nullptr)) return cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * 2 * E;
  const int th = act == nullptr ? 32 : 256;
  if (act_f32)
    moe_route_kernel<float><<<T, th, smem, s>>>(router, sr, router_bias, E, top, gu, sgu, ff, static_cast<float*>(act), sa, ids, wts);
  else
    moe_route_kernel<__nv_bfloat16><<<T, th, smem, s>>>(router, sr, router_bias, E, top, gu, sgu, ff, static_cast<__nv_bfloat16*>(act),
                                                        sa, ids, wts);
  return cudaGetLastError();
}

cudaError_t nrl_embed_norm(const void* embed, int w_f32, const int* tok, const float* w, float eps, float* x, void* h, int h_f32, int T,
                           int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const int th = W >= 1024 ? 256 : 128;
#define NRL_EN(WT_, HT_) embed_norm_kernel<WT_, HT_><<<T, th, 0, s>>>(static_cast<const WT_*>(embed), tok, w, eps, x, static_cast<HT_*>(h), W)
  if (w_f32 && h_f32) NRL_EN(float, float);
  else if (w_f32) NRL_EN(float, __nv_bfloat16);
  else if (h_f32) NRL_EN(__nv_bfloat16, float);
  else NRL_EN(__nv_bfloat16, __nv_bfloat16);
#undef NRL_EN
  return cudaGetLastError();
}

cudaError_t nrl_post_norm_residual(float* x, const float* o, const float* self_w, const float* w_post, const float* w_pre, float eps,
                                   void* h, int h_f32, int T, int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (o == nullptr || w_post == nullptr || W < 1 || W > 12 * 1024) return cudaErrorInvalidValue;
  const bool vec = W % 4 == 0 && aligned(x, 16) && aligned(o, 16) && aligned(w_post, 16) && (w_pre == nullptr || aligned(w_pre, 16)) &&
                   (h == nullptr || aligned(h, h_f32 ? 16 : 8));
  const int per = vec ? W / 4 : W;
  const int th = per <= 64 ? 64 : per <= 128 ? 128 : 256;
  const size_t smem = sizeof(float) * W;
#define NRL_PN(HT_, V_) post_norm_residual_kernel<HT_, V_><<<T, th, smem, s>>>(x, o, self_w, w_post, w_pre, eps, static_cast<HT_*>(h), W)
  if (h_f32) {
    if (vec) NRL_PN(float, 4);
    else NRL_PN(float, 1);
  } else {
    if (vec) NRL_PN(__nv_bfloat16, 4);
    else NRL_PN(__nv_bfloat16, 1);
  }
#undef NRL_PN
  return cudaGetLastError();
}

cudaError_t nrl_side_gate(const float* u, long su, const void* table, long st_, int w_f32, int col0, const int* tok, void* out, long so,
                          int out_f32, int T, int C, int Cpad, cudaStream_t s) {
  if (T <= 0 || Cpad <= 0) return cudaSuccess;
  if (C > Cpad) return cudaErrorInvalidValue;
  const long n = static_cast<long>(T) * Cpad;
  const int blocks = static_cast<int>((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
#define NRL_SG(WT_, OT_) side_gate_kernel<WT_, OT_><<<blocks, 256, 0, s>>>(u, su, static_cast<const WT_*>(table), st_, col0, tok, static_cast<OT_*>(out), so, T, C, Cpad)
  if (w_f32 && out_f32) NRL_SG(float, float);
  else if (w_f32) NRL_SG(float, __nv_bfloat16);
  else if (out_f32) NRL_SG(__nv_bfloat16, float);
  else NRL_SG(__nv_bfloat16, __nv_bfloat16);
#undef NRL_SG
  return cudaGetLastError();
}

cudaError_t nrl_swiglu_cols(const float* in, long si, const float* rgate, long srg, void* out, long so, int out_f32, int T, int C,
                            cudaStream_t s) {
  if (T <= 0 || C <= 0) return cudaSuccess;
  if (C % 4 == 0 && si % 4 == 0 && so % 4 == 0 && aligned(in, 16) && aligned(out, out_f32 ? 16 : 8)) {
    const long n4 = static_cast<long>(T) * (C / 4);
    const int blocks4 = static_cast<int>((n4 + 255) / 256 < 148 * 16 ? (n4 + 255) / 256 : 148 * 16);
    if (out_f32) swiglu_cols_vec4_kernel<float><<<blocks4, 256, 0, s>>>(in, si, rgate, srg, static_cast<float*>(out), so, T, C / 4);
    else swiglu_cols_vec4_kernel<__nv_bfloat16><<<blocks4, 256, 0, s>>>(in, si, rgate, srg, static_cast<__nv_bfloat16*>(out), so, T, C / 4);
    return cudaGetLastError();
  }
  const long n = static_cast<long>(T) * C;
  const int blocks = static_cast<int>((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (out_f32) swiglu_cols_kernel<float><<<blocks, 256, 0, s>>>(in, si, rgate, srg, static_cast<float*>(out), so, T, C);
  else swiglu_cols_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(in, si, rgate, srg, static_cast<__nv_bfloat16*>(out), so, T, C);
  return cudaGetLastError();
}

cudaError_t nrl_moe_route_all(const float* router, long sr, const float* correction, int E, int n_real, int top, float route_scale,
                              int groups, int keep, const float* gu, long sgu, int ff, void* act, long sa, int act_f32, int* ids,
                              float* wts, float* self_w, int T, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (E < 1 || top < 1 || top > E || top > 64 || E > 4096 || n_real < 0 || n_real > E || (n_real < E && self_w == nullptr))
    return cudaErrorInvalidValue;
  if (groups > 1 && (E % groups != 0 || keep < 1 || groups > 1024 || keep * (E / groups) < top)) return cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * 3 * E;
  const int th = act == nullptr ? 32 : 256;
  if (act_f32)
    moe_route_all_kernel<float><<<T, th, smem, s>>>(router, sr, correction, E, n_real, top, route_scale, groups, keep, gu, sgu, ff,
                                                    static_cast<float*>(act), sa, ids, wts, self_w);
  else
    moe_route_all_kernel<__nv_bfloat16><<<T, th, smem, s>>>(router, sr, correction, E, n_real, top, route_scale, groups, keep, gu, sgu,
                                                            ff, static_cast<__nv_bfloat16*>(act), sa, ids, wts, self_w);
  return cudaGetLastError();
}

cudaError_t nrl_stream_norm(float* results, long stride_r, int i, const float* o, const float* xprev, const float* dw,
                            const float* g, float eps, float* xcur, void* h, int h_f32, int T, int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const bool vec = W % 4 == 0 && stride_r % 4 == 0 && aligned(results, 16) && aligned(xcur, 16) && aligned(h, h_f32 ? 16 : 8) &&
                   (o == nullptr || (aligned(o, 16) && aligned(xprev, 16)));
  const int th = W >= 1024 * (vec ? 4 : 1) ? 256 : 128;
#define NRL_SN(HT_, V_)                                                                                                            \
  stream_norm_kernel<HT_, V_><<<T, th, 0, s>>>(results, stride_r, i, o, xprev, dw, g, eps, xcur, static_cast<HT_*>(h), W)
  if (h_f32) {
    if (vec) NRL_SN(float, 4);
    else NRL_SN(float, 1);
  } else {
    if (vec) NRL_SN(__nv_bfloat16, 4);
    else NRL_SN(__nv_bfloat16, 1);
  }
#undef NRL_SN
  return cudaGetLastError();
}

cudaError_t nrl_act_cols(const float* in, long si, void* out, long so, int out_f32, int act, int T, int C, cudaStream_t s) {
  if (T <= 0 || C <= 0) return cudaSuccess;
  const size_t out_align = out_f32 ? 16 : 8;
  if (C % 4 == 0 && si % 4 == 0 && so % 4 == 0 && aligned(in, 16) && aligned(out, out_align)) {
    const long n = static_cast<long>(T) * (C / 4);
    const int blocks = static_cast<int>((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (out_f32)
      act_cols_vec4_kernel<float><<<blocks, 256, 0, s>>>(in, si, static_cast<float*>(out), so, act, T, C / 4);
    else
      act_cols_vec4_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(in, si, static_cast<__nv_bfloat16*>(out), so, act, T, C / 4);
    return cudaGetLastError();
  }
  const long n = static_cast<long>(T) * C;
  const int blocks = static_cast<int>((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (out_f32)
    act_cols_kernel<float><<<blocks, 256, 0, s>>>(in, si, static_cast<float*>(out), so, act, T, C);
  else
    act_cols_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(in, si, static_cast<__nv_bfloat16*>(out), so, act, T, C);
  return cudaGetLastError();
}

cudaError_t nrl_gated_part_rmsnorm(const float* y, long sy, const float* gate, long sg, const float* w, int shared_w, int part,
                                   int gate_act, int gate_first, float eps, float scale, void* out, long so, int out_f32, int T,
                                   int n, cudaStream_t s) {
  if (T <= 0 || n <= 0) return cudaSuccess;
  if (part <= 0 || n % part != 0) return cudaErrorInvalidValue;
  const int nparts = n / part;
  const bool vec = part % 4 == 0 && sy % 4 == 0 && sg % 4 == 0 && so % 4 == 0 && aligned(y, 16) && aligned(gate, 16) && aligned(w, 16) &&
                   aligned(out, out_f32 ? 16 : 8);
#define NRL_GN(OT_, V_)                                                                                                            \
  return launch_gated_norm<OT_, V_>(y, sy, gate, sg, w, shared_w, part, gate_act, gate_first, eps, scale, static_cast<OT_*>(out), so, T, \
                                    nparts, s)
  if (out_f32) {
    if (vec) NRL_GN(float, 4);
    NRL_GN(float, 1);
  }
  if (vec) NRL_GN(__nv_bfloat16, 4);
  NRL_GN(__nv_bfloat16, 1);
#undef NRL_GN
}

cudaError_t nrl_embed_streams(const void* embed, int w_f32, const int* tok, float scale, float* xs, int T, int S, int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (S < 1) return cudaErrorInvalidValue;
  const int th = W >= 512 ? 256 : 128;
  if (w_f32) embed_streams_kernel<float><<<T, th, 0, s>>>(static_cast<const float*>(embed), tok, scale, xs, S, W);
  else embed_streams_kernel<__nv_bfloat16><<<T, th, 0, s>>>(static_cast<const __nv_bfloat16*>(embed), tok, scale, xs, S, W);
  return cudaGetLastError();
}

cudaError_t nrl_hyper_boundary(float* xs, int S, const float* o, const float* o_bias, const float* self_w, const float* mix,
                               const float* outw, const float* inw, const float* ln_w, const float* ln_b, float eps, void* h, int h_f32,
                               int T, int W, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (S < 1 || S > kMaxStreams || (h != nullptr && ln_w == nullptr) || (self_w != nullptr && h == nullptr)) return cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * W;
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  const bool vec = W % 4 == 0 && aligned(xs, 16) && (o == nullptr || aligned(o, 16)) && (o_bias == nullptr || aligned(o_bias, 16)) &&
                   (h == nullptr || aligned(h, h_f32 ? 16 : 8)) && (ln_w == nullptr || aligned(ln_w, 16)) &&
                   (ln_b == nullptr || aligned(ln_b, 16));
  const int th = W >= 1024 * (vec ? 4 : 1) ? 256 : 128;
#define NRL_HB(HT_, SM_, V_)                                                                                                       \
  hyper_boundary_kernel<HT_, SM_, V_><<<T, th, smem, s>>>(xs, S, o, o_bias, self_w, mix, outw, inw, ln_w, ln_b, eps, static_cast<HT_*>(h), W)
#define NRL_HB_S(HT_, V_)                                                                                                          \
  do {                                                                                                                             \
    if (S == 1) NRL_HB(HT_, 1, V_);                                                                                                \
    else if (S == 2) NRL_HB(HT_, 2, V_);                                                                                           \
    else if (S <= 4) NRL_HB(HT_, 4, V_);                                                                                           \
    else NRL_HB(HT_, 8, V_);                                                                                                       \
  } while (0)
  if (h_f32) {
    if (vec) NRL_HB_S(float, 4);
    else NRL_HB_S(float, 1);
  } else {
    if (vec) NRL_HB_S(__nv_bfloat16, 4);
    else NRL_HB_S(__nv_bfloat16, 1);
  }
#undef NRL_HB_S
#undef NRL_HB
  return cudaGetLastError();
}

}  // extern "C"
