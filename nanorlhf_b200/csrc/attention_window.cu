// Sliding-window attention over the paged KV cache, for prompt portions and decoded tokens alike: the keys of a step's own
// tokens are written to their pages first (nrl_qknorm_kv_write), then every token reads the last `window` keys of its
// sequence through the block table, so the result does not depend on how the sequence was cut into steps.
// Query / key sizes (D) and value size (Dv) are independent runtime values; scores, softmax and the output sum are float.
// Compiled WITHOUT fast-math.
#include <cuda_bf16.h>

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
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// first key a query at position p sees
__device__ __forceinline__ int first_key(int p, int window, int chunked) {
  if (chunked) return p - p % window;
  return p - window + 1 > 0 ? p - window + 1 : 0;
}
__device__ __forceinline__ float sigmoid_(float z) { return 1.f / (1.f + expf(-z)); }
// a scaled score with the optional terms: cap, then distance slope and distance bias (neither is scaled or capped)
__device__ __forceinline__ float score_terms(float sc, int dist, int h, int Hq, float slope, const NrlAttnMods& md) {
  if (md.softcap > 0.f) sc = md.softcap * tanhf(sc / md.softcap);
  sc -= slope * static_cast<float>(dist);
  if (md.dist_bias != nullptr) sc += md.dist_bias[static_cast<long>(dist < md.dist_max ? dist : md.dist_max) * Hq + h];
  return sc;
}

// warp per (token, key/value head): keys and (optionally blended) values into the pages
template <typename CT>
__global__ void kv_write_blend_kernel(const float* __restrict__ k, long sk, float* __restrict__ v, long sv, const float* __restrict__ v_other,
                                      long svo, const float* __restrict__ lambda, CT* __restrict__ k_cache, CT* __restrict__ v_cache,
                                      const int* __restrict__ kv_slot, long T, int Hkv, int D, int Dv, int page) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * Hkv) return;
  const long t = wid / Hkv;
  const int g = static_cast<int>(wid - t * Hkv);
  const int slot = kv_slot[t];
  const long pg = slot / page, off = slot % page;
  const float* kr = k + t * sk + static_cast<long>(g) * D;
  CT* kd = k_cache + ((pg * Hkv + g) * page + off) * D;
  for (int c = lane; c < D; c += 32) st(kd, c, kr[c]);
  float* vr = v + t * sv + static_cast<long>(g) * Dv;
  CT* vd = v_cache + ((pg * Hkv + g) * page + off) * Dv;
  if (v_other != nullptr) {
    const float lam = lambda[0];
    const float* vo = v_other + t * svo + static_cast<long>(g) * Dv;
    for (int c = lane; c < Dv; c += 32) {
      const float x = (1.f - lam) * vr[c] + lam * vo[c];
      vr[c] = x;
      st(vd, c, x);
    }
  } else {
    for (int c = lane; c < Dv; c += 32) st(vd, c, vr[c]);
  }
}

// warp per (token, head): heads 0..Hq-1 are queries (normalised in place), Hq..Hq+Hkv-1 keys (normalised into the cache),
// then Hkv value heads (copied into the cache)
template <typename CT>
__global__ void qknorm_kv_write_kernel(float* __restrict__ q, long sq, const float* __restrict__ k, long sk, const float* __restrict__ v,
                                       long sv, const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                       CT* __restrict__ k_cache, CT* __restrict__ v_cache, const int* __restrict__ kv_slot, long T,
                                       int Hq, int Hkv, int D, int Dv, int page) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int per = Hq + 2 * Hkv;
  if (wid >= T * per) return;
  const long t = wid / per;
  const int hh = static_cast<int>(wid - t * per);
  const int slot = kv_slot[t];
  const long pg = slot / page, off = slot % page;
  if (hh < Hq) {
    float* x = q + t * sq + static_cast<long>(hh) * D;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) ss += x[c] * x[c];
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    for (int c = lane; c < D; c += 32) x[c] = x[c] * r * qw[c];
  } else if (hh < Hq + Hkv) {
    const int g = hh - Hq;
    const float* x = k + t * sk + static_cast<long>(g) * D;
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) ss += x[c] * x[c];
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    CT* dst = k_cache + ((pg * Hkv + g) * page + off) * D;
    for (int c = lane; c < D; c += 32) st(dst, c, x[c] * r * kw[c]);
  } else {
    const int g = hh - Hq - Hkv;
    const float* x = v + t * sv + static_cast<long>(g) * Dv;
    CT* dst = v_cache + ((pg * Hkv + g) * page + off) * Dv;
    for (int c = lane; c < Dv; c += 32) st(dst, c, x[c]);
  }
}

// Latent attention, one launch per step: warp per (token, vector).  Vector 0 is the token's cache row
//   [ latent / rms(latent) * w  |  rotated shared key part ]   (rank + dr columns of the single key/value "head"),
// vectors 1..H are the heads' rotated query parts, written behind the absorbed unrotated part of the same head in
// qa (head h of token t at qa + t * sqa + h * sha, rank + dr columns).  Only the first `rdims` of the dr columns turn; (cos, sin) come from the angle p * freq[i] formed and
// reduced to [-pi, pi] in double, times `mult`.  interleaved: pairs (2i, 2i + 1); else (i, i + rdims / 2).
template <typename CT>
__global__ void latent_kv_write_kernel(const float* __restrict__ q, long sq, int H, int dn, int dr, const float* __restrict__ dkv, long sd,
                                       int rank, const float* __restrict__ w, float eps, const double* __restrict__ freq, int rdims,
                                       float mult, int interleaved, const int* __restrict__ pos, const int* __restrict__ kv_slot,
                                       CT* __restrict__ cache, int page, float* __restrict__ qa, long sqa, long sha,
                                       __nv_bfloat16* __restrict__ qn, long T) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * (H + 1)) return;
  const long t = wid / (H + 1);
  const int vec = static_cast<int>(wid - t * (H + 1));
  const int D = rank + dr;
  const double p = static_cast<double>(pos[t]);
  const float* src = vec == 0 ? dkv + t * sd + rank : q + t * sq + static_cast<long>(vec - 1) * (dn + dr) + dn;
  CT* crow = nullptr;
  if (vec == 0) {
    const int slot = kv_slot[t];
    crow = cache + static_cast<long>(slot) * D;               // one head: cell = page index * page + offset = slot
    const float* x = dkv + t * sd;
    float ss = 0.f;
    for (int c = lane; c < rank; c += 32) ss += x[c] * x[c];
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / static_cast<float>(rank) + eps);
    for (int c = lane; c < rank; c += 32) st(crow, c, x[c] * r * w[c]);
  }
  float* qrow = vec == 0 ? nullptr : qa + t * sqa + static_cast<long>(vec - 1) * sha + rank;
  if (vec > 0 && qn != nullptr) {                              // the head's unrotated columns as a bf16 GEMM operand [H, T, dn]
    const float* qs = q + t * sq + static_cast<long>(vec - 1) * (dn + dr);
    __nv_bfloat16* qd = qn + (static_cast<long>(vec - 1) * T + t) * dn;
    for (int c = lane; c < dn; c += 32) qd[c] = __float2bfloat16_rn(qs[c]);
  }
  const int half = rdims / 2;
  for (int i = lane; i < half; i += 32) {
    double a = p * freq[i];
    a -= 6.283185307179586476925 * rint(a * 0.15915494309189533577);
    float sn, cs;
    sincosf(static_cast<float>(a), &sn, &cs);
    sn *= mult;
    cs *= mult;
    const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
    const float u = src[iu], v = src[iv];
    const float ru = u * cs - v * sn, rv = v * cs + u * sn;
    if (vec == 0) {
      st(crow, rank + iu, ru);
      st(crow, rank + iv, rv);
    } else {
      qrow[iu] = ru;
      qrow[iv] = rv;
    }
  }
  for (int c = rdims + lane; c < dr; c += 32) {                // columns past the rotated ones pass unchanged
    if (vec == 0) st(crow, rank + c, src[c]);
    else qrow[c] = src[c];
  }
}

constexpr int kWarps = 4;
constexpr int kMaxDvPerLane = 16;      // Dv <= 512

// block per (token, query head); the window's keys are dealt to the warps in runs of 32 (one key per lane)
template <typename CT, typename OT>
__global__ void window_attention_kernel(const float* __restrict__ q, long sq, const CT* __restrict__ k_cache,
                                        const CT* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                                        const int* __restrict__ tok_entry, const int* __restrict__ pos, int window, float scale,
                                        float out_scale, OT* __restrict__ out, long so, int Hq, int Hkv, int D, int Dv, int page,
                                        NrlAttnMods md) {
  extern __shared__ float sm[];
  float* sq_ = sm;                               // [D]
  float* accs = sq_ + D;                         // [kWarps][Dv]
  float* ml = accs + kWarps * Dv;                // [kWarps][2]
  const long t = blockIdx.x;
  const int h = blockIdx.y, g = h / (Hq / Hkv);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int p = pos[t];
  const int* bt = block_table + static_cast<long>(tok_entry[t]) * max_blocks;
  for (int c = threadIdx.x; c < D; c += blockDim.x) sq_[c] = q[t * sq + static_cast<long>(h) * (md.q_head_stride ? md.q_head_stride : D) + c];
  __syncthreads();
  const int lo = first_key(p, window, md.chunked);
  const int kf = (!md.chunked && md.keep_first > 0) ? min(md.keep_first, lo) : 0;    // kept first keys in front of the window
  const int nkeys = kf + p - lo + 1;
  const int Hv = md.v_div > 1 ? Hkv / md.v_div : Hkv, gv = md.v_div > 1 ? g / md.v_div : g;
  if (md.head_scale != nullptr) scale *= md.head_scale[h];
  const float slope = md.head_slope != nullptr ? md.head_slope[h] : 0.f;
  if (md.gate != nullptr) out_scale *= sigmoid_(md.gate[t * md.gate_stride + h]);
  float m = -INFINITY, l = 0.f;
  float acc[kMaxDvPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDvPerLane; ++i) acc[i] = 0.f;
  for (int base = w * 32; base < nkeys; base += kWarps * 32) {
    const int vi = base + lane;
    const int j = vi < kf ? vi : lo + vi - kf;
    const bool ok = vi < nkeys;
    float sc = -INFINITY;
    long vrow = 0;
    if (ok) {
      const long pg = bt[j / page];
      const long cell = (pg * Hkv + g) * page + (j % page);
      const CT* kr = k_cache + cell * D;
      float d = 0.f;
      for (int c = 0; c < D; ++c) d += sq_[c] * ld(kr, c);
      sc = score_terms(d * scale, p - j, h, Hq, slope, md);
      vrow = md.kv_shared ? cell * D : ((pg * Hv + gv) * page + (j % page)) * Dv;
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float corr = expf(m - mn);               // m = -inf on the first run: exp(-inf) = 0
    const float pr = ok ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(pr);
#pragma unroll
    for (int i = 0; i < kMaxDvPerLane; ++i) acc[i] *= corr;
    const int cnt = nkeys - base < 32 ? nkeys - base : 32;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pr, jj);
      const long vr = __shfl_sync(0xffffffffu, vrow, jj);
#pragma unroll
      for (int i = 0; i < kMaxDvPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < Dv) acc[i] += pj * ld(v_cache, vr + c);
      }
    }
    m = mn;
  }
#pragma unroll
  for (int i = 0; i < kMaxDvPerLane; ++i) {
    const int c = lane + 32 * i;
    if (c < Dv) accs[w * Dv + c] = acc[i];
  }
  if (lane == 0) {
    ml[2 * w] = m;
    ml[2 * w + 1] = l;
  }
  __syncthreads();
  float mt = md.head_sink != nullptr ? md.head_sink[h] : -INFINITY;       // the sink: a score with no key and no value
  for (int i = 0; i < kWarps; ++i) mt = fmaxf(mt, ml[2 * i]);
  float lt = md.head_sink != nullptr ? expf(md.head_sink[h] - mt) : 0.f, f[kWarps];
  for (int i = 0; i < kWarps; ++i) {
    f[i] = ml[2 * i] == -INFINITY ? 0.f : expf(ml[2 * i] - mt);
    lt += f[i] * ml[2 * i + 1];
  }
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float a = 0.f;
    for (int i = 0; i < kWarps; ++i) a += f[i] * accs[i * Dv + c];
    const float val = out_scale * (a / lt);
    if (md.out_float != nullptr) md.out_float[t * md.out_float_stride + static_cast<long>(h) * Dv + c] = val;
    else st(out, t * so + static_cast<long>(h) * Dv + c, val);
  }
}


// ---------------------------------------------------------------------------------------------------------------------
// Tiled kernel: a block owns up to NQ queries that share their keys -- QT consecutive tokens x HB query heads of one
// key/value head -- so a key row is fetched once for all of them.  Lane = key for the scores (each lane keeps NQ running
// dot products against the queries in shared memory), lane = value columns for the output sum (softmax weights go
// through shared memory).  Tokens of different sequences that fall into one tile are handled one run after the other.
// ---------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void load8(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* o) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load4(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* o) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}

template <typename CT, typename OT, int NQ, int NVC>       // NVC: chunks of 128 value columns (Dv <= 128 NVC)
__global__ void __launch_bounds__(kWarps * 32)
window_attention_tile_kernel(const float* __restrict__ q, long sq, const CT* __restrict__ k_cache, const CT* __restrict__ v_cache,
                             const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_entry,
                             const int* __restrict__ pos, int window, float scale, float out_scale, OT* __restrict__ out, long so,
                             int T, int Hq, int Hkv, int D, int Dv, int page, int HB, int QT, NrlAttnMods md) {
  extern __shared__ float sm[];
  float* qs = sm;                                  // [NQ][D], scaled
  float* ps = qs + NQ * D;                         // [kWarps][32][NQ]
  float* racc = ps + kWarps * 32 * NQ;             // [kWarps][NQ][Dv]
  float* rml = racc + kWarps * NQ * Dv;            // [kWarps][NQ][2]
  const int g = blockIdx.y, per_g = Hq / Hkv;
  const int h0 = g * per_g + blockIdx.z * HB;
  const int hb = min(HB, per_g - static_cast<int>(blockIdx.z) * HB);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int t_begin = blockIdx.x * QT, t_end = min(T, t_begin + QT);
  const bool vec8 = (D % 8) == 0;
  float* myp = ps + w * 32 * NQ;
  int t = t_begin;
  while (t < t_end) {
    const int e = tok_entry[t];
    int tn = t + 1;
    while (tn < t_end && tok_entry[tn] == e) ++tn;
    const int nt = tn - t, nqs = nt * hb;
    const int p_first = pos[t];
    const int lo = first_key(p_first, window, md.chunked);       // the first key of a run's first token: later tokens start no earlier
    const int keep = md.chunked ? 0 : md.keep_first;
    const int kf = keep > 0 ? min(keep, lo) : 0;                 // kept first keys in front of the run's window
    const int nkeys = kf + p_first + nt - lo;
    const int* bt = block_table + static_cast<long>(e) * max_blocks;
    __syncthreads();
    for (int idx = threadIdx.x; idx < NQ * D; idx += blockDim.x) {
      const int qi = idx / D, c = idx - qi * D;
      float v = 0.f;
      if (qi < nqs) {
        const int hq = h0 + qi % hb;
        v = q[static_cast<long>(t + qi / hb) * sq + static_cast<long>(hq) * (md.q_head_stride ? md.q_head_stride : D) + c] * scale;
        if (md.head_scale != nullptr) v *= md.head_scale[hq];
      }
      qs[idx] = v;
    }
    __syncthreads();
    float m[NQ], l[NQ], acc[NQ][4 * NVC], slope[NQ];
    const long vstride = md.kv_shared ? D : Dv;
    const int Hv = md.v_div > 1 ? Hkv / md.v_div : Hkv, gv = md.v_div > 1 ? g / md.v_div : g;
    const bool terms = md.softcap > 0.f || md.dist_bias != nullptr;
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
      slope[i] = (md.head_slope != nullptr && i < nqs) ? md.head_slope[h0 + i % hb] : 0.f;
      m[i] = -INFINITY;
      l[i] = 0.f;
#pragma unroll
      for (int x = 0; x < 4 * NVC; ++x) acc[i][x] = 0.f;
    }
    for (int base = w * 32; base < nkeys; base += kWarps * 32) {
      const int vi = base + lane;
      const int j = vi < kf ? vi : lo + vi - kf;
      const bool ok = vi < nkeys;
      float s[NQ];
#pragma unroll
      for (int i = 0; i < NQ; ++i) s[i] = 0.f;
      long cell = 0, vcell = 0;
      if (ok) {
        const long pgj = bt[j / page];
        cell = (pgj * Hkv + g) * page + (j % page);
        vcell = md.kv_shared ? cell : (pgj * Hv + gv) * page + (j % page);
        const CT* kr = k_cache + cell * D;
        if (vec8) {
          for (int c = 0; c < D; c += 8) {
            float kv[8];
            load8(kr + c, kv);
#pragma unroll
            for (int i = 0; i < NQ; ++i) {
              const float4 a = *reinterpret_cast<const float4*>(qs + i * D + c), b = *reinterpret_cast<const float4*>(qs + i * D + c + 4);
              s[i] += a.x * kv[0] + a.y * kv[1] + a.z * kv[2] + a.w * kv[3] + b.x * kv[4] + b.y * kv[5] + b.z * kv[6] + b.w * kv[7];
            }
          }
        } else {
          for (int c = 0; c < D; ++c) {
            const float kv = ld(kr, c);
#pragma unroll
            for (int i = 0; i < NQ; ++i) s[i] += qs[i * D + c] * kv;
          }
        }
      }
#pragma unroll
      for (int i = 0; i < NQ; ++i) {
        const int pq = p_first + i / hb;                                   // position of query i
        const bool valid = ok && i < nqs && j <= pq && (j >= first_key(pq, window, md.chunked) || j < keep);
        float sc = -INFINITY;
        if (valid) sc = terms ? score_terms(s[i], pq - j, h0 + i % hb, Hq, slope[i], md) : s[i] - slope[i] * static_cast<float>(pq - j);
        const float mn = fmaxf(m[i], warp_max(sc));
        float pr = 0.f;
        if (mn != -INFINITY) {                                              // some key of this query has been seen
          const float corr = expf(m[i] - mn);
          pr = valid ? expf(sc - mn) : 0.f;
          l[i] = l[i] * corr + warp_sum(pr);
#pragma unroll
          for (int x = 0; x < 4 * NVC; ++x) acc[i][x] *= corr;
          m[i] = mn;
        }
        myp[lane * NQ + i] = pr;
      }
      __syncwarp();
      const int cnt = nkeys - base < 32 ? nkeys - base : 32;
      for (int jj = 0; jj < cnt; ++jj) {
        const long vr = __shfl_sync(0xffffffffu, vcell, jj) * vstride;
#pragma unroll
        for (int x = 0; x < NVC; ++x) {
          const int c0 = lane * 4 + 128 * x;
          float vv[4] = {0.f, 0.f, 0.f, 0.f};
          if (c0 < Dv) load4(v_cache + vr + c0, vv);
#pragma unroll
          for (int i = 0; i < NQ; ++i) {
            const float pj = myp[jj * NQ + i];
            acc[i][4 * x] += pj * vv[0]; acc[i][4 * x + 1] += pj * vv[1]; acc[i][4 * x + 2] += pj * vv[2]; acc[i][4 * x + 3] += pj * vv[3];
          }
        }
      }
      __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < NQ; ++i) {
#pragma unroll
      for (int x = 0; x < NVC; ++x) {
        const int c0 = lane * 4 + 128 * x;
        if (c0 < Dv) {
          float* d = racc + (static_cast<long>(w) * NQ + i) * Dv + c0;
          d[0] = acc[i][4 * x]; d[1] = acc[i][4 * x + 1]; d[2] = acc[i][4 * x + 2]; d[3] = acc[i][4 * x + 3];
        }
      }
      if (lane == 0) {
        rml[(w * NQ + i) * 2] = m[i];
        rml[(w * NQ + i) * 2 + 1] = l[i];
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nqs * Dv; idx += blockDim.x) {
      const int qi = idx / Dv, c = idx - qi * Dv;
      const float sink = md.head_sink != nullptr ? md.head_sink[h0 + qi % hb] : -INFINITY;    // a score with no key and no value
      float mt = sink;
      for (int x = 0; x < kWarps; ++x) mt = fmaxf(mt, rml[(x * NQ + qi) * 2]);
      float lt = md.head_sink != nullptr ? expf(sink - mt) : 0.f, a = 0.f;
      for (int x = 0; x < kWarps; ++x) {
        const float mx = rml[(x * NQ + qi) * 2];
        const float f = mx == -INFINITY ? 0.f : expf(mx - mt);
        lt += f * rml[(x * NQ + qi) * 2 + 1];
        a += f * racc[(static_cast<long>(x) * NQ + qi) * Dv + c];
      }
      float os = out_scale;
      if (md.gate != nullptr) os *= sigmoid_(md.gate[static_cast<long>(t + qi / hb) * md.gate_stride + h0 + qi % hb]);
      const long orow = t + qi / hb, ocol = static_cast<long>(h0 + qi % hb) * Dv + c;
      if (md.out_float != nullptr) md.out_float[orow * md.out_float_stride + ocol] = os * (a / lt);
      else st(out, orow * so + ocol, os * (a / lt));
    }
    t = tn;
  }
}

template <typename CT, typename OT, int NQ, int NVC>
cudaError_t launch_tile(const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
                        const int* tok_entry, const int* pos, int window, float scale, float out_scale, void* out, long so, int T,
                        int Hq, int Hkv, int D, int Dv, int page, const NrlAttnMods& md, cudaStream_t s) {
  const int per_g = Hq / Hkv;
  const int HB = per_g < NQ ? per_g : NQ, QT = NQ / HB > 1 ? NQ / HB : 1;
  const size_t smem = sizeof(float) * (static_cast<size_t>(NQ) * D + kWarps * 32 * NQ + static_cast<size_t>(kWarps) * NQ * Dv + kWarps * NQ * 2);
  if (smem > 160 * 1024) return cudaErrorInvalidValue;
  auto kern = window_attention_tile_kernel<CT, OT, NQ, NVC>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const dim3 grid((T + QT - 1) / QT, Hkv, (per_g + HB - 1) / HB);
  kern<<<grid, kWarps * 32, smem, s>>>(q, sq, static_cast<const CT*>(k_cache), static_cast<const CT*>(v_cache), block_table, max_blocks,
                                       tok_entry, pos, window, scale, out_scale, static_cast<OT*>(out), so, T, Hq, Hkv, D, Dv, page, HB, QT, md);
  return cudaGetLastError();
}

template <typename CT, typename OT>
cudaError_t launch_tile_nq(int nq, const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table,
                           int max_blocks, const int* tok_entry, const int* pos, int window, float scale, float out_scale, void* out,
                           long so, int T, int Hq, int Hkv, int D, int Dv, int page, const NrlAttnMods& md, cudaStream_t s) {
#define NRL_WA(NQ_, NVC_) return launch_tile<CT, OT, NQ_, NVC_>(q, sq, k_cache, v_cache, block_table, max_blocks, tok_entry, pos, window, \
                                                                 scale, out_scale, out, so, T, Hq, Hkv, D, Dv, page, md, s)
  if (Dv > 256) {                        // wider values: fewer queries per block, so that the sums still fit the registers
    if (nq <= 2) NRL_WA(2, 4);
    NRL_WA(4, 4);
  }
  if (Dv > 128) {
    if (nq <= 2) NRL_WA(2, 2);
    if (nq <= 4) NRL_WA(4, 2);
    NRL_WA(8, 2);
  }
  if (nq <= 2) NRL_WA(2, 1);
  if (nq <= 4) NRL_WA(4, 1);
  if (nq <= 8) NRL_WA(8, 1);
  NRL_WA(16, 1);
#undef NRL_WA
}

// ---------------------------------------------------------------------------------------------------------------------
// Write side of rotated attention, one launch per step: warp per (token, vector).  Vectors 0 .. Hq-1 are the query heads
// (float, finished in place), Hq .. Hq+Hk-1 the key heads (finished into their page), then Hv value heads (copied into their
// page; v == nullptr: the values are the keys as projected, bias included, before rotation and norm, written by the key's warp).
// A vector is staged in shared memory: + bias, the first `rdims` columns rotated by the angles pos * freq[i] (formed and reduced
// to [-pi, pi] in double; cos and sin times `mult`; interleaved pairs (2i, 2i + 1), else (i, i + rdims / 2)), then, with
// unit_norm, divided by its root mean square (eps inside the root; times norm_w [D] when given).  k == nullptr: queries only
// (a layer that reads another layer's pages).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kRotWarps = 4;

template <typename CT>
__global__ void rot_kv_write_kernel(float* __restrict__ q, long sq, const float* __restrict__ q_bias, const float* __restrict__ k, long sk,
                                    const float* __restrict__ k_bias, const float* __restrict__ v, long sv, const double* __restrict__ freq,
                                    int rdims, float mult, int interleaved, int unit_norm, const float* __restrict__ q_norm_w,
                                    const float* __restrict__ k_norm_w, float eps, const int* __restrict__ pos,
                                    const int* __restrict__ kv_slot, CT* __restrict__ k_cache, CT* __restrict__ v_cache, int page, long T,
                                    int Hq, int Hk, int Hv, int D, int Dv) {
  extern __shared__ float rot_stage[];                      // [kRotWarps][D]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const long wid = blockIdx.x * static_cast<long>(kRotWarps) + w;
  const int nk = k != nullptr ? Hk : 0, nv = (k != nullptr && v != nullptr) ? Hv : 0;
  const int per = Hq + nk + nv;
  if (wid >= T * per) return;
  const long t = wid / per;
  const int vec = static_cast<int>(wid - t * per);
  const int slot = k != nullptr ? kv_slot[t] : 0;
  const long pg = slot / page, off = slot % page;
  if (vec >= Hq + nk) {                                      // a value head: plain copy
    const int g = vec - Hq - nk;
    const float* x = v + t * sv + static_cast<long>(g) * Dv;
    CT* dst = v_cache + ((pg * Hv + g) * page + off) * Dv;
    for (int c = lane; c < Dv; c += 32) st(dst, c, x[c]);
    return;
  }
  const bool is_q = vec < Hq;
  const int hd = is_q ? vec : vec - Hq;
  const float* src = is_q ? q + t * sq + static_cast<long>(hd) * D : k + t * sk + static_cast<long>(hd) * D;
  const float* bias = is_q ? q_bias : k_bias;
  float* x = rot_stage + w * D;
  for (int c = lane; c < D; c += 32) x[c] = src[c] + (bias != nullptr ? bias[static_cast<long>(hd) * D + c] : 0.f);
  __syncwarp();
  if (!is_q && v == nullptr) {                               // the values are the keys as projected
    CT* dst = v_cache + ((pg * Hk + hd) * page + off) * D;
    for (int c = lane; c < D; c += 32) st(dst, c, x[c]);
  }
  const double p = static_cast<double>(pos[t]);
  const int half = rdims / 2;
  for (int i = lane; i < half; i += 32) {
    double a = p * freq[i];
    a -= 6.283185307179586476925 * rint(a * 0.15915494309189533577);
    float sn, cs;
    sincosf(static_cast<float>(a), &sn, &cs);
    sn *= mult;
    cs *= mult;
    const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
    const float u = x[iu], vv = x[iv];
    x[iu] = u * cs - vv * sn;
    x[iv] = vv * cs + u * sn;
  }
  __syncwarp();
  float r = 1.f;
  const float* nw = nullptr;
  if (unit_norm) {
    float ss = 0.f;
    for (int c = lane; c < D; c += 32) ss += x[c] * x[c];
    ss = warp_sum(ss);
    r = 1.f / sqrtf(ss / static_cast<float>(D) + eps);
    nw = is_q ? q_norm_w : k_norm_w;
  }
  if (is_q) {
    float* dst = q + t * sq + static_cast<long>(hd) * D;
    for (int c = lane; c < D; c += 32) dst[c] = x[c] * r * (nw != nullptr ? nw[c] : 1.f);
  } else {
    CT* dst = k_cache + ((pg * Hk + hd) * page + off) * D;
    for (int c = lane; c < D; c += 32) st(dst, c, x[c] * r * (nw != nullptr ? nw[c] : 1.f));
  }
}

// Differential attention, read side: a [T, maps * H, Dv] (typed) holds the outputs of two score maps over the same values, the heads
// ordered (key/value head g, map m, query head r of the group): o = a_1 - lambda a_2, divided by its root mean square over the
// head's Dv values (eps inside the root), times post, times sigmoid(gate[t, h * Dv + c]) (gate float or null), times out_scale.
// warp per (token, head); out typed [T, H * Dv] in the model's head order h = g * R + r.
template <typename AT, typename OT>
__global__ void diff_combine_kernel(const AT* __restrict__ a, long sa, float lambda, float post, float eps, const float* __restrict__ gate,
                                    long sg, float out_scale, OT* __restrict__ out, long so, long T, int H, int R, int Dv) {
  const long wid = (blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= T * H) return;
  const long t = wid / H;
  const int h = static_cast<int>(wid - t * H), g = h / R, r = h % R;
  const AT* a1 = a + t * sa + (static_cast<long>(2 * g) * R + r) * Dv;
  const AT* a2 = a + t * sa + (static_cast<long>(2 * g + 1) * R + r) * Dv;
  float ss = 0.f;
  for (int c = lane; c < Dv; c += 32) {
    const float o = ld(a1, c) - lambda * ld(a2, c);
    ss += o * o;
  }
  ss = warp_sum(ss);
  const float f = post * out_scale / sqrtf(ss / static_cast<float>(Dv) + eps);
  for (int c = lane; c < Dv; c += 32) {
    const long col = static_cast<long>(h) * Dv + c;
    float o = (ld(a1, c) - lambda * ld(a2, c)) * f;
    if (gate != nullptr) o *= sigmoid_(gate[t * sg + col]);
    st(out, t * so + col, o);
  }
}

}  // namespace

extern "C" {

cudaError_t nrl_qknorm_kv_write(float* q, long sq, const float* k, long sk, const float* v, long sv, const float* qw, const float* kw,
                                float eps, void* k_cache, void* v_cache, int cache_f32, const int* kv_slot, int T, int Hq, int Hkv,
                                int D, int Dv, int page, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  const long warps = static_cast<long>(T) * (Hq + 2 * Hkv);
  const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
  if (cache_f32)
    qknorm_kv_write_kernel<float><<<blocks, 128, 0, s>>>(q, sq, k, sk, v, sv, qw, kw, eps, static_cast<float*>(k_cache),
                                                         static_cast<float*>(v_cache), kv_slot, T, Hq, Hkv, D, Dv, page);
  else
    qknorm_kv_write_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(q, sq, k, sk, v, sv, qw, kw, eps,
                                                                 static_cast<__nv_bfloat16*>(k_cache),
                                                                 static_cast<__nv_bfloat16*>(v_cache), kv_slot, T, Hq, Hkv, D, Dv, page);
  return cudaGetLastError();
}

cudaError_t nrl_kv_write_blend(const float* k, long sk, float* v, long sv, const float* v_other, long svo, const float* lambda,
                               void* k_cache, void* v_cache, int cache_f32, const int* kv_slot, int T, int Hkv, int D, int Dv, int page,
                               cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (v_other != nullptr && lambda == nullptr) return cudaErrorInvalidValue;
  const long warps = static_cast<long>(T) * Hkv;
  const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
  if (cache_f32)
    kv_write_blend_kernel<float><<<blocks, 128, 0, s>>>(k, sk, v, sv, v_other, svo, lambda, static_cast<float*>(k_cache),
                                                        static_cast<float*>(v_cache), kv_slot, T, Hkv, D, Dv, page);
  else
    kv_write_blend_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(k, sk, v, sv, v_other, svo, lambda, static_cast<__nv_bfloat16*>(k_cache),
                                                                static_cast<__nv_bfloat16*>(v_cache), kv_slot, T, Hkv, D, Dv, page);
  return cudaGetLastError();
}

cudaError_t nrl_latent_kv_write(const float* q, long sq, int H, int dn, int dr, const float* dkv, long sd, int rank, const float* w,
                                float eps, const double* freq, int rdims, float mult, int interleaved, const int* pos, const int* kv_slot,
                                void* cache, int cache_f32, int page, float* qa, long sqa, long sha, void* qn, int T, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (rdims < 0 || rdims > dr || rdims % 2 != 0 || rank < 1 || H < 1) return cudaErrorInvalidValue;
  const long warps = static_cast<long>(T) * (H + 1);
  const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
  if (cache_f32)
    latent_kv_write_kernel<float><<<blocks, 128, 0, s>>>(q, sq, H, dn, dr, dkv, sd, rank, w, eps, freq, rdims, mult, interleaved, pos,
                                                         kv_slot, static_cast<float*>(cache), page, qa, sqa, sha, static_cast<__nv_bfloat16*>(qn), T);
  else
    latent_kv_write_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(q, sq, H, dn, dr, dkv, sd, rank, w, eps, freq, rdims, mult, interleaved,
                                                                 pos, kv_slot, static_cast<__nv_bfloat16*>(cache), page, qa, sqa, sha,
                                                                 static_cast<__nv_bfloat16*>(qn), T);
  return cudaGetLastError();
}

cudaError_t nrl_window_attention(const float* q, long sq, const void* k_cache, const void* v_cache, int cache_f32,
                                 const int* block_table, int max_blocks, const int* tok_entry, const int* pos, int window,
                                 float scale, float out_scale, void* out, long so, int out_f32, int T, int Hq, int Hkv, int D, int Dv,
                                 int page, int single_token, int impl, int nsplit, float* part, const NrlAttnMods* mods, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (Hq % Hkv != 0 || window < 1 || cache_f32 != out_f32) return cudaErrorInvalidValue;
  NrlAttnMods md = {0, nullptr, nullptr, nullptr, 0};
  if (mods != nullptr) md = *mods;
  if (md.kv_shared && (Dv > D || v_cache != k_cache)) return cudaErrorInvalidValue;
  if (md.v_div > 1 && (Hkv % md.v_div != 0 || md.kv_shared)) return cudaErrorInvalidValue;
  if (md.dist_bias != nullptr && md.dist_max < 0) return cudaErrorInvalidValue;
  // latent attention (one shared row per token is key and value of every head, causal) over bf16 pages: its own tensor-core kernels
  if ((impl == 0 || impl == 3) && !cache_f32 && md.kv_shared && Hkv == 1 && window >= (1 << 30) && !md.chunked &&
      md.head_scale == nullptr && md.head_slope == nullptr && nrl_latent_attention_mma_fits(out, so, D, Dv, page))
    return nrl_latent_attention_mma(q, sq, k_cache, block_table, max_blocks, tok_entry, pos, scale, out_scale, out, so, T, Hq, D, Dv, page,
                                    single_token, nsplit, part, &md, s);
  // prompt portions over bf16 pages: tensor cores
  if ((impl == 0 || impl == 3) && !cache_f32 && nrl_window_attention_mma_fits(out, so, Hq, Hkv, D, Dv, page) && !md.kv_shared) {
    if (single_token && nsplit >= 1 && part != nullptr)
      return nrl_window_attention_decode(q, sq, k_cache, v_cache, block_table, max_blocks, tok_entry, pos, window, scale, out_scale, out,
                                         so, T, Hq, Hkv, D, Dv, page, nsplit, part, &md, s);
    return nrl_window_attention_mma(q, sq, k_cache, v_cache, block_table, max_blocks, tok_entry, pos, window, scale, out_scale, out, so,
                                    T, Hq, Hkv, D, Dv, page, single_token, &md, s);
  }
  if (impl == 3) return cudaErrorInvalidValue;
  if (impl != 2 && Dv <= 512 && Dv % 4 == 0 && D <= 1024 && (!md.kv_shared || D % 4 == 0)) {
    // queries per block: the heads of one key/value head for single-token steps, 16 (tokens x heads) when entries hold runs
    const int nq = single_token ? Hq / Hkv : 16;
    return cache_f32 ? launch_tile_nq<float, float>(nq, q, sq, k_cache, v_cache, block_table, max_blocks, tok_entry, pos, window, scale,
                                                    out_scale, out, so, T, Hq, Hkv, D, Dv, page, md, s)
                     : launch_tile_nq<__nv_bfloat16, __nv_bfloat16>(nq, q, sq, k_cache, v_cache, block_table, max_blocks, tok_entry, pos,
                                                                    window, scale, out_scale, out, so, T, Hq, Hkv, D, Dv, page, md, s);
  }
  const size_t smem = sizeof(float) * (D + kWarps * Dv + 2 * kWarps);
  if (smem > 48 * 1024 || Dv > 32 * kMaxDvPerLane) return cudaErrorInvalidValue;
  const dim3 grid(T, Hq);
  if (cache_f32)
    window_attention_kernel<float, float><<<grid, kWarps * 32, smem, s>>>(
        q, sq, static_cast<const float*>(k_cache), static_cast<const float*>(v_cache), block_table, max_blocks, tok_entry, pos, window,
        scale, out_scale, static_cast<float*>(out), so, Hq, Hkv, D, Dv, page, md);
  else
    window_attention_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, kWarps * 32, smem, s>>>(
        q, sq, static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache), block_table, max_blocks,
        tok_entry, pos, window, scale, out_scale, static_cast<__nv_bfloat16*>(out), so, Hq, Hkv, D, Dv, page, md);
  return cudaGetLastError();
}

cudaError_t nrl_rot_kv_write(float* q, long sq, const float* q_bias, const float* k, long sk, const float* k_bias, const float* v, long sv,
                             const double* freq, int rdims, float mult, int interleaved, int unit_norm, const float* q_norm_w,
                             const float* k_norm_w, float eps, const int* pos, const int* kv_slot, void* k_cache, void* v_cache,
                             int cache_f32, int page, int T, int Hq, int Hk, int Hv, int D, int Dv, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (rdims < 0 || rdims > D || rdims % 2 != 0 || (rdims > 0 && freq == nullptr) || D < 1 || D > 2048) return cudaErrorInvalidValue;
  if (k != nullptr && v == nullptr && (Hv != Hk || Dv != D)) return cudaErrorInvalidValue;
  const int per = Hq + (k != nullptr ? Hk + (v != nullptr ? Hv : 0) : 0);
  const long warps = static_cast<long>(T) * per;
  const unsigned blocks = static_cast<unsigned>((warps + kRotWarps - 1) / kRotWarps);
  const size_t smem = sizeof(float) * kRotWarps * D;
  if (cache_f32)
    rot_kv_write_kernel<float><<<blocks, kRotWarps * 32, smem, s>>>(q, sq, q_bias, k, sk, k_bias, v, sv, freq, rdims, mult, interleaved,
                                                                    unit_norm, q_norm_w, k_norm_w, eps, pos, kv_slot,
                                                                    static_cast<float*>(k_cache), static_cast<float*>(v_cache), page, T, Hq,
                                                                    Hk, Hv, D, Dv);
  else
    rot_kv_write_kernel<__nv_bfloat16><<<blocks, kRotWarps * 32, smem, s>>>(q, sq, q_bias, k, sk, k_bias, v, sv, freq, rdims, mult,
                                                                            interleaved, unit_norm, q_norm_w, k_norm_w, eps, pos, kv_slot,
                                                                            static_cast<__nv_bfloat16*>(k_cache),
                                                                            static_cast<__nv_bfloat16*>(v_cache), page, T, Hq, Hk, Hv, D, Dv);
  return cudaGetLastError();
}

cudaError_t nrl_diff_combine(const void* a, long sa, int a_f32, float lambda, float post, float eps, const float* gate, long sg,
                             float out_scale, void* out, long so, int out_f32, int T, int H, int Hkv, int Dv, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (Hkv < 1 || H % Hkv != 0) return cudaErrorInvalidValue;
  const long warps = static_cast<long>(T) * H;
  const unsigned blocks = static_cast<unsigned>((warps + 3) / 4);
  const int R = H / Hkv;
#define NRL_DC(AT_, OT_)                                                                                                           \
  diff_combine_kernel<AT_, OT_><<<blocks, 128, 0, s>>>(static_cast<const AT_*>(a), sa, lambda, post, eps, gate, sg, out_scale,       \
                                                       static_cast<OT_*>(out), so, T, H, R, Dv)
  if (a_f32 && out_f32) NRL_DC(float, float);
  else if (a_f32) NRL_DC(float, __nv_bfloat16);
  else if (out_f32) NRL_DC(__nv_bfloat16, float);
  else NRL_DC(__nv_bfloat16, __nv_bfloat16);
#undef NRL_DC
  return cudaGetLastError();
}

}  // extern "C"
