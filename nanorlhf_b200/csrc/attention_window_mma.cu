// Sliding-window (or chunked) attention on the tensor cores, reading the 16-token bf16 pages in place.  The optional terms of
// NrlAttnMods (chunk mask, per-head score multiplier and distance slope, per-head output gate, capped scores, a bias per distance,
// first keys that stay visible behind the window, a sink in the denominator, several key heads over one value head) are applied
// in float.
//
// Prompt portions (window_attention_mma_kernel): a block owns 64 query rows that share one key/value head -- QT
// consecutive tokens x HB query heads -- as four warps of 16 rows, and walks the keys its rows can see in blocks of 64
// (four pages), double buffered through shared memory with cp.async.  Per block: S = Q K^T (bf16 operands, float
// accumulators); scores scaled and masked in float (key j is seen by the query at position p when p - window < j <= p;
// blocks that no window edge crosses skip the mask); online softmax in float, base 2 with ex2.approx; P is rounded to bf16
// only as the operand of O += P V (float accumulators).  Tokens of different sequences that fall into one tile are handled
// one run after the other over the same accumulators (a row belongs to one run only).
// Steps of single tokens (window_attention_decode_kernel): every warp walks its own pages; see there.
// Query / key size D and value size Dv are runtime values (multiples of 8 up to 128); the templates fix the padded sizes
// (32, 64 or 128), the padding is zero-filled in shared memory.  Compiled WITHOUT fast-math.
#include <cuda_bf16.h>

#include <cstdint>

#include "hybrid_kernels.h"

namespace {

constexpr int kBM = 64;        // query rows per block
constexpr int kBN = 64;        // keys per block of the walk
constexpr int kThreads = 128;
constexpr int kPad = 8;        // bf16 elements appended to a shared-memory row (ldmatrix without bank conflicts)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }

// 2^x on the special-function unit (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// cap * tanh(x / cap) through 2^x on the special-function unit: tanh(z) = (1 - e) / (1 + e), e = exp(-2 |z|) (relative error of a
// few 2^-22: far below the bf16 rounding of the weights that follow)
__device__ __forceinline__ float softcap_(float x, float cap, float inv_cap) {
  const float e = ex2(-2.885390081777927f * fabsf(x * inv_cap));
  return copysignf(cap * __fdividef(1.f - e, 1.f + e), x);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// first key a query at position p sees (window form: not clamped at 0, callers compare or clamp)
__device__ __forceinline__ int first_key(int p, int window, int chunked) { return chunked ? p - p % window : p - window + 1; }
__device__ __forceinline__ float sigmoid_(float z) { return 1.f / (1.f + expf(-z)); }

__device__ __forceinline__ int sel4(const int (&v)[4], int i) { return i == 0 ? v[0] : i == 1 ? v[1] : i == 2 ? v[2] : v[3]; }

// the four pages that hold keys kb .. kb + 63 of a sequence (0 where the sequence ends before)
__device__ __forceinline__ void block_pages(const int* bt, int kb, int hi, int (&pg)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) pg[i] = kb + 16 * i <= hi ? bt[(kb >> 4) + i] : 0;
}

// one 64-key block of K or V into shared memory: rows = keys kb .. kb + 63 of the sequence, `width` real columns of WP
// (WP / 8 is a power of two: the index arithmetic is shifts)
template <int WP>
__device__ __forceinline__ void load_kv_block(__nv_bfloat16* dst, const __nv_bfloat16* cache, const int (&pg)[4], int Hkv, int g, int kb,
                                              int hi, int width) {
  constexpr int chunks = WP / 8, ld = WP + kPad;
#pragma unroll
  for (int idx = threadIdx.x; idx < kBN * chunks; idx += kThreads) {
    const int key = idx / chunks, ch = idx % chunks;
    __nv_bfloat16* d = dst + key * ld + ch * 8;
    if (kb + key <= hi && ch * 8 < width) {
      const long cell = (static_cast<long>(sel4(pg, key >> 4)) * Hkv + g) * 16 + (key & 15);
      cp_async16(smem_u32(d), cache + cell * width + ch * 8);
    } else {
      *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

template <int KS, int NV>      // padded D = 16 KS, padded Dv = 16 NV
__global__ void __launch_bounds__(kThreads, 3)
window_attention_mma_kernel(const float* __restrict__ q, long sq, const __nv_bfloat16* __restrict__ k_cache,
                            const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                            const int* __restrict__ tok_entry, const int* __restrict__ pos, int window, float scale, float out_scale,
                            __nv_bfloat16* __restrict__ out, long so, int T, int Hq, int Hkv, int D, int Dv, int HB, int QT,
                            NrlAttnMods md) {
  constexpr int DP = 16 * KS, DVP = 16 * NV, LDK = DP + kPad, LDV = DVP + kPad;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [2][kBN][LDK]
  __nv_bfloat16* sV = sK + 2 * kBN * LDK;                                     // [2][kBN][LDV]
  __nv_bfloat16* sQ = sK + kBN * LDK;     // [kBM][LDK]: lives in K buffer 1, which is first filled after the queries left for registers
  const int zb = static_cast<int>(blockIdx.z);
  const int g = blockIdx.y, per_g = Hq / Hkv, h0 = g * per_g + zb * HB;
  const int hb = min(HB, per_g - zb * HB);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  const int t_begin = blockIdx.x * QT, t_end = min(T, t_begin + QT);

  // ---- queries: float -> bf16 into shared memory (zero rows / columns where there is no query), then A fragments ----
  for (int idx = threadIdx.x; idx < kBM * DP; idx += kThreads) {
    const int r = idx / DP, c = idx - r * DP;
    const int tt = t_begin + r / HB, hh = r % HB;
    float v = 0.f;
    if (r < QT * HB && tt < t_end && hh < hb && c < D) v = q[static_cast<long>(tt) * sq + static_cast<long>(h0 + hh) * D + c];
    sQ[r * LDK + c] = __float2bfloat16_rn(v);
  }
  __syncthreads();
  uint32_t qf[KS][4];
  {
    const int m = lane >> 3, rr = w * 16 + (m & 1) * 8 + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldsm_x4(smem_u32(sQ + rr * LDK + ks * 16 + (m >> 1) * 8), qf[ks]);
  }
  // the two rows of this thread: w*16 + gq and w*16 + gq + 8
  int row_t[2];
  bool row_ok[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int r = w * 16 + gq + hf * 8;
    row_t[hf] = t_begin + r / HB;
    row_ok[hf] = r < QT * HB && row_t[hf] < t_end && (r % HB) < hb;
  }
  // tokens that the rows of this warp cover (to skip key blocks none of them sees)
  const int wt_lo = t_begin + (w * 16) / HB, wt_hi = min(t_end - 1, t_begin + (w * 16 + 15) / HB);

  float o[2 * NV][4];
#pragma unroll
  for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // running maxima live in the log2 domain
  // per row (= per query head): score multiplier and distance slope, both in the log2 domain
  float sl2[2], slr[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int hq = min(h0 + (w * 16 + gq + hf * 8) % HB, Hq - 1);
    sl2[hf] = scale * 1.4426950408889634f * (md.head_scale != nullptr ? md.head_scale[hq] : 1.f);
    slr[hf] = md.head_slope != nullptr ? md.head_slope[hq] * 1.4426950408889634f : 0.f;
  }
  const bool sloped = md.head_slope != nullptr;
  // capped scores and a bias per distance work on the natural-log score of every element: no shortcut for interior blocks
  const bool terms = md.softcap > 0.f || md.dist_bias != nullptr;
  float sc_nat[2];
  int hq_row[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    hq_row[hf] = min(h0 + (w * 16 + gq + hf * 8) % HB, Hq - 1);
    sc_nat[hf] = scale * (md.head_scale != nullptr ? md.head_scale[hq_row[hf]] : 1.f);
  }
  const int keep = md.chunked ? 0 : md.keep_first;          // keys below `keep` stay visible behind the window
  const int Hv = md.v_div > 1 ? Hkv / md.v_div : Hkv, gv = md.v_div > 1 ? g / md.v_div : g;
  const float inv_cap = md.softcap > 0.f ? 1.f / md.softcap : 0.f;
  const float* brow[2] = {md.dist_bias != nullptr ? md.dist_bias + hq_row[0] : nullptr, md.dist_bias != nullptr ? md.dist_bias + hq_row[1] : nullptr};
  // one score with its terms, natural-log domain in, log2 domain out (the slope is already in the log2 domain)
  auto with_terms = [&](float raw, int hf, int dist) {
    float x = raw * sc_nat[hf];
    if (md.softcap > 0.f) x = softcap_(x, md.softcap, inv_cap);
    if (md.dist_bias != nullptr) x += __ldg(brow[hf] + min(max(dist, 0), md.dist_max) * Hq);
    return x * 1.4426950408889634f - slr[hf] * static_cast<float>(dist);
  };

  int t = t_begin;
  while (t < t_end) {
    const int e = tok_entry[t];
    int tn = t + 1;
    while (tn < t_end && tok_entry[tn] == e) ++tn;
    const int p_first = pos[t];
    const int lo = max(0, first_key(p_first, window, md.chunked)), hi = p_first + (tn - t) - 1;
    const int* bt = block_table + static_cast<long>(e) * max_blocks;
    const int kb0 = (lo / kBN) * kBN;
    // blocks of kept first keys in front of the window's blocks (they end at or before kb0: no key is walked twice)
    const int nkb = keep > 0 ? (min(keep, kb0) + kBN - 1) / kBN : 0;
    const int nblk = nkb + (hi - kb0) / kBN + 1;
    auto block_start = [&](int ib) { return ib < nkb ? ib * kBN : kb0 + (ib - nkb) * kBN; };
    // positions of this thread's rows inside the run (or "not in this run")
    int pq[2], plo[2];
    bool act[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      act[hf] = row_ok[hf] && row_t[hf] >= t && row_t[hf] < tn;
      pq[hf] = p_first + (row_t[hf] - t);
      plo[hf] = first_key(pq[hf], window, md.chunked);
    }
    // keys the warp's rows of this run can see: [wlo, whi]
    const int wa = max(wt_lo, t), wb = min(wt_hi, tn - 1);
    const bool warp_in = wa <= wb;
    const bool warp_full = wt_lo >= t && wt_hi < tn;       // every row of the warp that holds a query belongs to this run
    const int whi = p_first + (wb - t), wlo = first_key(p_first + (wa - t), window, md.chunked);
    const int whi_lo = first_key(whi, window, md.chunked);  // first key of the warp's last row: blocks from here on are seen by all

    __syncthreads();                                       // the previous run's last block has been consumed
    int pg[4];
    block_pages(bt, block_start(0), hi, pg);
    load_kv_block<DP>(sK, k_cache, pg, Hkv, g, block_start(0), hi, D);
    load_kv_block<DVP>(sV, v_cache, pg, Hv, gv, block_start(0), hi, Dv);
    cp_commit();
    if (nblk > 1) block_pages(bt, block_start(1), hi, pg);  // page ids are fetched a block ahead of their use
    for (int ib = 0; ib < nblk; ++ib) {
      const int kb = block_start(ib), buf = ib & 1;
      if (ib + 1 < nblk) {
        const int kn = block_start(ib + 1);
        load_kv_block<DP>(sK + (buf ^ 1) * kBN * LDK, k_cache, pg, Hkv, g, kn, hi, D);
        load_kv_block<DVP>(sV + (buf ^ 1) * kBN * LDV, v_cache, pg, Hv, gv, kn, hi, Dv);
        cp_commit();
        if (ib + 2 < nblk) block_pages(bt, block_start(ib + 2), hi, pg);
        cp_wait<1>();
      } else {
        cp_wait<0>();
      }
      __syncthreads();
      if (warp_in && kb <= whi && (kb + kBN - 1 >= wlo || kb < keep)) {
        const __nv_bfloat16* bK = sK + buf * kBN * LDK;
        const __nv_bfloat16* bV = sV + buf * kBN * LDV;
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        {
          const int m = lane >> 3;
          const int krow = (m >> 1) * 8 + (lane & 7), kcol = (m & 1) * 8;
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
              uint32_t b[4];
              ldsm_x4(smem_u32(bK + (np * 16 + krow) * LDK + ks * 16 + kcol), b);
              mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
              mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
            }
          }
        }
        // scale (log2 domain), mask, online softmax (float).  A block that every row of the warp sees whole needs no mask.
        const bool interior = !sloped && warp_full && kb + kBN - 1 <= p_first + (wt_lo - t) && kb >= whi_lo;
        float mx[2] = {-INFINITY, -INFINITY};
        if (interior && terms) {                           // every key is seen by every row: the terms without the mask
#pragma unroll
          for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int hf = i >> 1;
              s[n][i] = with_terms(s[n][i], hf, pq[hf] - (kb + n * 8 + 2 * tq + (i & 1)));
              mx[hf] = fmaxf(mx[hf], s[n][i]);
            }
          }
        } else if (interior) {
#pragma unroll
          for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              s[n][i] *= sl2[i >> 1];
              mx[i >> 1] = fmaxf(mx[i >> 1], s[n][i]);
            }
          }
        } else {
#pragma unroll
          for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int hf = i >> 1, j = kb + n * 8 + 2 * tq + (i & 1);
              const bool valid = act[hf] && j <= pq[hf] && (j >= plo[hf] || j < keep);
              float sc = -INFINITY;
              if (valid && !terms) {
                sc = s[n][i] * sl2[hf] - slr[hf] * static_cast<float>(pq[hf] - j);
              } else if (valid) {
                sc = with_terms(s[n][i], hf, pq[hf] - j);
              }
              s[n][i] = sc;
              mx[hf] = fmaxf(mx[hf], sc);
            }
          }
        }
        float corr[2], m_sub[2];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
          mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
          const float mn = fmaxf(m_run[hf], mx[hf]);
          corr[hf] = mn == -INFINITY ? 1.f : ex2(m_run[hf] - mn);            // nothing seen yet: nothing to rescale
          m_run[hf] = mn;
          m_sub[hf] = mn == -INFINITY ? 0.f : mn;                             // 2^(-inf - 0) = 0 for a row without keys so far
          l_run[hf] *= corr[hf];
        }
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int hf = i >> 1;
            const float pr = ex2(s[n][i] - m_sub[hf]);
            s[n][i] = pr;
            l_run[hf] += pr;                                                  // per-thread part of the row sum
          }
        }
#pragma unroll
        for (int i = 0; i < 2 * NV; ++i) {
          o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        {
          const int m = lane >> 3;
          const int vrow = (m & 1) * 8 + (lane & 7), vcol = (m >> 1) * 8;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int nv = 0; nv < NV; ++nv) {
              uint32_t b[4];
              ldsm_x4_t(smem_u32(bV + (kk * 16 + vrow) * LDV + nv * 16 + vcol), b);
              mma_bf16(o[2 * nv], pa, b[0], b[1]);
              mma_bf16(o[2 * nv + 1], pa, b[2], b[3]);
            }
          }
        }
      }
      __syncthreads();                                     // all warps are done with `buf` before it is filled again
    }
    t = tn;
  }
  // ---- out = out_scale * O / l ----
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    float l = l_run[hf];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (!row_ok[hf]) continue;
    const int r = w * 16 + gq + hf * 8;
    __nv_bfloat16* dst = out + static_cast<long>(row_t[hf]) * so + static_cast<long>(h0 + r % HB) * Dv;
    float f = out_scale / l;
    if (md.head_sink != nullptr) {                         // one more term in the denominator: a score with no key and no value
      const float s2 = md.head_sink[h0 + r % HB] * 1.4426950408889634f, mt = fmaxf(m_run[hf], s2);
      const float fo = ex2(m_run[hf] - mt);
      f = out_scale * fo / (l * fo + ex2(s2 - mt));
    }
    if (md.gate != nullptr) f *= sigmoid_(md.gate[static_cast<long>(row_t[hf]) * md.gate_stride + h0 + r % HB]);
    float* dstf = md.out_float != nullptr
                      ? md.out_float + static_cast<long>(row_t[hf]) * md.out_float_stride + static_cast<long>(h0 + r % HB) * Dv : nullptr;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) {
      const int c = i * 8 + 2 * tq;
      if (c < Dv) {
        if (dstf != nullptr) {
          dstf[c] = o[i][2 * hf] * f;
          dstf[c + 1] = o[i][2 * hf + 1] * f;
        } else {
          *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(o[i][2 * hf] * f, o[i][2 * hf + 1] * f);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Steps of single tokens: the work is reading the window's pages once, so every WARP walks its own run of pages with its
// own cp.async ring (kDecStages pages of 16 keys in flight, no block barrier in the loop) for the <= 16 query heads that
// share the key/value head, and leaves (O, max, l) of its run as one part; the merge launch combines the parts.
// grid (token, key/value head, split); parts per (token, head) = 4 warps x splits.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kDecStages = 3;

template <int KS, int NV>
__global__ void __launch_bounds__(kThreads)
window_attention_decode_kernel(const float* __restrict__ q, long sq, const __nv_bfloat16* __restrict__ k_cache,
                               const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                               const int* __restrict__ tok_entry, const int* __restrict__ pos, int window, float scale,
                               float* __restrict__ part, int Hq, int Hkv, int D, int Dv, int nsplit, NrlAttnMods md) {
  constexpr int DP = 16 * KS, DVP = 16 * NV, LDK = DP + kPad, LDV = DVP + kPad;
  constexpr int kStageElems = 16 * LDK + 16 * LDV;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [16][LDK]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  __nv_bfloat16* ring = sQ + 16 * LDK + w * kDecStages * kStageElems;        // this warp's [kDecStages]{K [16][LDK], V [16][LDV]}
  const long t = blockIdx.x;
  const int g = blockIdx.y, split = blockIdx.z, per_g = Hq / Hkv, h0 = g * per_g;
  const int nparts = nsplit * 4, pi = split * 4 + w;

  for (int idx = threadIdx.x; idx < 16 * DP; idx += kThreads) {
    const int r = idx / DP, c = idx - r * DP;
    float v = 0.f;
    if (r < per_g && c < D) v = q[t * sq + static_cast<long>(h0 + r) * D + c];
    sQ[r * LDK + c] = __float2bfloat16_rn(v);
  }
  __syncthreads();
  uint32_t qf[KS][4];
  {
    const int m = lane >> 3, rr = (m & 1) * 8 + (lane & 7);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldsm_x4(smem_u32(sQ + rr * LDK + ks * 16 + (m >> 1) * 8), qf[ks]);
  }
  const int p = pos[t];
  const int lo = max(0, first_key(p, window, md.chunked));
  const int* bt = block_table + static_cast<long>(tok_entry[t]) * max_blocks;
  const int keep = md.chunked ? 0 : md.keep_first;          // keys below `keep` stay visible behind the window
  const int Hv = md.v_div > 1 ? Hkv / md.v_div : Hkv, gv = md.v_div > 1 ? g / md.v_div : g;
  // the walk: pages of kept first keys in front of the window's pages; a walk index below nkp is a kept page
  const int pg_first = lo >> 4, nkp = keep > 0 ? min((keep + 15) >> 4, pg_first) : 0, npages = nkp + (p >> 4) - pg_first + 1;
  const int per_part = (npages + nparts - 1) / nparts;
  const int pg0 = pi * per_part, pg1 = min(npages, pg0 + per_part);     // this warp's walk indices [pg0, pg1)
  auto page_of = [&](int wi) { return wi < nkp ? wi : pg_first + wi - nkp; };

  auto load_page = [&](int stage, int wi) {
    const int pg = page_of(wi);
    __nv_bfloat16* sK = ring + stage * kStageElems;
    __nv_bfloat16* sV = sK + 16 * LDK;
    const long cell0 = (static_cast<long>(bt[pg]) * Hkv + g) * 16;
    const long vcell0 = (static_cast<long>(bt[pg]) * Hv + gv) * 16;
    constexpr int kch = DP / 8, vch = DVP / 8;              // powers of two: shifts
#pragma unroll
    for (int idx = lane; idx < 16 * kch; idx += 32) {
      const int key = idx / kch, ch = idx % kch;
      __nv_bfloat16* d = sK + key * LDK + ch * 8;
      if (pg * 16 + key <= p && ch * 8 < D) cp_async16(smem_u32(d), k_cache + (cell0 + key) * D + ch * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);          // padding, or cells after the token
    }
#pragma unroll
    for (int idx = lane; idx < 16 * vch; idx += 32) {
      const int key = idx / vch, ch = idx % vch;
      __nv_bfloat16* d = sV + key * LDV + ch * 8;
      if (pg * 16 + key <= p && ch * 8 < Dv) cp_async16(smem_u32(d), v_cache + (vcell0 + key) * Dv + ch * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  };

  float o[2 * NV][4];
#pragma unroll
  for (int i = 0; i < 2 * NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float sl2[2], slr[2], sc_nat[2];                         // per row (= query head); sl2 / slr in the log2 domain
  int hq_row[2];
  const bool terms = md.softcap > 0.f || md.dist_bias != nullptr;
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int hq = min(h0 + gq + hf * 8, Hq - 1);
    hq_row[hf] = hq;
    sc_nat[hf] = scale * (md.head_scale != nullptr ? md.head_scale[hq] : 1.f);
    sl2[hf] = sc_nat[hf] * 1.4426950408889634f;
    slr[hf] = md.head_slope != nullptr ? md.head_slope[hq] * 1.4426950408889634f : 0.f;
  }
#pragma unroll
  for (int i = 0; i < kDecStages - 1; ++i) {
    if (pg0 + i < pg1) load_page(i, pg0 + i);
    cp_commit();
  }
  for (int wi = pg0; wi < pg1; ++wi) {
    const int pg = page_of(wi);
    const int stage = (wi - pg0) % kDecStages;
    if (wi + kDecStages - 1 < pg1) load_page((wi - pg0 + kDecStages - 1) % kDecStages, wi + kDecStages - 1);
    cp_commit();
    cp_wait<kDecStages - 1>();
    __syncwarp();
    const __nv_bfloat16* bK = ring + stage * kStageElems;
    const __nv_bfloat16* bV = bK + 16 * LDK;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int m = lane >> 3;
      const int krow = (m >> 1) * 8 + (lane & 7), kcol = (m & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b[4];
        ldsm_x4(smem_u32(bK + krow * LDK + ks * 16 + kcol), b);
        mma_bf16(s[0], qf[ks], b[0], b[1]);
        mma_bf16(s[1], qf[ks], b[2], b[3]);
      }
    }
    float mrow[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = pg * 16 + n * 8 + 2 * tq + (i & 1), hf = i >> 1;
        const bool valid = j <= p && (j >= lo || j < keep);
        float sc = -INFINITY;
        if (valid && !terms) {
          sc = s[n][i] * sl2[hf] - slr[hf] * static_cast<float>(p - j);
        } else if (valid) {
          float x = s[n][i] * sc_nat[hf];
          if (md.softcap > 0.f) x = softcap_(x, md.softcap, 1.f / md.softcap);
          if (md.dist_bias != nullptr) x += __ldg(md.dist_bias + static_cast<long>(min(p - j, md.dist_max)) * Hq + hq_row[hf]);
          sc = x * 1.4426950408889634f - slr[hf] * static_cast<float>(p - j);
        }
        s[n][i] = sc;
        mrow[i >> 1] = fmaxf(mrow[i >> 1], sc);
      }
    }
    float corr[2], m_sub[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      mrow[hf] = fmaxf(mrow[hf], __shfl_xor_sync(0xffffffffu, mrow[hf], 1));
      mrow[hf] = fmaxf(mrow[hf], __shfl_xor_sync(0xffffffffu, mrow[hf], 2));
      const float mn = fmaxf(m_run[hf], mrow[hf]);
      corr[hf] = mn == -INFINITY ? 1.f : ex2(m_run[hf] - mn);
      m_run[hf] = mn;
      m_sub[hf] = mn == -INFINITY ? 0.f : mn;
      l_run[hf] *= corr[hf];
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pr = ex2(s[n][i] - m_sub[i >> 1]);
        s[n][i] = pr;
        l_run[i >> 1] += pr;
      }
    }
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
      const int m = lane >> 3;
      const int vrow = (m & 1) * 8 + (lane & 7), vcol = (m >> 1) * 8;
#pragma unroll
      for (int nv = 0; nv < NV; ++nv) {
        uint32_t b[4];
        ldsm_x4_t(smem_u32(bV + vrow * LDV + nv * 16 + vcol), b);
        mma_bf16(o[2 * nv], pa, b[0], b[1]);
        mma_bf16(o[2 * nv + 1], pa, b[2], b[3]);
      }
    }
    __syncwarp();                                          // the stage may be filled again
  }
  cp_wait<0>();
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    float l = l_run[hf];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int r = gq + hf * 8;
    if (r >= per_g) continue;
    float* pd = part + ((t * Hq + h0 + r) * nparts + pi) * (Dv + 2);
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i) {
      const int c = i * 8 + 2 * tq;
      if (c < Dv) {
        pd[c] = o[i][2 * hf];
        pd[c + 1] = o[i][2 * hf + 1];
      }
    }
    if (tq == 0) {
      pd[Dv] = m_run[hf];
      pd[Dv + 1] = l;
    }
  }
}

// block per (token, query head): out = out_scale * sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s
__global__ void window_attention_merge_kernel(const float* __restrict__ part, int nsplit, int Hq, int Dv, float out_scale,
                                              __nv_bfloat16* __restrict__ out, long so, const float* __restrict__ gate, long gate_stride,
                                              const float* __restrict__ head_sink, float* __restrict__ out_float, long out_float_stride) {
  const long t = blockIdx.x;
  const int h = blockIdx.y;
  if (gate != nullptr) out_scale *= sigmoid_(gate[t * gate_stride + h]);
  const float* p = part + (t * Hq + h) * nsplit * (Dv + 2);
  const float sink2 = head_sink != nullptr ? head_sink[h] * 1.4426950408889634f : -INFINITY;   // the sink joins as a part without values
  float M = sink2;
  for (int x = 0; x < nsplit; ++x) M = fmaxf(M, p[x * (Dv + 2) + Dv]);
  float L = head_sink != nullptr ? ex2(sink2 - M) : 0.f;
  for (int x = 0; x < nsplit; ++x) {
    const float m = p[x * (Dv + 2) + Dv];
    if (m != -INFINITY) L += ex2(m - M) * p[x * (Dv + 2) + Dv + 1];
  }
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float a = 0.f;
    for (int x = 0; x < nsplit; ++x) {
      const float m = p[x * (Dv + 2) + Dv];
      if (m != -INFINITY) a += ex2(m - M) * p[x * (Dv + 2) + c];
    }
    if (out_float != nullptr) out_float[t * out_float_stride + static_cast<long>(h) * Dv + c] = out_scale * (a / L);
    else out[t * so + static_cast<long>(h) * Dv + c] = __float2bfloat16_rn(out_scale * (a / L));
  }
}

template <int KS, int NV>
cudaError_t launch(const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
                   const int* tok_entry, const int* pos, int window, float scale, float out_scale, void* out, long so, int T, int Hq,
                   int Hkv, int D, int Dv, int single_token, const NrlAttnMods& md, cudaStream_t s) {
  const int per_g = Hq / Hkv;
  // a step of single tokens that the per-warp kernel does not take: one token per block
  const int HB = per_g < kBM ? per_g : kBM, QT = single_token ? 1 : kBM / HB;
  static_assert(kBM == kBN, "the query tile borrows a key buffer");
  constexpr size_t smem = sizeof(__nv_bfloat16) * (2 * kBN * (16 * KS + kPad) + 2 * kBN * (16 * NV + kPad));
  auto kern = window_attention_mma_kernel<KS, NV>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const dim3 grid((T + QT - 1) / QT, Hkv, (per_g + HB - 1) / HB);
  kern<<<grid, kThreads, smem, s>>>(q, sq, static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache),
                                    block_table, max_blocks, tok_entry, pos, window, scale, out_scale, static_cast<__nv_bfloat16*>(out), so,
                                    T, Hq, Hkv, D, Dv, HB, QT, md);
  return cudaGetLastError();
}

template <int KS, int NV>
cudaError_t launch_decode(const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table, int max_blocks,
                          const int* tok_entry, const int* pos, int window, float scale, float out_scale, void* out, long so, int T,
                          int Hq, int Hkv, int D, int Dv, int nsplit, float* part, const NrlAttnMods& md, cudaStream_t s) {
  constexpr size_t smem = sizeof(__nv_bfloat16) * (16 * (16 * KS + kPad) +
                                                   4 * kDecStages * (16 * (16 * KS + kPad) + 16 * (16 * NV + kPad)));
  auto kern = window_attention_decode_kernel<KS, NV>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kern<<<dim3(T, Hkv, nsplit), kThreads, smem, s>>>(q, sq, static_cast<const __nv_bfloat16*>(k_cache),
                                                    static_cast<const __nv_bfloat16*>(v_cache), block_table, max_blocks, tok_entry, pos,
                                                    window, scale, part, Hq, Hkv, D, Dv, nsplit, md);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  window_attention_merge_kernel<<<dim3(T, Hq), Dv <= 32 ? 32 : Dv <= 64 ? 64 : 128, 0, s>>>(part, nsplit * 4, Hq, Dv, out_scale,
                                                                                          static_cast<__nv_bfloat16*>(out), so, md.gate,
                                                                                          md.gate_stride, md.head_sink, md.out_float, md.out_float_stride);
  return cudaGetLastError();
}

}  // namespace

extern "C" {

// Steps of single tokens (<= 16 query heads per key/value head): every warp walks its own pages and leaves a part.
// `part`: float [T, Hq, 4 nsplit, Dv + 2].
cudaError_t nrl_window_attention_decode(const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table,
                                        int max_blocks, const int* tok_entry, const int* pos, int window, float scale,
                                        float out_scale, void* out, long so, int T, int Hq, int Hkv, int D, int Dv, int page,
                                        int nsplit, float* part, const NrlAttnMods* mods, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  NrlAttnMods md = {0, nullptr, nullptr, nullptr, 0};
  if (mods != nullptr) md = *mods;
  if (!nrl_window_attention_mma_fits(out, so, Hq, Hkv, D, Dv, page) || Hq / Hkv > 16 || window < 1 || nsplit < 1 || part == nullptr)
    return cudaErrorInvalidValue;
  const int ks = D <= 32 ? 2 : D <= 64 ? 4 : 8, nv = Dv <= 32 ? 2 : Dv <= 64 ? 4 : 8;
#define NRL_WD(KS_, NV_)                                                                                                         \
  if (ks == KS_ && nv == NV_)                                                                                                    \
    return launch_decode<KS_, NV_>(q, sq, k_cache, v_cache, block_table, max_blocks, tok_entry, pos, window, scale, out_scale, out, so, \
                                   T, Hq, Hkv, D, Dv, nsplit, part, md, s);
  NRL_WD(2, 2) NRL_WD(2, 4) NRL_WD(2, 8) NRL_WD(4, 2) NRL_WD(4, 4) NRL_WD(4, 8) NRL_WD(8, 2) NRL_WD(8, 4) NRL_WD(8, 8)
#undef NRL_WD
  return cudaErrorInvalidValue;
}

// In how many parts a step of single tokens walks its keys so that the grid fills the GPU (1: no parts, no merge).
int nrl_window_attention_splits(int T, int Hq, int Hkv, int window, int max_blocks, int page) {
  if (Hkv <= 0 || Hq / Hkv > 16) return 0;                  // 0: the single-token kernel does not take this shape
  const long keys = static_cast<long>(max_blocks) * page < window ? static_cast<long>(max_blocks) * page : window;
  const long pages = (keys + 15) / 16 + 1;
  const long blocks = static_cast<long>(T) * Hkv;
  long want = (2 * 148 + blocks - 1) / blocks;              // two blocks per SM
  if (want > pages / 8) want = pages / 8;                   // at least two pages per warp
  if (want > 8) want = 8;
  return want < 1 ? 1 : static_cast<int>(want);
}

int nrl_window_attention_mma_fits(const void* out, long so, int Hq, int Hkv, int D, int Dv, int page) {
  return page == 16 && Hkv > 0 && Hq % Hkv == 0 && D % 8 == 0 && Dv % 8 == 0 && D <= 128 && Dv <= 128 && so % 2 == 0 &&
         reinterpret_cast<uintptr_t>(out) % 4 == 0;
}

cudaError_t nrl_window_attention_mma(const float* q, long sq, const void* k_cache, const void* v_cache, const int* block_table,
                                     int max_blocks, const int* tok_entry, const int* pos, int window, float scale, float out_scale,
                                     void* out, long so, int T, int Hq, int Hkv, int D, int Dv, int page, int single_token,
                                     const NrlAttnMods* mods, cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  NrlAttnMods md = {0, nullptr, nullptr, nullptr, 0};
  if (mods != nullptr) md = *mods;
  if (!nrl_window_attention_mma_fits(out, so, Hq, Hkv, D, Dv, page) || window < 1) return cudaErrorInvalidValue;
  const int ks = D <= 32 ? 2 : D <= 64 ? 4 : 8, nv = Dv <= 32 ? 2 : Dv <= 64 ? 4 : 8;
#define NRL_WM(KS_, NV_)                                                                                                         \
  if (ks == KS_ && nv == NV_)                                                                                                    \
    return launch<KS_, NV_>(q, sq, k_cache, v_cache, block_table, max_blocks, tok_entry, pos, window, scale, out_scale, out, so, T, Hq, \
                            Hkv, D, Dv, single_token, md, s);
  NRL_WM(2, 2) NRL_WM(2, 4) NRL_WM(2, 8) NRL_WM(4, 2) NRL_WM(4, 4) NRL_WM(4, 8) NRL_WM(8, 2) NRL_WM(8, 4) NRL_WM(8, 8)
#undef NRL_WM
  return cudaErrorInvalidValue;
}

}  // extern "C"
