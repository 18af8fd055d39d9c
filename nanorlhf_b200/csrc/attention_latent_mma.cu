// Latent attention on the tensor cores, reading the 16-token bf16 pages in place.  A page row is [latent (Dv columns) | rotated
// shared key part] = D columns; it is the key of every head (queries arrive absorbed into that space) and its first Dv
// columns are the value of every head, so ONE shared-memory tile per key block feeds both S = Q K^T and O += P V.  Causal;
// the softmax denominator may hold exp(sink_h); a sigmoid gate per head scales the result (NrlAttnMods).
//
// Prompt portions (latent_attention_mma_kernel): a block owns 64 query rows -- QT consecutive tokens x HB heads -- as four
// warps of 16 rows and walks the keys its rows can see in blocks of 64 or 32 (whole pages), double buffered with cp.async.
// Rows can be up to 576 columns wide (tiles of 128 to 576 columns), so the queries stay in shared memory (A fragments are
// fetched per 16 columns) and a block accumulates a slice of 128 or (values wider than 128) 256 value columns; further slices
// are further blocks, which repeat S.
// Scores, mask and online softmax are float (base 2, ex2.approx); P is rounded to bf16 only as the operand of O += P V.
// Steps of single tokens (latent_attention_decode_kernel): every warp walks its own pages for up to 16 heads and leaves
// (O, max, l) as one part; window_attention_merge (attention_window_mma.cu's form, here with the sink) combines the parts.
// Compiled WITHOUT fast-math.
#include <cuda_bf16.h>

#include <cstdint>

#include "hybrid_kernels.h"

namespace {

constexpr int kBM = 64;        // query rows per block
constexpr int kThreads = 128;
constexpr int kPad = 8;        // bf16 elements appended to a shared-memory row (ldmatrix without bank conflicts)
constexpr float kLog2e = 1.4426950408889634f;

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
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float sigmoid_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ int sel4(const int (&v)[4], int i) { return i == 0 ? v[0] : i == 1 ? v[1] : i == 2 ? v[2] : v[3]; }

__device__ __forceinline__ void block_pages(const int* bt, int kb, int hi, int (&pg)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) pg[i] = kb + 16 * i <= hi ? bt[(kb >> 4) + i] : 0;
}

// one block of BN keys (cache rows) into shared memory: rows = keys kb .. kb + BN - 1 of the sequence, D real columns of DP
template <int DP, int BN>
__device__ __forceinline__ void load_rows(__nv_bfloat16* dst, const __nv_bfloat16* cache, const int (&pg)[4], int kb, int hi, int D) {
  constexpr int chunks = DP / 8, ld = DP + kPad;
  for (int idx = threadIdx.x; idx < BN * chunks; idx += kThreads) {
    const int key = idx / chunks, ch = idx - key * chunks;
    __nv_bfloat16* d = dst + key * ld + ch * 8;
    if (kb + key <= hi && ch * 8 < D) {
      const long cell = static_cast<long>(sel4(pg, key >> 4)) * 16 + (key & 15);
      cp_async16(smem_u32(d), cache + cell * D + ch * 8);
    } else {
      *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// shared memory of the prompt kernel: ST key buffers and the queries; two blocks per SM need <= 113 KB each, three <= 75 KB
__host__ __device__ constexpr size_t prefill_smem(int ks, int bn, int st) {
  return sizeof(__nv_bfloat16) * (st * bn + kBM) * (16 * ks + kPad);
}

// padded D = 16 KS; BN keys per block of the walk (64, or 32 where that lets two blocks share an SM); ST key buffers in flight;
// VG 16-column value groups per block (8, or 16: all of 256 value columns from one S, at 128 accumulator registers)
template <int KS, int BN, int ST, int VG>
__global__ void __launch_bounds__(kThreads, (VG <= 8 && prefill_smem(KS, BN, ST) <= 75 * 1024) ? 3 : prefill_smem(KS, BN, ST) <= 113 * 1024 ? 2 : 1)
latent_attention_mma_kernel(const float* __restrict__ q, long sq, const __nv_bfloat16* __restrict__ cache,
                            const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_entry,
                            const int* __restrict__ pos, float scale, float out_scale, __nv_bfloat16* __restrict__ out, long so, int T,
                            int H, int D, int Dv, int HB, int QT, NrlAttnMods md) {
  constexpr int DP = 16 * KS, LDK = DP + kPad;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [ST][BN][LDK]
  __nv_bfloat16* sQ = sK + ST * BN * LDK;                                     // [kBM][LDK]
  constexpr int NB = BN / 8;                                                  // 8-key score fragments per block
  const int zb = static_cast<int>(blockIdx.z), vs = static_cast<int>(blockIdx.y);
  const int h0 = zb * HB, hb = min(HB, H - zb * HB);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  const int t_begin = blockIdx.x * QT, t_end = min(T, t_begin + QT);
  const long qhs = md.q_head_stride ? md.q_head_stride : D;
  const int v0 = vs * VG * 16;                              // first value column of this block
  const int nvg = min(VG, (DP - v0) / 16);                   // 16-column groups of the slice that lie inside the tile

  for (int idx = threadIdx.x; idx < kBM * DP; idx += kThreads) {
    const int r = idx / DP, c = idx - r * DP;
    const int tt = t_begin + r / HB, hh = r % HB;
    float v = 0.f;
    if (r < QT * HB && tt < t_end && hh < hb && c < D) v = q[static_cast<long>(tt) * sq + static_cast<long>(h0 + hh) * qhs + c];
    sQ[r * LDK + c] = __float2bfloat16_rn(v);
  }
  __syncthreads();
  int row_t[2];
  bool row_ok[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int r = w * 16 + gq + hf * 8;
    row_t[hf] = t_begin + r / HB;
    row_ok[hf] = r < QT * HB && row_t[hf] < t_end && (r % HB) < hb;
  }
  const int wt_lo = t_begin + (w * 16) / HB, wt_hi = min(t_end - 1, t_begin + (w * 16 + 15) / HB);
  const uint32_t q_addr = smem_u32(sQ + (w * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDK + (lane >> 4) * 8);

  float o[2 * VG][4];
#pragma unroll
  for (int i = 0; i < 2 * VG; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // running maxima live in the log2 domain
  const float sl2 = scale * kLog2e;

  int t = t_begin;
  while (t < t_end) {
    const int e = tok_entry[t];
    int tn = t + 1;
    while (tn < t_end && tok_entry[tn] == e) ++tn;
    const int p_first = pos[t];
    const int hi = p_first + (tn - t) - 1;
    const int* bt = block_table + static_cast<long>(e) * max_blocks;
    const int nblk = hi / BN + 1;
    int pq[2];
    bool act[2];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      act[hf] = row_ok[hf] && row_t[hf] >= t && row_t[hf] < tn;
      pq[hf] = p_first + (row_t[hf] - t);
    }
    const int wa = max(wt_lo, t), wb = min(wt_hi, tn - 1);
    const bool warp_in = wa <= wb;
    const bool warp_full = wt_lo >= t && wt_hi < tn;
    const int whi = p_first + (wb - t);                     // the last key any row of the warp sees

    __syncthreads();                                       // the previous run's last block has been consumed
    int pg[4];
    block_pages(bt, 0, hi, pg);
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {                      // ST - 1 key blocks in flight before the first is used
      if (i < nblk) {
        load_rows<DP, BN>(sK + i * BN * LDK, cache, pg, i * BN, hi, D);
        if (i + 1 < nblk) block_pages(bt, (i + 1) * BN, hi, pg);      // page ids are fetched a block ahead of their use
      }
      cp_commit();                                         // (an empty group keeps the count per iteration fixed)
    }
    for (int ib = 0; ib < nblk; ++ib) {
      const int kb = ib * BN, buf = ib % ST, nxt = ib + ST - 1;
      if (nxt < nblk) {                                    // its buffer held block ib - 1, which every warp has left
        load_rows<DP, BN>(sK + (nxt % ST) * BN * LDK, cache, pg, nxt * BN, hi, D);
        if (nxt + 1 < nblk) block_pages(bt, (nxt + 1) * BN, hi, pg);
      }
      cp_commit();
      cp_wait<ST - 1>();
      __syncthreads();
      if (warp_in && kb <= whi) {
        const __nv_bfloat16* bK = sK + buf * BN * LDK;
        float s[NB][4];
#pragma unroll
        for (int i = 0; i < NB; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        {
          const int m = lane >> 3;
          const uint32_t k_addr = smem_u32(bK + ((m >> 1) * 8 + (lane & 7)) * LDK + (m & 1) * 8);
#pragma unroll 4
          for (int ks = 0; ks < KS; ++ks) {
            uint32_t qf[4];
            ldsm_x4(q_addr + ks * 32, qf);
#pragma unroll
            for (int np = 0; np < NB / 2; ++np) {
              uint32_t b[4];
              ldsm_x4(k_addr + (np * 16 * LDK + ks * 16) * 2, b);
              mma_bf16(s[2 * np], qf, b[0], b[1]);
              mma_bf16(s[2 * np + 1], qf, b[2], b[3]);
            }
          }
        }
        // a block whose last key no row of the warp precedes needs no mask
        const bool interior = warp_full && kb + BN - 1 <= p_first + (wt_lo - t);
        float mx[2] = {-INFINITY, -INFINITY};
        if (interior) {
#pragma unroll
          for (int n = 0; n < NB; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              s[n][i] *= sl2;
              mx[i >> 1] = fmaxf(mx[i >> 1], s[n][i]);
            }
          }
        } else {
#pragma unroll
          for (int n = 0; n < NB; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int hf = i >> 1, j = kb + n * 8 + 2 * tq + (i & 1);
              const float sc = (act[hf] && j <= pq[hf]) ? s[n][i] * sl2 : -INFINITY;
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
          corr[hf] = mn == -INFINITY ? 1.f : ex2(m_run[hf] - mn);
          m_run[hf] = mn;
          m_sub[hf] = mn == -INFINITY ? 0.f : mn;
          l_run[hf] *= corr[hf];
        }
#pragma unroll
        for (int n = 0; n < NB; ++n) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float pr = ex2(s[n][i] - m_sub[i >> 1]);
            s[n][i] = pr;
            l_run[i >> 1] += pr;
          }
        }
#pragma unroll
        for (int i = 0; i < 2 * VG; ++i) {
          o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        {
          const int m = lane >> 3;
          const uint32_t v_addr = smem_u32(bK + ((m & 1) * 8 + (lane & 7)) * LDK + v0 + (m >> 1) * 8);
#pragma unroll
          for (int kk = 0; kk < NB / 2; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int nv = 0; nv < VG; ++nv) {
              if (nv < nvg) {
                uint32_t b[4];
                ldsm_x4_t(v_addr + (kk * 16 * LDK + nv * 16) * 2, b);
                mma_bf16(o[2 * nv], pa, b[0], b[1]);
                mma_bf16(o[2 * nv + 1], pa, b[2], b[3]);
              }
            }
          }
        }
      }
      __syncthreads();                                     // all warps are done with `buf` before it is filled again
    }
    t = tn;
  }
  // ---- out = out_scale * gate * O / (l + 2^(sink - m)) ----
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    float l = l_run[hf];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (!row_ok[hf]) continue;
    const int r = w * 16 + gq + hf * 8, hq = h0 + r % HB;
    if (md.head_sink != nullptr) l += ex2(md.head_sink[hq] * kLog2e - m_run[hf]);
    __nv_bfloat16* dst = out + static_cast<long>(row_t[hf]) * so + static_cast<long>(hq) * Dv;
    float f = out_scale / l;
    if (md.gate != nullptr) f *= sigmoid_(md.gate[static_cast<long>(row_t[hf]) * md.gate_stride + hq]);
#pragma unroll
    for (int i = 0; i < 2 * VG; ++i) {
      const int c = v0 + i * 8 + 2 * tq;
      if (c < Dv) *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(o[i][2 * hf] * f, o[i][2 * hf + 1] * f);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Steps of single tokens.  grid (token, head group of <= 16 heads x value slice, split); every warp walks its own run of pages
// with its own cp.async ring and leaves (O slice, max, l) as one part: float [T, H, 4 nsplit, Dv + 2].
// ---------------------------------------------------------------------------------------------------------------------
template <int KS, int STAGES, int VG>      // VG: 16-column value groups per block (8 or 16)
__global__ void __launch_bounds__(kThreads)
latent_attention_decode_kernel(const float* __restrict__ q, long sq, const __nv_bfloat16* __restrict__ cache,
                               const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_entry,
                               const int* __restrict__ pos, float scale, float* __restrict__ part, int H, int D, int Dv, int nvs, int nsplit,
                               long qhs) {
  constexpr int DP = 16 * KS, LDK = DP + kPad;
  constexpr int kStageElems = 16 * LDK;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [16][LDK]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  __nv_bfloat16* ring = sQ + 16 * LDK + w * STAGES * kStageElems;            // this warp's [STAGES][16][LDK]
  const long t = blockIdx.x;
  const int hg = static_cast<int>(blockIdx.y) / nvs, vs = static_cast<int>(blockIdx.y) % nvs, split = blockIdx.z;
  const int h0 = hg * 16, per = min(16, H - h0);
  const int nparts = nsplit * 4, pi = split * 4 + w;
  const int v0 = vs * VG * 16, nvg = min(VG, (DP - v0) / 16);

  for (int idx = threadIdx.x; idx < 16 * DP; idx += kThreads) {
    const int r = idx / DP, c = idx - r * DP;
    float v = 0.f;
    if (r < per && c < D) v = q[t * sq + static_cast<long>(h0 + r) * qhs + c];
    sQ[r * LDK + c] = __float2bfloat16_rn(v);
  }
  __syncthreads();
  const uint32_t q_addr = smem_u32(sQ + (((lane >> 3) & 1) * 8 + (lane & 7)) * LDK + (lane >> 4) * 8);
  const int p = pos[t];
  const int* bt = block_table + static_cast<long>(tok_entry[t]) * max_blocks;
  const int npages = (p >> 4) + 1;
  const int per_part = (npages + nparts - 1) / nparts;
  const int pg0 = pi * per_part, pg1 = min(npages, pg0 + per_part);          // this warp's pages [pg0, pg1)

  // A page is 16 rows of D columns, contiguous in global memory; in shared memory its rows are LDK apart.  The padding columns
  // (D .. DP) of every stage are zeroed once; a page's copy then walks the real 16-byte chunks with running (row, chunk) counters.
  const int dch = D >> 3;                                  // real 16-byte chunks per row
  if (dch < DP / 8) {
    for (int idx = lane; idx < STAGES * 16 * (DP / 8 - dch); idx += 32) {
      const int row = idx / (DP / 8 - dch), ch = dch + idx % (DP / 8 - dch);
      *reinterpret_cast<uint4*>(ring + row * LDK + ch * 8) = make_uint4(0u, 0u, 0u, 0u);      // rows of all stages are LDK apart
    }
  }
  const int key_first = lane / dch, ch_first = lane - key_first * dch;
  const int key_step = 32 / dch, ch_step = 32 - key_step * dch;
  auto load_page = [&](int stage, int pg) {
    __nv_bfloat16* sK = ring + stage * kStageElems;
    const __nv_bfloat16* src = cache + static_cast<long>(bt[pg]) * 16 * D;
    const int last = min(15, p - pg * 16);                 // rows after the token's own (last page only) are zero-filled
    int key = key_first, ch = ch_first;
    for (int idx = lane; idx < 16 * dch; idx += 32) {
      __nv_bfloat16* d = sK + key * LDK + ch * 8;
      if (key <= last) cp_async16(smem_u32(d), src + static_cast<long>(idx) * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
      key += key_step;
      ch += ch_step;
      if (ch >= dch) {
        ch -= dch;
        ++key;
      }
    }
  };

  float o[2 * VG][4];
#pragma unroll
  for (int i = 0; i < 2 * VG; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = scale * kLog2e;
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (pg0 + i < pg1) load_page(i, pg0 + i);
    cp_commit();
  }
  for (int pg = pg0; pg < pg1; ++pg) {
    const int stage = (pg - pg0) % STAGES;
    if (pg + STAGES - 1 < pg1) load_page((pg - pg0 + STAGES - 1) % STAGES, pg + STAGES - 1);
    cp_commit();
    cp_wait<STAGES - 1>();
    __syncwarp();
    const __nv_bfloat16* bK = ring + stage * kStageElems;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int m = lane >> 3;
      const uint32_t k_addr = smem_u32(bK + ((m >> 1) * 8 + (lane & 7)) * LDK + (m & 1) * 8);
      // two accumulator sets (even / odd 16-column steps): the chain of dependent mma is half as long
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 2
      for (int ks = 0; ks + 1 < KS; ks += 2) {
        uint32_t qf[4], b[4], qg[4], c[4];
        ldsm_x4(q_addr + ks * 32, qf);
        ldsm_x4(k_addr + ks * 32, b);
        ldsm_x4(q_addr + ks * 32 + 32, qg);
        ldsm_x4(k_addr + ks * 32 + 32, c);
        mma_bf16(s[0], qf, b[0], b[1]);
        mma_bf16(s[1], qf, b[2], b[3]);
        mma_bf16(s2[0], qg, c[0], c[1]);
        mma_bf16(s2[1], qg, c[2], c[3]);
      }
      if (KS & 1) {
        uint32_t qf[4], b[4];
        ldsm_x4(q_addr + (KS - 1) * 32, qf);
        ldsm_x4(k_addr + (KS - 1) * 32, b);
        mma_bf16(s[0], qf, b[0], b[1]);
        mma_bf16(s[1], qf, b[2], b[3]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s[0][i] += s2[0][i];
        s[1][i] += s2[1][i];
      }
    }
    float mrow[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = pg * 16 + n * 8 + 2 * tq + (i & 1);
        const float sc = j <= p ? s[n][i] * sl2 : -INFINITY;
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
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {      // a maximum grew (rare after the first pages)
#pragma unroll
      for (int i = 0; i < 2 * VG; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
    }
    {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
      const int m = lane >> 3;
      const uint32_t v_addr = smem_u32(bK + ((m & 1) * 8 + (lane & 7)) * LDK + v0 + (m >> 1) * 8);
#pragma unroll
      for (int nv = 0; nv < VG; ++nv) {
        if (nv < nvg) {
          uint32_t b[4];
          ldsm_x4_t(v_addr + nv * 32, b);
          mma_bf16(o[2 * nv], pa, b[0], b[1]);
          mma_bf16(o[2 * nv + 1], pa, b[2], b[3]);
        }
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
    if (r >= per) continue;
    float* pd = part + ((t * H + h0 + r) * nparts + pi) * (Dv + 2);
#pragma unroll
    for (int i = 0; i < 2 * VG; ++i) {
      const int c = v0 + i * 8 + 2 * tq;
      if (c < Dv) {
        pd[c] = o[i][2 * hf];
        pd[c + 1] = o[i][2 * hf + 1];
      }
    }
    if (tq == 0 && vs == 0) {                              // every value slice finds the same maximum and sum
      pd[Dv] = m_run[hf];
      pd[Dv + 1] = l;
    }
  }
}

// block per (token, head): out = out_scale * gate * sum_s 2^(m_s - M) O_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)).
// The first warp turns the parts' maxima and sums into one weight per part (nparts <= 32), then every thread sums its columns.
__global__ void latent_attention_merge_kernel(const float* __restrict__ part, int nparts, int H, int Dv, float out_scale,
                                              __nv_bfloat16* __restrict__ out, long so, const float* __restrict__ gate, long gate_stride,
                                              const float* __restrict__ sink) {
  __shared__ float wsh[32];
  const long t = blockIdx.x;
  const int h = blockIdx.y;
  const float* p = part + (t * H + h) * nparts * (Dv + 2);
  if (threadIdx.x < 32) {
    const int x = threadIdx.x;
    const float m = x < nparts ? p[x * (Dv + 2) + Dv] : -INFINITY;
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float w = m == -INFINITY ? 0.f : ex2(m - M);
    float L = x < nparts ? w * p[x * (Dv + 2) + Dv + 1] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (sink != nullptr) L += ex2(sink[h] * kLog2e - M);
    if (gate != nullptr) out_scale *= sigmoid_(gate[t * gate_stride + h]);
    wsh[x] = w * (out_scale / L);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < Dv; c += blockDim.x) {
    float a = 0.f;
    for (int x = 0; x < nparts; ++x) {
      const float w = wsh[x];
      if (w != 0.f) a += w * p[x * (Dv + 2) + c];
    }
    out[t * so + static_cast<long>(h) * Dv + c] = __float2bfloat16_rn(a);
  }
}

template <int KS, int BN, int ST, int VG>
cudaError_t launch_prefill(const float* q, long sq, const void* cache, const int* block_table, int max_blocks, const int* tok_entry,
                           const int* pos, float scale, float out_scale, void* out, long so, int T, int H, int D, int Dv, int single_token,
                           const NrlAttnMods& md, cudaStream_t s) {
  const int HB = H < kBM ? H : kBM, QT = single_token ? 1 : kBM / HB;
  constexpr size_t smem = prefill_smem(KS, BN, ST);
  auto kern = latent_attention_mma_kernel<KS, BN, ST, VG>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const dim3 grid((T + QT - 1) / QT, (Dv + VG * 16 - 1) / (VG * 16), (H + HB - 1) / HB);
  kern<<<grid, kThreads, smem, s>>>(q, sq, static_cast<const __nv_bfloat16*>(cache), block_table, max_blocks, tok_entry, pos, scale,
                                    out_scale, static_cast<__nv_bfloat16*>(out), so, T, H, D, Dv, HB, QT, md);
  return cudaGetLastError();
}

template <int KS, int STAGES, int VG>
cudaError_t launch_decode(const float* q, long sq, const void* cache, const int* block_table, int max_blocks, const int* tok_entry,
                          const int* pos, float scale, float out_scale, void* out, long so, int T, int H, int D, int Dv, int nsplit,
                          float* part, const NrlAttnMods& md, cudaStream_t s) {
  constexpr size_t smem = sizeof(__nv_bfloat16) * (16 + 4 * STAGES * 16) * (16 * KS + kPad);
  auto kern = latent_attention_decode_kernel<KS, STAGES, VG>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int nvs = (Dv + VG * 16 - 1) / (VG * 16);
  kern<<<dim3(T, ((H + 15) / 16) * nvs, nsplit), kThreads, smem, s>>>(q, sq, static_cast<const __nv_bfloat16*>(cache), block_table, max_blocks,
                                                                      tok_entry, pos, scale, part, H, D, Dv, nvs, nsplit,
                                                                      md.q_head_stride ? md.q_head_stride : D);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  latent_attention_merge_kernel<<<dim3(T, H), Dv <= 32 ? 32 : Dv <= 64 ? 64 : 128, 0, s>>>(part, nsplit * 4, H, Dv, out_scale,
                                                                                         static_cast<__nv_bfloat16*>(out), so, md.gate,
                                                                                         md.gate_stride, md.head_sink);
  return cudaGetLastError();
}

}  // namespace

extern "C" {

int nrl_latent_attention_mma_fits(const void* out, long so, int D, int Dv, int page) {
  return page == 16 && D % 8 == 0 && Dv % 8 == 0 && Dv >= 8 && Dv <= D && D <= 576 && so % 2 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0;
}

// In how many parts a step of single tokens walks its keys so that the grid fills the GPU.
int nrl_latent_attention_splits(int T, int H, int Dv, int max_blocks) {
  const long blocks = static_cast<long>(T) * ((H + 15) / 16) * ((Dv + 255) / 256);
  long want = (2 * 148 + blocks - 1) / blocks;              // two blocks per SM
  const long pages = max_blocks;
  if (want > pages / 8) want = pages / 8;                   // at least two pages per warp
  if (want > 8) want = 8;
  return want < 1 ? 1 : static_cast<int>(want);
}

// out typed bf16 [T, H * Dv] (row stride so) = out_scale * gate * softmax_with_sink(scale q . row) rows[:, :Dv] over the causal
// keys of each token's sequence.  q float [T, H * D] (row stride sq); cache bf16 [pages, 1, 16, D].  nsplit >= 1 with `part`
// float [T, H, 4 nsplit, Dv + 2] selects the single-token kernel (+ merge) for steps in which every entry holds one token.
cudaError_t nrl_latent_attention_mma(const float* q, long sq, const void* cache, const int* block_table, int max_blocks,
                                     const int* tok_entry, const int* pos, float scale, float out_scale, void* out, long so, int T, int H,
                                     int D, int Dv, int page, int single_token, int nsplit, float* part, const NrlAttnMods* mods,
                                     cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  NrlAttnMods md = {0, nullptr, nullptr, nullptr, 0, nullptr, 0, 0};
  if (mods != nullptr) md = *mods;
  if (!nrl_latent_attention_mma_fits(out, so, D, Dv, page) || H < 1 || md.chunked || md.head_scale != nullptr || md.head_slope != nullptr)
    return cudaErrorInvalidValue;
  const int ks = D <= 128 ? 8 : D <= 192 ? 12 : D <= 256 ? 16 : D <= 320 ? 20 : D <= 384 ? 24 : D <= 448 ? 28 : 36;
  if (single_token && nsplit >= 1 && part != nullptr) {
    // values of more than 128 columns: 256 per block, so that a page is read and scored once per 256 (not 128) value columns
#define NRL_LD(KS_, ST_, VG_)                                                                                                    \
  if (ks == KS_)                                                                                                                 \
    return launch_decode<KS_, ST_, VG_>(q, sq, cache, block_table, max_blocks, tok_entry, pos, scale, out_scale, out, so, T, H, D, Dv,  \
                                        nsplit, part, md, s);
    // stages: two blocks per SM where shared memory allows (rows up to 384 columns) -- at rows of 320 columns one block with a
    // five-page ring per warp measured 163 us where two blocks with two pages each take 120: the warps' instruction streams,
    // not the bytes in flight, bound the walk
    NRL_LD(8, 3, 8) NRL_LD(12, 4, 16) NRL_LD(16, 3, 16) NRL_LD(20, 2, 16) NRL_LD(24, 2, 16) NRL_LD(28, 3, 16) NRL_LD(36, 2, 16)
#undef NRL_LD
  }
#define NRL_LP(KS_, BN_, ST_)                                                                                                    \
  if (ks == KS_ && (KS_ <= 8 || Dv <= 128))                                                                                      \
    return launch_prefill<KS_, BN_, ST_, 8>(q, sq, cache, block_table, max_blocks, tok_entry, pos, scale, out_scale, out, so, T, H, \
                                            D, Dv, single_token, md, s);                                                          \
  if (ks == KS_)                                                                                                                 \
    return launch_prefill<(KS_ <= 8 ? 12 : KS_), BN_, ST_, 16>(q, sq, cache, block_table, max_blocks, tok_entry, pos, scale, out_scale, \
                                                               out, so, T, H, D, Dv, single_token, md, s);
  // 64 keys per block where two or three blocks still share an SM, else 32 (two blocks up to rows of 384 columns); a third
  // key buffer where it costs no block per SM
  NRL_LP(8, 64, 2) NRL_LP(12, 64, 2) NRL_LP(16, 32, 2) NRL_LP(20, 32, 3) NRL_LP(24, 32, 2) NRL_LP(28, 32, 3) NRL_LP(36, 32, 3)
#undef NRL_LP
  return cudaErrorInvalidValue;
}

}  // extern "C"
