// Mixture-of-experts plumbing around the grouped tcgen05 GEMM (gemm_tc.cu, GROUPED): the routing result (expert ids per token)
// is turned, on the device, into a permutation that sorts the (token, choice) pairs by expert, a table of row tiles for the
// GEMM, and after the two expert GEMMs the rows are combined back per token with the router's weights.  Nothing here
// returns to the host: a step's launches do not depend on the routing.  Compiled WITHOUT fast-math.
#include <cuda_bf16.h>

#include <cstdint>

#include "hybrid_kernels.h"

namespace {

// One block.  ids [R] (R = tokens * top): expert of every pair.  Outputs: slot_of[R] (row of the pair in expert order),
// row_token[R] (token of every row), seg[E + 1] (first row of every expert), tiles [*, 3] = (expert, first row, end row of the
// expert) for every `tile_rows` rows of every expert that has rows, num_tiles[1].
__global__ void moe_plan_kernel(const int* __restrict__ ids, int R, int top, int E, int n_real, int tile_rows, int* __restrict__ slot_of,
                                int* __restrict__ row_token, int* __restrict__ seg, int* __restrict__ tiles, int* __restrict__ num_tiles) {
  extern __shared__ int sh[];
  int* cnt = sh;             // [E]
  int* start = sh + E;       // [E + 1]
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = run;
      const int end = run + cnt[e];
      for (int m0 = run; m0 < end && e < n_real; m0 += tile_rows) {       // identity experts (e >= n_real) have no GEMM tiles
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = m0;
        tiles[3 * nt + 2] = end;
        ++nt;
      }
      run = end;
    }
    start[E] = run;
    num_tiles[0] = nt;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    seg[e] = start[e];
    if (e < E) cnt[e] = start[e];                 // becomes the expert's write cursor
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int s = atomicAdd(&cnt[ids[i]], 1);     // the order of an expert's rows is arbitrary: rows are independent
    slot_of[i] = s;
    row_token[s] = i / top;
  }
}

// out[r, :] = in[row_token[r], :] (16-bit elements, rows of `W` elements; W % 8 == 0, 16-byte aligned rows)
__global__ void gather_rows_kernel(const uint4* __restrict__ in, long in_stride16, const int* __restrict__ row_token, uint4* __restrict__ out,
                                   int R, int W16) {
  const long n = static_cast<long>(R) * W16;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = idx / W16;
    const int c = static_cast<int>(idx - r * W16);
    out[idx] = in[static_cast<long>(row_token[r]) * in_stride16 + c];
  }
}

// act[r, c] (bf16) = silu(gu[r, c]) * gu[r, ff + c];  four columns per thread
__global__ void swiglu_rows_kernel(const float* __restrict__ gu, long sg, __nv_bfloat16* __restrict__ act, long sa, int R, int ff4) {
  const long n = static_cast<long>(R) * ff4;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = idx / ff4;
    const int c = static_cast<int>(idx - r * ff4) * 4;
    const float4 g = *reinterpret_cast<const float4*>(gu + r * sg + c);
    const float4 u = *reinterpret_cast<const float4*>(gu + r * sg + ff4 * 4 + c);
    const float a0 = g.x / (1.f + expf(-g.x)) * u.x, a1 = g.y / (1.f + expf(-g.y)) * u.y;
    const float a2 = g.z / (1.f + expf(-g.z)) * u.z, a3 = g.w / (1.f + expf(-g.w)) * u.w;
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1), hi = __floats2bfloat162_rn(a2, a3);
    uint2 o;
    o.x = *reinterpret_cast<const unsigned*>(&lo);
    o.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(act + r * sa + c) = o;
  }
}

// out[t, :] = sum_k wts[t, k] * y[slot_of[t * top + k], :] in the order of k;  four columns per thread
__global__ void moe_combine_kernel(const float* __restrict__ y, long sy, const int* __restrict__ slot_of, const float* __restrict__ wts,
                                   int top, float* __restrict__ out, long so, int T, int W4) {
  const long n = static_cast<long>(T) * W4;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const long t = idx / W4;
    const int c = static_cast<int>(idx - t * W4) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top; ++k) {
      const float w = wts[t * top + k];
      if (w == 0.f) continue;                       // an identity expert's pair: its row was never computed
      const float4 v = *reinterpret_cast<const float4*>(y + static_cast<long>(slot_of[t * top + k]) * sy + c);
      acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    }
    *reinterpret_cast<float4*>(out + t * so + c) = acc;
  }
}

inline int grid_for(long n, int threads) {
  const long b = (n + threads - 1) / threads;
  return static_cast<int>(b < 148 * 16 ? (b < 1 ? 1 : b) : 148 * 16);
}

}  // namespace

extern "C" {

cudaError_t nrl_moe_plan(const int* ids, int R, int top, int E, int n_real, int tile_rows, int* slot_of, int* row_token, int* seg, int* tiles,
                         int* num_tiles, cudaStream_t s) {
  if (R <= 0) return cudaSuccess;
  if (E < 1 || E > 8192 || top < 1 || tile_rows < 1 || n_real < 0 || n_real > E) return cudaErrorInvalidValue;
  moe_plan_kernel<<<1, 1024, sizeof(int) * (2 * E + 1), s>>>(ids, R, top, E, n_real, tile_rows, slot_of, row_token, seg, tiles, num_tiles);
  return cudaGetLastError();
}

cudaError_t nrl_gather_rows16(const void* in, long in_stride, const int* row_token, void* out, int R, int W, cudaStream_t s) {
  if (R <= 0) return cudaSuccess;
  if (W % 8 != 0 || in_stride % 8 != 0 || reinterpret_cast<uintptr_t>(in) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0)
    return cudaErrorInvalidValue;
  const long n = static_cast<long>(R) * (W / 8);
  gather_rows_kernel<<<grid_for(n, 256), 256, 0, s>>>(static_cast<const uint4*>(in), in_stride / 8, row_token, static_cast<uint4*>(out), R, W / 8);
  return cudaGetLastError();
}

cudaError_t nrl_swiglu_rows(const float* gu, long sg, void* act, long sa, int R, int ff, cudaStream_t s) {
  if (R <= 0) return cudaSuccess;
  if (ff % 4 != 0 || sg % 4 != 0 || sa % 4 != 0 || reinterpret_cast<uintptr_t>(gu) % 16 != 0 || reinterpret_cast<uintptr_t>(act) % 8 != 0)
    return cudaErrorInvalidValue;
  const long n = static_cast<long>(R) * (ff / 4);
  swiglu_rows_kernel<<<grid_for(n, 256), 256, 0, s>>>(gu, sg, static_cast<__nv_bfloat16*>(act), sa, R, ff / 4);
  return cudaGetLastError();
}

cudaError_t nrl_moe_combine(const float* y, long sy, const int* slot_of, const float* wts, int top, float* out, long so, int T, int W,
                            cudaStream_t s) {
  if (T <= 0) return cudaSuccess;
  if (W % 4 != 0 || sy % 4 != 0 || so % 4 != 0 || reinterpret_cast<uintptr_t>(y) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0)
    return cudaErrorInvalidValue;
  const long n = static_cast<long>(T) * (W / 4);
  moe_combine_kernel<<<grid_for(n, 256), 256, 0, s>>>(y, sy, slot_of, wts, top, out, so, T, W / 4);
  return cudaGetLastError();
}

}  // extern "C"
