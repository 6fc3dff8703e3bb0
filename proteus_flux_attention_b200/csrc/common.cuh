// Shared helpers for the ASPA sm_100a kernels: error reporting, dtype loads,
// order-preserving float keys, warp/block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/aspa_b200.h"

namespace aspa {

void set_error(const char* fmt, ...);

#define ASPA_CHECK_ARG(cond, msg)                 \
  do {                                            \
    if (!(cond)) {                                \
      ::aspa::set_error("%s: %s", __func__, msg); \
      return ASPA_ERR_ARG;                        \
    }                                             \
  } while (0)

#define ASPA_CHECK_LAUNCH()                                                            \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess) {                                                          \
      ::aspa::set_error("%s: launch failed: %s", __func__, cudaGetErrorString(e__));   \
      return ASPA_ERR_CUDA;                                                            \
    }                                                                                  \
  } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- dtype access -----------------------------------------------------------
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p, int64_t i);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float ld_as_float<int8_t>(const int8_t* p, int64_t i) { return (float)p[i]; }

template <typename T>
__device__ __forceinline__ void st_from_float(T* p, int64_t i, float v);
template <>
__device__ __forceinline__ void st_from_float<float>(float* p, int64_t i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void st_from_float<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) {
  p[i] = __float2bfloat16_rn(v);
}

// ---- ordering ---------------------------------------------------------------
// Monotone map float -> uint32: a > b  <=>  key(a) > key(b)  (-0 < +0; NaNs land at the ends).
__device__ __forceinline__ uint32_t float_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// ---- reductions -------------------------------------------------------------
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
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide exclusive scan of one int per thread (blockDim.x <= 1024, multiple of 32).
// `warp_tot` is shared scratch of 33 ints. Returns the exclusive prefix; *total gets the block sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_tot, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = lane < nwarp ? warp_tot[lane] : 0;
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < nwarp) warp_tot[lane] = winc - w;
    if (lane == 31) warp_tot[32] = winc;
  }
  __syncthreads();
  int res = warp_tot[warp] + inc - v;
  *total = warp_tot[32];
  __syncthreads();
  return res;
}

// ---- selection on keys held in registers ---------------------------------------------------------------
// Block-wide sum of one int per thread (blockDim.x multiple of 32, <= 1024); `tmp` is 33 ints of shared memory.
__device__ __forceinline__ int block_sum_int(int v, int* tmp) {
  v = warp_sum_int(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) tmp[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (int)(blockDim.x >> 5) ? tmp[lane] : 0;
    w = warp_sum_int(w);
    if (lane == 0) tmp[32] = w;
  }
  __syncthreads();
  return tmp[32];
}

// Block-wide sum with ONE barrier: hardware warp reduction, one shared slot per warp, every warp re-reduces the
// slots.  `buf` holds 64 ints; `parity` (a register of the caller, uniform across the block) alternates between
// its two halves so that a slot is never overwritten before every warp has read it.
__device__ __forceinline__ int block_sum_1bar(int v, int* buf, int& parity) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  v = __reduce_add_sync(0xffffffffu, v);
  int* b = buf + (parity ? 32 : 0);
  parity ^= 1;
  if (lane == 0) b[warp] = v;
  __syncthreads();
  return __reduce_add_sync(0xffffffffu, lane < nwarp ? b[lane] : 0);
}

// The need-th largest (1-based) of the block's keys, found bit by bit: 32 rounds of "how many keys >= candidate",
// no atomics and no histogram, so heavily skewed key distributions cost nothing extra.
// Thread t holds EPT keys; unused slots must hold 0 and real keys must be > 0.  `tmp` holds 64 ints.
template <int EPT>
__device__ __forceinline__ uint32_t block_kth_largest(const uint32_t (&keys)[EPT], int need, int* tmp) {
  uint32_t thr = 0;
  int parity = 0;
  __syncthreads();
  for (int bit = 31; bit >= 0; --bit) {
    const uint32_t cand = thr | (1u << bit);
    int c = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) c += keys[j] >= cand ? 1 : 0;
    if (block_sum_1bar(c, tmp, parity) >= need) thr = cand;
  }
  __syncthreads();
  return thr;
}

// Same search with the keys produced on the fly by `key_of(j)` (j = 0..EPT-1), for callers short of registers.
template <int EPT, typename F>
__device__ __forceinline__ uint32_t block_kth_largest_fn(F key_of, int need, int* tmp) {
  uint32_t thr = 0;
  int parity = 0;
  __syncthreads();
  for (int bit = 31; bit >= 0; --bit) {
    const uint32_t cand = thr | (1u << bit);
    int c = 0;
#pragma unroll
    for (int j = 0; j < EPT; ++j) c += key_of(j) >= cand ? 1 : 0;
    if (block_sum_1bar(c, tmp, parity) >= need) thr = cand;
  }
  __syncthreads();
  return thr;
}

}  // namespace aspa
