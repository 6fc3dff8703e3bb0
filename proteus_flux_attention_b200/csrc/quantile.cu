// Per-head quantile of |x| for the percentile modes of the INT8 quantiser (reference models/aspa.py:1330-1338:
// torch.quantile(abs_flat, percentile, dim=1) with its default linear interpolation, replaced by the maximum where
// the quantile is zero).
//
// The two order statistics a linear quantile needs are found exactly with a most-significant-byte-first radix
// select over the bit patterns of |x| (non-negative floats order like their unsigned bit patterns): four passes, each
// a histogram of one byte over the elements that still match the prefix found so far, followed by a one-block-per-head
// pick of the bucket that holds the wanted rank.  No sort, no atomics on the data, 1 KB of histogram per head.
#include <algorithm>

#include "common.cuh"

namespace aspa {

template <typename T>
__device__ __forceinline__ uint32_t abs_bits(const T* p, int64_t i);
template <>
__device__ __forceinline__ uint32_t abs_bits<float>(const float* p, int64_t i) { return __float_as_uint(p[i]) & 0x7fffffffu; }
template <>
__device__ __forceinline__ uint32_t abs_bits<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) {
  return ((uint32_t)reinterpret_cast<const unsigned short*>(p)[i] << 16) & 0x7fffffffu;
}

// hist[(head * 2 + which) * 256 + byte]: `which` selects the lower / upper order statistic (their prefixes may differ)
template <typename T>
__global__ void __launch_bounds__(256) quantile_hist_kernel(const T* __restrict__ x, int64_t per_head, int shift,
                                                            const uint32_t* __restrict__ prefix, int n_which,
                                                            unsigned int* __restrict__ hist) {
  __shared__ unsigned int h[2][256];
  const int head = blockIdx.y;
  h[0][threadIdx.x] = h[1][threadIdx.x] = 0u;
  __syncthreads();
  const uint32_t p0 = prefix[head * 2], p1 = prefix[head * 2 + 1];
  const uint32_t hi_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
  const bool same = n_which == 1 || (p0 & hi_mask) == (p1 & hi_mask);
  const T* xh = x + (int64_t)head * per_head;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_head; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t u = abs_bits<T>(xh, i);
    if ((u & hi_mask) == (p0 & hi_mask)) atomicAdd(&h[0][(u >> shift) & 255u], 1u);
    if (!same && (u & hi_mask) == (p1 & hi_mask)) atomicAdd(&h[1][(u >> shift) & 255u], 1u);
  }
  __syncthreads();
  const unsigned int c0 = h[0][threadIdx.x];
  if (c0) atomicAdd(&hist[(head * 2) * 256 + threadIdx.x], c0);
  if (n_which == 2) {
    const unsigned int c1 = same ? c0 : h[1][threadIdx.x];
    if (c1) atomicAdd(&hist[(head * 2 + 1) * 256 + threadIdx.x], c1);
  }
}

// One block of 256 threads per (head, which): find the bucket holding the wanted 0-based ascending rank, extend the
// prefix by it, reduce the rank to the rank inside the bucket, clear the histogram for the next pass.
__global__ void __launch_bounds__(256) quantile_pick_kernel(unsigned int* __restrict__ hist, int shift,
                                                            uint32_t* __restrict__ prefix, long long* __restrict__ rank) {
  __shared__ int tmp[33];
  const int slot = blockIdx.x;   // head * 2 + which
  const int c = (int)hist[slot * 256 + threadIdx.x];
  int total;
  const int before = block_exclusive_scan(c, tmp, &total);
  const long long r = rank[slot];
  __syncthreads();
  if (c > 0 && r >= before && r < (long long)before + c) {
    prefix[slot] |= (uint32_t)threadIdx.x << shift;
    rank[slot] = r - before;
  }
  hist[slot * 256 + threadIdx.x] = 0u;
}

__global__ void quantile_init_kernel(uint32_t* prefix, long long* rank, unsigned int* hist, int heads, long long lower,
                                     long long upper) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < heads * 2) {
    prefix[i] = 0u;
    rank[i] = (i & 1) ? upper : lower;
  }
  if (i < heads * 2 * 256) hist[i] = 0u;
}

// base = lerp(lower value, upper value, weight) with torch's formula; the maximum where that is not positive
__global__ void quantile_finish_kernel(const uint32_t* __restrict__ prefix, int heads, float weight, int n_which,
                                       const float* __restrict__ amax, float* __restrict__ base) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= heads) return;
  const float a = __uint_as_float(prefix[h * 2]);
  const float b = n_which == 2 ? __uint_as_float(prefix[h * 2 + 1]) : a;
  const float diff = __fsub_rn(b, a);
  const float v = weight < 0.5f ? __fadd_rn(a, __fmul_rn(weight, diff)) : __fsub_rn(b, __fmul_rn(diff, __fsub_rn(1.f, weight)));
  base[h] = v > 0.f ? v : amax[h];
}

}  // namespace aspa

using namespace aspa;

extern "C" int64_t aspa_head_abs_quantile_scratch(int heads) {
  return (int64_t)heads * 2 * (256 * sizeof(unsigned int) + sizeof(uint32_t) + sizeof(long long)) + 64;
}

extern "C" int aspa_head_abs_quantile(const void* x, int dtype, int heads, int64_t per_head, double q, const float* amax,
                                      void* scratch, float* base, void* stream) {
  ASPA_CHECK_ARG(x && amax && scratch && base, "null pointer");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "x must be float32 or bfloat16");
  ASPA_CHECK_ARG(heads > 0 && per_head > 0 && q > 0.0 && q <= 1.0, "need heads > 0, elements > 0 and 0 < q <= 1");
  cudaStream_t st = (cudaStream_t)stream;
  // torch.quantile: ranks = q * (n - 1) in the tensor's own type (float32), floor / ceil / fractional weight
  const float rank_f = (float)q * (float)(per_head - 1);
  const long long lower = (long long)floorf(rank_f), upper = (long long)ceilf(rank_f);
  const float weight = rank_f - (float)lower;
  const int n_which = upper != lower ? 2 : 1;
  long long* rank = reinterpret_cast<long long*>(scratch);
  uint32_t* prefix = reinterpret_cast<uint32_t*>(rank + heads * 2);
  unsigned int* hist = reinterpret_cast<unsigned int*>(prefix + heads * 2);
  quantile_init_kernel<<<(unsigned)ceil_div((int64_t)heads * 2 * 256, 256), 256, 0, st>>>(prefix, rank, hist, heads, lower,
                                                                                         std::min(upper, (long long)per_head - 1));
  ASPA_CHECK_LAUNCH();
  const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(per_head, 256 * 16), 1024));
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (dtype == ASPA_F32)
      quantile_hist_kernel<float><<<dim3(blocks, heads), 256, 0, st>>>((const float*)x, per_head, shift, prefix, n_which, hist);
    else
      quantile_hist_kernel<__nv_bfloat16><<<dim3(blocks, heads), 256, 0, st>>>((const __nv_bfloat16*)x, per_head, shift, prefix,
                                                                                n_which, hist);
    ASPA_CHECK_LAUNCH();
    quantile_pick_kernel<<<heads * 2, 256, 0, st>>>(hist, shift, prefix, rank);
    ASPA_CHECK_LAUNCH();
  }
  quantile_finish_kernel<<<(unsigned)ceil_div(heads, 128), 128, 0, st>>>(prefix, heads, weight, n_which, amax, base);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
