// Selection across a thread-block cluster: the keys of one row are spread over the registers of up to 8 CTAs
// (8 SMs), and counts travel between the CTAs through distributed shared memory.  One row of 65536 keys would
// fill the whole register file of a single SM; spread over a cluster every thread holds 8 keys.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace aspa {

namespace cg = cooperative_groups;

constexpr int CL_MAX = 8;      // portable cluster size limit
constexpr int CL_EPT = 8;      // keys per thread
constexpr int CL_THREADS = 1024;
constexpr int CL_KEYS_PER_CTA = CL_EPT * CL_THREADS;

// Shared scratch of one CTA for the cluster reductions below.
struct ClusterScratch {
  uint32_t warp_slots[32 * 4];
  uint32_t cta_slots[2][CL_MAX * 4];  // [parity][rank * NV + k], written by every CTA of the cluster
  int scan_tmp[33];
};

struct OpAdd {
  static __device__ __forceinline__ uint32_t warp(uint32_t v) { return __reduce_add_sync(0xffffffffu, v); }
  static __device__ __forceinline__ uint32_t join(uint32_t a, uint32_t b) { return a + b; }
  static constexpr uint32_t identity = 0u;
};
struct OpMax {
  static __device__ __forceinline__ uint32_t warp(uint32_t v) { return __reduce_max_sync(0xffffffffu, v); }
  static __device__ __forceinline__ uint32_t join(uint32_t a, uint32_t b) { return a > b ? a : b; }
  static constexpr uint32_t identity = 0u;
};

// Reduce NV (<= 4) unsigned values per thread over every thread of the cluster; all threads get the results in v.
// `below` (optional) receives the reduction over the CTAs of lower rank only (an exclusive prefix by rank).
// Cost: one CTA barrier and one cluster barrier.  `parity` is a caller register, uniform over the cluster.
template <int NV, typename Op>
__device__ __forceinline__ void cluster_reduce(uint32_t (&v)[NV], ClusterScratch& s, int& parity,
                                               uint32_t* below = nullptr) {
  cg::cluster_group cluster = cg::this_cluster();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int rank = (int)cluster.block_rank(), csize = (int)cluster.num_blocks();
#pragma unroll
  for (int k = 0; k < NV; ++k) v[k] = Op::warp(v[k]);
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < NV; ++k) s.warp_slots[warp * NV + k] = v[k];
  }
  __syncthreads();
  if (warp == 0) {
    uint32_t t[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) t[k] = Op::warp(lane < nwarp ? s.warp_slots[lane * NV + k] : Op::identity);
    if (lane < csize) {
      uint32_t* remote = cluster.map_shared_rank(&s.cta_slots[parity][rank * NV], lane);
#pragma unroll
      for (int k = 0; k < NV; ++k) remote[k] = t[k];
    }
  }
  cluster.sync();
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    uint32_t acc = Op::identity, lo = Op::identity;
    for (int r = 0; r < csize; ++r) {
      if (r == rank) lo = acc;
      acc = Op::join(acc, s.cta_slots[parity][r * NV + k]);
    }
    v[k] = acc;
    if (below) below[k] = lo;
  }
  parity ^= 1;
}

// Sum of one float per thread over the cluster, accumulated in a fixed order (warps, then ranks).
__device__ __forceinline__ float cluster_sum_float(float x, ClusterScratch& s, int& parity) {
  cg::cluster_group cluster = cg::this_cluster();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int rank = (int)cluster.block_rank(), csize = (int)cluster.num_blocks();
  x = warp_sum(x);
  if (lane == 0) s.warp_slots[warp] = __float_as_uint(x);
  __syncthreads();
  if (warp == 0) {
    float t = warp_sum(lane < nwarp ? __uint_as_float(s.warp_slots[lane]) : 0.f);
    if (lane < csize) *cluster.map_shared_rank(&s.cta_slots[parity][rank], lane) = __float_as_uint(t);
  }
  cluster.sync();
  float acc = 0.f;
  for (int r = 0; r < csize; ++r) acc += __uint_as_float(s.cta_slots[parity][r]);
  parity ^= 1;
  return acc;
}

// The need-th largest (1-based) key of the cluster, two bits per round (three candidate thresholds counted at
// once): 16 rounds of one cluster barrier each.  Unused key slots must hold 0 and real keys must be > 0.
template <int EPT, typename F>
__device__ __forceinline__ uint32_t cluster_kth_largest_fn(F key_of, int need, ClusterScratch& s, int& parity) {
  uint32_t thr = 0;
  for (int bit = 30; bit >= 0; bit -= 2) {
    const uint32_t c1 = thr | (1u << bit), c2 = thr | (2u << bit), c3 = thr | (3u << bit);
    uint32_t v[3] = {0u, 0u, 0u};
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
      const uint32_t k = key_of(j);
      v[0] += k >= c1 ? 1u : 0u;
      v[1] += k >= c2 ? 1u : 0u;
      v[2] += k >= c3 ? 1u : 0u;
    }
    cluster_reduce<3, OpAdd>(v, s, parity);
    if ((int)v[2] >= need) thr = c3;
    else if ((int)v[1] >= need) thr = c2;
    else if ((int)v[0] >= need) thr = c1;
  }
  return thr;
}

template <int EPT>
__device__ __forceinline__ uint32_t cluster_kth_largest(const uint32_t (&keys)[EPT], int need, ClusterScratch& s,
                                                        int& parity) {
  return cluster_kth_largest_fn<EPT>([&](int j) { return keys[j]; }, need, s, parity);
}

// Launch `kernel` with clusters of `csize` CTAs of CL_THREADS threads; `rows` clusters in all.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_clusters(void (*kernel)(KArgs...), int rows, int csize, size_t smem,
                                          cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * csize));
  cfg.blockDim = dim3(CL_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace aspa
