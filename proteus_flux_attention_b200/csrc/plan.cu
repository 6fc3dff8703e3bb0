// Shortlist planning: block-wise prefix top-k of prototype scores, and the explicit (N, L) candidate
// table for callers of the functional API.
#include <utility>

#include "common.cuh"

namespace aspa {

constexpr int PLAN_BLOCK = 128;

// In-place bitonic sort (ascending) of n = power-of-two 64-bit keys in shared memory.
__device__ void bitonic_sort_u64(unsigned long long* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const unsigned long long x = a[i], y = a[ixj];
          const bool up = (i & k) == 0;
          if ((x > y) == up) {
            a[i] = y;
            a[ixj] = x;
          }
        }
      }
      __syncthreads();
    }
  }
}

__device__ void bitonic_sort_i32(int* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const int x = a[i], y = a[ixj];
          const bool up = (i & k) == 0;
          if ((x > y) == up) {
            a[i] = y;
            a[ixj] = x;
          }
        }
      }
      __syncthreads();
    }
  }
}

// Radix select over scores[0..n): key of the need-th largest and how many ties to accept.
__device__ void prefix_select(const float* __restrict__ scores, int n, int need, int* hist, int* sh,
                              uint32_t* thr_key, int* take_ties) {
  uint32_t prefix = 0, mask = 0;
  int remaining = need;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t k = float_key(scores[i]);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, b = 255;
      for (; b > 0; --b) {
        if (acc + hist[b] >= remaining) break;
        acc += hist[b];
      }
      sh[0] = b;
      sh[1] = remaining - acc;
    }
    __syncthreads();
    prefix |= ((uint32_t)sh[0]) << shift;
    mask |= 255u << shift;
    remaining = sh[1];
    __syncthreads();
  }
  *thr_key = prefix;
  *take_ties = remaining;
}

// Collect the `need` best entries of scores[0..n) (ties: lowest index) as 64-bit sort keys
// (~score_key << 32 | index) appended at dst[*fill ...].  Block-wide; `fill` lives in shared memory.
__device__ void collect_top(const float* __restrict__ scores, int n, int need, int* hist, int* sh, int* scan_tmp,
                            unsigned long long* dst, int* fill) {
  if (need <= 0 || n <= 0) return;
  if (need >= n) {
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      dst[*fill + i] = ((unsigned long long)(~float_key(scores[i])) << 32) | (unsigned)i;
    __syncthreads();
    if (threadIdx.x == 0) *fill += n;
    __syncthreads();
    return;
  }
  uint32_t thr;
  int take;
  prefix_select(scores, n, need, hist, sh, &thr, &take);
  int ties_seen = 0;
  const int base_fill = *fill;
  int written = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    uint32_t k = 0;
    bool gt = false, tie = false;
    if (i < n) {
      k = float_key(scores[i]);
      gt = k > thr;
      tie = k == thr;
    }
    int tot_t;
    const int rank_t = block_exclusive_scan(tie ? 1 : 0, scan_tmp, &tot_t);
    const bool on = gt || (tie && ties_seen + rank_t < take);
    int tot_o;
    const int pos = block_exclusive_scan(on ? 1 : 0, scan_tmp, &tot_o);
    if (on) dst[base_fill + written + pos] = ((unsigned long long)(~k) << 32) | (unsigned)i;
    written += tot_o;
    ties_seen += tot_t;
  }
  __syncthreads();
  if (threadIdx.x == 0) *fill = base_fill + written;
  __syncthreads();
}

// One CTA per (batch, 128-token block).
__global__ void __launch_bounds__(256) proto_plan_kernel(const float* __restrict__ proto_scores, int T, int cap,
                                                         int list_stride, int32_t* __restrict__ lists,
                                                         int32_t* __restrict__ limits) {
  extern __shared__ unsigned long long keys[];  // [P2]
  __shared__ int hist[256];
  __shared__ int sh[4];
  __shared__ int scan_tmp[33];
  __shared__ int fill;
  const int blk = blockIdx.x, b = blockIdx.y;
  const int nblk = gridDim.x;
  const float* sc = proto_scores + (int64_t)b * T;
  const int t0 = blk * PLAN_BLOCK;
  const int nb = min(PLAN_BLOCK, T - t0);
  int P2 = 1;
  while (P2 < cap + PLAN_BLOCK) P2 <<= 1;
  for (int i = threadIdx.x; i < P2; i += blockDim.x) keys[i] = ~0ull;
  if (threadIdx.x == 0) fill = 0;
  __syncthreads();
  collect_top(sc, t0, min(cap, t0), hist, sh, scan_tmp, keys, &fill);
  const int nprefix = fill;
  for (int i = threadIdx.x; i < nb; i += blockDim.x)
    keys[nprefix + i] = ((unsigned long long)(~float_key(sc[t0 + i])) << 32) | (unsigned)(t0 + i);
  __syncthreads();
  const int total = nprefix + nb;
  bitonic_sort_u64(keys, P2);
  int32_t* out = lists + ((int64_t)b * nblk + blk) * list_stride;
  for (int i = threadIdx.x; i < list_stride; i += blockDim.x)
    out[i] = i < total ? (int32_t)(keys[i] & 0xffffffffu) : -1;
  // per token: how many leading list entries hold its min(t+1, cap) picks
  if ((int)threadIdx.x < nb) {
    const int t = t0 + threadIdx.x;
    const int want = min(t + 1, cap);
    int have = 0, pos = 0;
    while (pos < total && have < want) {
      const int idx = (int)(keys[pos] & 0xffffffffu);
      if (idx <= t) ++have;
      ++pos;
    }
    limits[(int64_t)b * T + t] = pos;
  }
}

// ------------------------------------------------------------------------------------------------
// Hierarchical plan (prototype cap <= PLAN_FAST_CAP): the prefix top-k of a block is assembled from
//   A. the sorted top-cap list of every 1024-token super-block (its own tokens only),
//   B. an inclusive scan of those lists with "top-cap of the union" as the (associative) operator,
//   C. per block: top-cap of [scanned list of the super-blocks before mine] U [tokens of my super-block before me],
// so a block looks at about cap + 1024 scores instead of its whole prefix.  Same lists, same limits as
// proto_plan_kernel (the order (score desc, index asc) is total, so every top-cap set is unique).
// ------------------------------------------------------------------------------------------------
constexpr int PLAN_SB = 1024;          // tokens per super-block (8 blocks)
constexpr int PLAN_FAST_CAP = 960;     // 2 * cap and cap + PLAN_SB must fit a 2048-entry sort

__device__ __forceinline__ unsigned long long plan_key(float score, int idx) {
  return ((unsigned long long)(~float_key(score)) << 32) | (unsigned)idx;
}

// A: grid (nsb, B).  lists_out[(b*nsb + s) * cap + i]: sorted keys of super-block s, ~0 padded.
__global__ void __launch_bounds__(256) plan_superblock_kernel(const float* __restrict__ proto_scores, int T, int cap,
                                                              unsigned long long* __restrict__ lists_out) {
  __shared__ unsigned long long keys[PLAN_SB];
  const int s = blockIdx.x, b = blockIdx.y, nsb = gridDim.x;
  const float* sc = proto_scores + (int64_t)b * T;
  const int t0 = s * PLAN_SB;
  for (int i = threadIdx.x; i < PLAN_SB; i += blockDim.x) keys[i] = t0 + i < T ? plan_key(sc[t0 + i], t0 + i) : ~0ull;
  __syncthreads();
  bitonic_sort_u64(keys, PLAN_SB);
  unsigned long long* out = lists_out + ((int64_t)b * nsb + s) * cap;
  for (int i = threadIdx.x; i < cap; i += blockDim.x) out[i] = i < PLAN_SB ? keys[i] : ~0ull;
}

// B: one Hillis-Steele level.  out[s] = top-cap(in[s] U in[s - d]) for s >= d, else in[s].  grid (nsb, B).
__global__ void __launch_bounds__(256) plan_scan_level_kernel(const unsigned long long* __restrict__ in, int cap, int d,
                                                              unsigned long long* __restrict__ out) {
  __shared__ unsigned long long keys[2048];
  const int s = blockIdx.x, b = blockIdx.y, nsb = gridDim.x;
  const unsigned long long* a = in + ((int64_t)b * nsb + s) * cap;
  unsigned long long* o = out + ((int64_t)b * nsb + s) * cap;
  if (s < d) {
    for (int i = threadIdx.x; i < cap; i += blockDim.x) o[i] = a[i];
    return;
  }
  const unsigned long long* c = in + ((int64_t)b * nsb + s - d) * cap;
  int P2 = 2;
  while (P2 < 2 * cap) P2 <<= 1;
  for (int i = threadIdx.x; i < P2; i += blockDim.x) keys[i] = i < cap ? a[i] : (i < 2 * cap ? c[i - cap] : ~0ull);
  __syncthreads();
  bitonic_sort_u64(keys, P2);
  for (int i = threadIdx.x; i < cap; i += blockDim.x) o[i] = keys[i];
}

// C: grid (nblk, B).  `scanned` holds the inclusive scan of the super-block lists.
__global__ void __launch_bounds__(256) plan_block_kernel(const float* __restrict__ proto_scores, int T, int cap,
                                                         const unsigned long long* __restrict__ scanned, int nsb,
                                                         int list_stride, int32_t* __restrict__ lists,
                                                         int32_t* __restrict__ limits) {
  __shared__ unsigned long long keys[2048];
  const int blk = blockIdx.x, b = blockIdx.y, nblk = gridDim.x;
  const float* sc = proto_scores + (int64_t)b * T;
  const int t0 = blk * PLAN_BLOCK;
  const int nb = min(PLAN_BLOCK, T - t0);
  const int s = t0 / PLAN_SB, sb0 = s * PLAN_SB;
  // candidates of the prefix [0, t0): everything kept from earlier super-blocks + my super-block up to t0
  const unsigned long long* prev = s > 0 ? scanned + ((int64_t)b * nsb + s - 1) * cap : nullptr;
  const int n_prev = prev ? cap : 0, n_mine = t0 - sb0;
  int P2 = 2;
  while (P2 < n_prev + n_mine) P2 <<= 1;
  for (int i = threadIdx.x; i < P2; i += blockDim.x) {
    unsigned long long k = ~0ull;
    if (i < n_prev) k = prev[i];
    else if (i < n_prev + n_mine) k = plan_key(sc[sb0 + i - n_prev], sb0 + i - n_prev);
    keys[i] = k;
  }
  __syncthreads();
  if (n_prev + n_mine > 1) bitonic_sort_u64(keys, P2);
  // keep min(cap, t0) of them (pads sort last; real keys are fewer than that only when t0 < cap), add my tokens
  const int nprefix = min(cap, t0);
  __syncthreads();
  int Q2 = 1;
  while (Q2 < cap + PLAN_BLOCK) Q2 <<= 1;
  for (int i = threadIdx.x; i < Q2; i += blockDim.x) {
    if (i >= nprefix) keys[i] = (i - nprefix) < nb ? plan_key(sc[t0 + i - nprefix], t0 + i - nprefix) : ~0ull;
  }
  __syncthreads();
  const int total = nprefix + nb;
  bitonic_sort_u64(keys, Q2);
  int32_t* out = lists + ((int64_t)b * nblk + blk) * list_stride;
  for (int i = threadIdx.x; i < list_stride; i += blockDim.x)
    out[i] = i < total ? (int32_t)(keys[i] & 0xffffffffu) : -1;
  if ((int)threadIdx.x < nb) {
    const int t = t0 + threadIdx.x;
    const int want = min(t + 1, cap);
    int have = 0, pos = 0;
    while (pos < total && have < want) {
      const int idx = (int)(keys[pos] & 0xffffffffu);
      if (idx <= t) ++have;
      ++pos;
    }
    limits[(int64_t)b * T + t] = pos;
  }
}

// Explicit candidate table: one CTA per row.
__global__ void __launch_bounds__(256) build_candidates_kernel(
    const int64_t* __restrict__ rows, const int64_t* __restrict__ row_batch, int seq_len, int L, int w_local,
    int slots, int stride, const float* __restrict__ proto_scores, int pcap, int P2,
    int64_t* __restrict__ cand_out, int64_t* __restrict__ len_out) {
  extern __shared__ unsigned long long dyn[];
  int* buf = reinterpret_cast<int*>(dyn);                                         // [P2] candidate ids
  unsigned long long* pk = dyn + (P2 + 1) / 2;                                    // [pcap] prototype picks
  __shared__ int hist[256];
  __shared__ int sh[4];
  __shared__ int scan_tmp[33];
  __shared__ int fill;
  const int64_t r = blockIdx.x;
  const int t = (int)rows[r];
  const int hi = max(seq_len - 1, 0);
  for (int i = threadIdx.x; i < P2; i += blockDim.x) buf[i] = 0x7fffffff;
  if (threadIdx.x == 0) fill = 0;
  __syncthreads();
  int n = 0;
  if (w_local > 0) {
    const int ln = min(t + 1, w_local);
    const int st = max(t - ln + 1, 0);
    for (int s = threadIdx.x; s < w_local; s += blockDim.x) buf[n + s] = s < ln ? st + s : t;
    n += w_local;
  }
  if (slots > 0) {
    for (int j = threadIdx.x; j < slots; j += blockDim.x) {
      const long long a = (long long)t - (long long)(j + 1) * stride;
      buf[n + j] = (int)max(a, 0LL);
    }
    n += slots;
  }
  __syncthreads();
  if (proto_scores != nullptr && pcap > 0) {
    const int b = row_batch ? (int)row_batch[r] : 0;
    const float* sc = proto_scores + (int64_t)b * seq_len;
    const int upto = min(t + 1, seq_len);
    collect_top(sc, upto, min(pcap, upto), hist, sh, scan_tmp, pk, &fill);
    const int got = fill;
    for (int i = threadIdx.x; i < pcap; i += blockDim.x) buf[n + i] = i < got ? (int)(pk[i] & 0xffffffffu) : t;
    n += pcap;
  }
  __syncthreads();
  // clamp to [0, seq_len-1], then to <= t; the row itself is appended afterwards, unclamped (sa.py:570-572)
  for (int i = threadIdx.x; i < n; i += blockDim.x) buf[i] = min(min(max(buf[i], 0), hi), t);
  if (threadIdx.x == 0) buf[n] = t;
  n += 1;
  __syncthreads();
  bitonic_sort_i32(buf, P2);
  // unique + first L
  int64_t* out = cand_out + r * L;
  for (int i = threadIdx.x; i < L; i += blockDim.x) out[i] = t;
  __syncthreads();
  int running = 0;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const bool first = i < n && (i == 0 || buf[i] != buf[i - 1]);
    int tot;
    const int pos = block_exclusive_scan(first ? 1 : 0, scan_tmp, &tot);
    if (first && running + pos < L) out[running + pos] = buf[i];
    running += tot;
  }
  if (threadIdx.x == 0) len_out[r] = max(1, min(running, L));
}

}  // namespace aspa

using namespace aspa;

extern "C" int64_t aspa_proto_plan_scratch(int B, int T, int proto_cap) {
  if (proto_cap <= 0 || proto_cap > PLAN_FAST_CAP || T <= 2 * PLAN_SB) return 16;  // the one-kernel plan needs none
  const int64_t nsb = ceil_div(T, PLAN_SB);
  return 2 * (int64_t)B * nsb * proto_cap * (int64_t)sizeof(unsigned long long);   // two scan buffers
}

extern "C" int aspa_proto_plan(const float* proto_scores, int B, int T, int proto_cap, void* scratch,
                               int32_t* proto_lists, int32_t* proto_limit, void* stream) {
  ASPA_CHECK_ARG(proto_scores && proto_lists && proto_limit, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && proto_cap > 0, "bad sizes");
  cudaStream_t st = (cudaStream_t)stream;
  if (proto_cap <= PLAN_FAST_CAP && T > 2 * PLAN_SB) {
    ASPA_CHECK_ARG(scratch != nullptr, "scratch of aspa_proto_plan_scratch() bytes required");
    const int nsb = (int)ceil_div(T, PLAN_SB), nblk = (int)ceil_div(T, PLAN_BLOCK);
    unsigned long long* buf0 = reinterpret_cast<unsigned long long*>(scratch);
    unsigned long long* buf1 = buf0 + (int64_t)B * nsb * proto_cap;
    plan_superblock_kernel<<<dim3(nsb, B), 256, 0, st>>>(proto_scores, T, proto_cap, buf0);
    unsigned long long *in = buf0, *out = buf1;
    for (int d = 1; d < nsb; d <<= 1) {
      plan_scan_level_kernel<<<dim3(nsb, B), 256, 0, st>>>(in, proto_cap, d, out);
      std::swap(in, out);
    }
    plan_block_kernel<<<dim3(nblk, B), 256, 0, st>>>(proto_scores, T, proto_cap, in, nsb, proto_cap + PLAN_BLOCK,
                                                     proto_lists, proto_limit);
    ASPA_CHECK_LAUNCH();
    return ASPA_OK;
  }
  int P2 = 1;
  while (P2 < proto_cap + PLAN_BLOCK) P2 <<= 1;
  const size_t smem = sizeof(unsigned long long) * P2;
  ASPA_CHECK_ARG(smem <= 200 * 1024, "proto_cap too large for the planning kernel (max ~ 25000)");
  cudaFuncSetAttribute(proto_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const dim3 grid((unsigned)ceil_div(T, PLAN_BLOCK), B);
  proto_plan_kernel<<<grid, 256, smem, st>>>(proto_scores, T, proto_cap, proto_cap + PLAN_BLOCK, proto_lists, proto_limit);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_build_candidates(const int64_t* rows, const int64_t* row_batch, int64_t N, int seq_len, int L,
                                     int linear_window, int anchor_stride, int use_local, int use_anchors,
                                     const float* proto_scores, int local_cap, int anchor_cap, int proto_cap,
                                     int64_t* cand_out, int64_t* len_out, void* stream) {
  ASPA_CHECK_ARG(rows && cand_out && len_out, "null pointer");
  ASPA_CHECK_ARG(N >= 0 && L > 0 && seq_len >= 0, "bad sizes");
  if (N == 0) return ASPA_OK;
  // None-caps of the reference (sa.py:490-504)
  const int lc = local_cap >= 0 ? local_cap : (use_local ? L : 0);
  const int ac = anchor_cap >= 0 ? anchor_cap : (use_anchors ? L : 0);
  const int pc = proto_cap >= 0 ? proto_cap : (proto_scores ? L : 0);
  int w_local = 0, slots = 0, pcap = 0;
  if (use_local && lc > 0) w_local = std::max(0, std::min(std::min(linear_window, L), lc));
  if (use_anchors && anchor_stride > 0 && ac > 0) slots = std::min(std::min(ac, L), std::max(1, seq_len));
  if (proto_scores && pc > 0) pcap = std::max(0, std::min(std::min(L, pc), seq_len));
  const int n = w_local + slots + pcap + 1;
  int P2 = 2;
  while (P2 < n) P2 <<= 1;
  const size_t smem = sizeof(unsigned long long) * ((P2 + 1) / 2 + pcap + 1);
  ASPA_CHECK_ARG(smem <= 200 * 1024, "candidate width too large for the table builder");
  cudaFuncSetAttribute(build_candidates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  build_candidates_kernel<<<(unsigned)N, 256, smem, (cudaStream_t)stream>>>(
      rows, row_batch, seq_len, L, w_local, slots, anchor_stride, pcap > 0 ? proto_scores : nullptr, pcap, P2,
      cand_out, len_out);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
