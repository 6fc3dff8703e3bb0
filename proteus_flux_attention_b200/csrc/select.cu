// Token keep (radix select), head budget, per-token head top-k and row packing.
#include <algorithm>
#include <mutex>

#include "cluster.cuh"
#include "common.cuh"

namespace aspa {

// ---------------------------------------------------------------------------------------------
// Radix select helper: one CTA finds the key of rank `need` (1-based, descending) among `n` floats
// and how many entries equal to it must still be taken.  Keys stream from global/L2 once per pass.
// ---------------------------------------------------------------------------------------------
struct SelectResult {
  uint32_t thr_key;  // key of the need-th largest element
  int take_ties;     // number of entries == thr_key to accept (lowest indices first)
};

template <typename KeyFn>
__device__ SelectResult block_radix_select(int n, int need, KeyFn key_of, int* hist /*256*/, int* sh /*4*/) {
  uint32_t prefix = 0, mask = 0;
  int remaining = need;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t k = key_of(i);
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
  SelectResult r;
  r.thr_key = prefix;
  r.take_ties = remaining;
  return r;
}

__global__ void __launch_bounds__(1024) token_select_kernel(const float* __restrict__ importance, int T, int need0,
                                                            float threshold, int guard,
                                                            uint8_t* __restrict__ token_mask,
                                                            int32_t* __restrict__ kept) {
  __shared__ int hist[256];
  __shared__ int sh[4];
  __shared__ int scan_tmp[33];
  const float* imp = importance + (int64_t)blockIdx.x * T;
  uint8_t* out = token_mask + (int64_t)blockIdx.x * T;
  int need = need0;
  if (threshold > 0.f) {
    int c = 0;
    for (int i = threadIdx.x; i < T; i += blockDim.x) c += imp[i] >= threshold ? 1 : 0;
    int tot;
    block_exclusive_scan(c, scan_tmp, &tot);
    need = max(need, tot);
  }
  need = max(need, guard);
  need = min(max(1, need), T);
  if (need >= T) {
    for (int i = threadIdx.x; i < T; i += blockDim.x) out[i] = 1;
    if (threadIdx.x == 0) kept[blockIdx.x] = T;
    return;
  }
  auto key_of = [imp](int i) { return float_key(imp[i]); };
  const SelectResult sel = block_radix_select(T, need, key_of, hist, sh);
  int ties_seen = 0, kept_total = 0;
  for (int base = 0; base < T; base += blockDim.x) {
    const int i = base + threadIdx.x;
    uint32_t k = 0;
    bool tie = false, gt = false;
    if (i < T) {
      k = float_key(imp[i]);
      gt = k > sel.thr_key;
      tie = k == sel.thr_key;
    }
    int tot;
    const int rank = block_exclusive_scan(tie ? 1 : 0, scan_tmp, &tot);
    if (i < T) {
      bool on = gt || (tie && (ties_seen + rank) < sel.take_ties);
      if (threshold > 0.f && imp[i] >= threshold) on = true;
      if (i < guard) on = true;
      out[i] = on ? 1 : 0;
      kept_total += on ? 1 : 0;
    }
    ties_seen += tot;
  }
  int tot;
  block_exclusive_scan(kept_total, scan_tmp, &tot);
  if (threadIdx.x == 0) kept[blockIdx.x] = tot;
}

// Token keep with every key of the batch row held in registers (T <= 1024 * EPT).  Thread t owns the EPT
// consecutive tokens [t*EPT, (t+1)*EPT): index order is thread order, so ranking tied keys by index takes one
// block scan.  One pass over HBM, then the threshold search and the marking run out of registers.
template <int EPT>
__global__ void __launch_bounds__(1024) token_select_regs_kernel(const float* __restrict__ importance, int T,
                                                                 int need0, float threshold, int guard,
                                                                 uint8_t* __restrict__ token_mask,
                                                                 int32_t* __restrict__ kept) {
  __shared__ int tmp[64];
  const float* imp = importance + (int64_t)blockIdx.x * T;
  uint8_t* out = token_mask + (int64_t)blockIdx.x * T;
  const int base = threadIdx.x * EPT;
  uint32_t keys[EPT];
  int above = 0;
  const bool vec_ok = (T % 4 == 0) && (EPT % 4 == 0);
#pragma unroll
  for (int j = 0; j < EPT; j += 4) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec_ok && base + j + 3 < T) {
      const float4 f = *reinterpret_cast<const float4*>(imp + base + j);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (base + j + e < T) v[e] = imp[base + j + e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const bool in = base + j + e < T;
      keys[j + e] = in ? max(float_key(v[e]), 1u) : 0u;
      above += (in && threshold > 0.f && v[e] >= threshold) ? 1 : 0;
    }
  }
  int need = need0;
  if (threshold > 0.f) need = max(need, block_sum_int(above, tmp));
  need = max(need, guard);
  need = min(max(1, need), T);
  if (need >= T) {
    for (int i = threadIdx.x; i < T; i += 1024) out[i] = 1;
    if (threadIdx.x == 0) kept[blockIdx.x] = T;
    return;
  }
  const uint32_t thr = block_kth_largest<EPT>(keys, need, tmp);
  int gt = 0, eq = 0;
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    gt += keys[j] > thr ? 1 : 0;
    eq += keys[j] == thr ? 1 : 0;
  }
  const int n_gt = block_sum_int(gt, tmp);
  const int take = need - n_gt;  // ties to accept, lowest token index first
  int n_eq;
  int tie_rank = block_exclusive_scan(eq, tmp, &n_eq);  // ties owned by lower threads = ties at lower indices
  int kept_total = 0;
  const float thr_f = threshold;
#pragma unroll
  for (int j = 0; j < EPT; j += 4) {
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = base + j + e;
      const uint32_t k = keys[j + e];
      bool on = k > thr;
      if (k == thr && k != 0) {
        on = tie_rank < take;
        ++tie_rank;
      }
      if (i < T) {
        if (thr_f > 0.f && key_float(k) >= thr_f) on = true;
        if (i < guard) on = true;
        kept_total += on ? 1 : 0;
        packed |= (on ? 1u : 0u) << (8 * e);
      }
    }
    if (base + j + 3 < T && (T % 4 == 0)) {
      *reinterpret_cast<uint32_t*>(out + base + j) = packed;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (base + j + e < T) out[base + j + e] = (uint8_t)((packed >> (8 * e)) & 1u);
    }
  }
  const int tot = block_sum_int(kept_total, tmp);
  if (threadIdx.x == 0) kept[blockIdx.x] = tot;
}

// Token keep with the row's keys spread over a cluster of CTAs (8 keys per thread, 8192 tokens per CTA, up to
// 8 CTAs): CTA r of the cluster owns tokens [r*8192, (r+1)*8192) and thread t of it the 8 consecutive tokens from
// r*8192 + t*8, so index order is (rank, thread, slot) order and tied keys rank by one scan.  grid = rows * csize.
template <int EPT>
__global__ void __launch_bounds__(CL_THREADS) token_select_cluster_kernel(const float* __restrict__ importance, int T,
                                                                          int need0, float threshold, int guard,
                                                                          uint8_t* __restrict__ token_mask,
                                                                          int32_t* __restrict__ kept,
                                                                          int64_t* __restrict__ kept_idx,
                                                                          int32_t* __restrict__ slot_of,
                                                                          int slots_per_row) {
  __shared__ ClusterScratch cs;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), csize = (int)cluster.num_blocks();
  const int row = blockIdx.x / csize;
  const float* imp = importance + (int64_t)row * T;
  uint8_t* out = token_mask + (int64_t)row * T;
  const int base = rank * (EPT * CL_THREADS) + threadIdx.x * EPT;
  int parity = 0;
  uint32_t keys[EPT];
  uint32_t above = 0;
  const bool vec_ok = (T % 4 == 0);
#pragma unroll
  for (int j = 0; j < EPT; j += 4) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec_ok && base + j + 3 < T) {
      const float4 f = *reinterpret_cast<const float4*>(imp + base + j);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (base + j + e < T) v[e] = imp[base + j + e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const bool in = base + j + e < T;
      keys[j + e] = in ? max(float_key(v[e]), 1u) : 0u;
      above += (in && threshold > 0.f && v[e] >= threshold) ? 1u : 0u;
    }
  }
  int need = need0;
  if (threshold > 0.f) {
    uint32_t a[1] = {above};
    cluster_reduce<1, OpAdd>(a, cs, parity);
    need = max(need, (int)a[0]);
  }
  need = max(need, guard);
  need = min(max(1, need), T);
  if (need >= T) {  // uniform over the cluster
#pragma unroll
    for (int j = 0; j < EPT; ++j)
      if (base + j < T) {
        out[base + j] = 1;
        if (kept_idx != nullptr) {
          if (base + j < slots_per_row) kept_idx[(int64_t)row * slots_per_row + base + j] = (int64_t)row * T + base + j;
          slot_of[(int64_t)row * T + base + j] = row * slots_per_row + base + j;
        }
      }
    if (kept_idx != nullptr)
      for (int i = T + rank * CL_THREADS + threadIdx.x; i < slots_per_row; i += csize * CL_THREADS)
        kept_idx[(int64_t)row * slots_per_row + i] = -1;
    if (rank == 0 && threadIdx.x == 0) kept[row] = T;
    return;
  }
  const uint32_t thr = cluster_kth_largest<EPT>(keys, need, cs, parity);
  uint32_t ge[2] = {0u, 0u}, lower[2];
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    ge[0] += keys[j] > thr ? 1u : 0u;
    ge[1] += keys[j] == thr ? 1u : 0u;
  }
  const int my_eq = (int)ge[1];
  cluster_reduce<2, OpAdd>(ge, cs, parity, lower);
  const int take = need - (int)ge[0];  // ties to accept, lowest token index first
  int n_eq;
  int tie_rank = (int)lower[1] + block_exclusive_scan(my_eq, cs.scan_tmp, &n_eq);
  uint32_t kept_total = 0, on_bits = 0;
#pragma unroll
  for (int j = 0; j < EPT; j += 4) {
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = base + j + e;
      const uint32_t k = keys[j + e];
      bool on = k > thr;
      if (k == thr && k != 0) {
        on = tie_rank < take;
        ++tie_rank;
      }
      if (i < T) {
        if (threshold > 0.f && key_float(k) >= threshold) on = true;
        if (i < guard) on = true;
        kept_total += on ? 1u : 0u;
        packed |= (on ? 1u : 0u) << (8 * e);
        on_bits |= (on ? 1u : 0u) << (j + e);
      }
    }
    if (vec_ok && base + j + 3 < T) {
      *reinterpret_cast<uint32_t*>(out + base + j) = packed;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (base + j + e < T) out[base + j + e] = (uint8_t)((packed >> (8 * e)) & 1u);
    }
  }
  int cta_total = 0;
  int slot = 0;
  if (kept_idx != nullptr) slot = block_exclusive_scan((int)kept_total, cs.scan_tmp, &cta_total);
  uint32_t kt[1] = {kept_total}, kt_lower[1];
  cluster_reduce<1, OpAdd>(kt, cs, parity, kt_lower);
  if (rank == 0 && threadIdx.x == 0) kept[row] = (int)kt[0];
  if (kept_idx != nullptr) {
    // ordered compaction of the kept tokens of this row: slots [row * slots_per_row, ...), padded with -1
    slot += (int)kt_lower[0];
    const int64_t s0 = (int64_t)row * slots_per_row;
#pragma unroll
    for (int j = 0; j < EPT; ++j)
      if ((on_bits >> j) & 1u) {
        if (slot < slots_per_row) kept_idx[s0 + slot] = (int64_t)row * T + base + j;
        slot_of[(int64_t)row * T + base + j] = (int)min(s0 + slot, (int64_t)0x7fffffff);
        ++slot;
      }
    for (int i = (int)kt[0] + rank * CL_THREADS + threadIdx.x; i < slots_per_row; i += csize * CL_THREADS)
      kept_idx[s0 + i] = -1;
  }
}

// ---------------------------------------------------------------------------------------------
// Head budget
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) head_colsum_kernel(const float* __restrict__ gate_probs, int64_t n, int G,
                                                          const int32_t* __restrict__ gate_to_head, int H,
                                                          float* __restrict__ partials /*[H][nblk]*/) {
  // block handles 1024 tokens; thread t sums gate column (t % G) over a strided subset, then shared tree per head
  const int64_t t0 = (int64_t)blockIdx.x * 1024;
  const int64_t t1 = min(n, t0 + 1024);
  const int lanes_per_tok = G;  // consecutive threads read consecutive gates of a token
  const int toks_per_iter = blockDim.x / lanes_per_tok;
  const int g = threadIdx.x % lanes_per_tok, sub = threadIdx.x / lanes_per_tok;
  float acc = 0.f;
  if (sub < toks_per_iter)
    for (int64_t t = t0 + sub; t < t1; t += toks_per_iter) acc += gate_probs[t * G + g];
  // deterministic: each (g, sub) writes its own slot, then one thread per head adds in fixed order
  __shared__ float slots[256];
  slots[threadIdx.x] = (sub < toks_per_iter) ? acc : 0.f;
  __syncthreads();
  if (threadIdx.x < H) {
    float s = 0.f;
    for (int gg = 0; gg < G; ++gg)
      if (gate_to_head[gg] == (int)threadIdx.x)
        for (int sb = 0; sb < toks_per_iter; ++sb) s += slots[sb * lanes_per_tok + gg];
    partials[(int64_t)threadIdx.x * gridDim.x + blockIdx.x] = s;
  }
}

__global__ void head_budget_kernel(const float* __restrict__ partials, int64_t nblk, int H, double n_tokens,
                                   double top_p, int dense_k, int h_active_min, int linear_head_k, double alpha,
                                   int32_t* __restrict__ k_out) {
  __shared__ float mean[64];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int h = w; h < H; h += (blockDim.x >> 5)) {
    float a = 0.f;
    for (int64_t i = lane; i < nblk; i += 32) a += partials[(int64_t)h * nblk + i];
    a = warp_sum(a);
    if (lane == 0) {
      float m = (float)((double)a / n_tokens);
      mean[h] = isfinite(m) ? m : 0.f;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int nucleus = 1;
    if (dense_k <= 1) {
      nucleus = max(1, dense_k);
    } else {
      float total = 0.f;
      for (int h = 0; h < H; ++h) total += mean[h];
      if (total > 0.f) {
        // selection sort descending (H <= 64)
        float v[64];
        for (int h = 0; h < H; ++h) v[h] = mean[h];
        for (int i = 0; i < H; ++i) {
          int b = i;
          for (int j = i + 1; j < H; ++j)
            if (v[j] > v[b]) b = j;
          float t = v[i];
          v[i] = v[b];
          v[b] = t;
        }
        const float target = (float)((double)total * top_p);  // double product, compared in fp32
        float c = 0.f;
        int keep = 0;
        for (int h = 0; h < H; ++h) {
          c += v[h];
          if (c < target) ++keep;
        }
        if (keep < H) ++keep;
        nucleus = min(dense_k, max(1, keep));
      }
    }
    const int adaptive = max(h_active_min, min(dense_k, nucleus));
    const int lin = max(1, min(adaptive, linear_head_k));
    const double blended = (1.0 - alpha) * (double)adaptive + alpha * (double)lin;
    int topk = max(1, (int)rint(blended));  // rint = round-half-to-even, as Python's round()
    topk = min(adaptive, topk);
    k_out[0] = topk;
    k_out[1] = adaptive;
  }
}

// ---------------------------------------------------------------------------------------------
// Per-token head top-k
// ---------------------------------------------------------------------------------------------
// One thread per token, head scores in registers (HT = compile-time bound on H, statically indexed).  When
// `seg_counts` is given (T a multiple of 256, so a CTA is exactly one packing segment) the CTA also counts the rows
// of every head in its segment, which is the first phase of the row packing.
template <int HT>
__global__ void __launch_bounds__(256) head_select_kernel(const float* __restrict__ gate_probs, int64_t n, int G,
                                                          const int32_t* __restrict__ gate_to_head, int H,
                                                          int k_host, const int32_t* __restrict__ k_dev, int kmax,
                                                          const uint8_t* __restrict__ token_mask,
                                                          uint64_t* __restrict__ head_bits,
                                                          int32_t* __restrict__ top_idx,
                                                          float* __restrict__ top_score,
                                                          float* __restrict__ stat_partials, int T, int nseg,
                                                          int32_t* __restrict__ seg_counts) {
  __shared__ int g2h[128];
  __shared__ float red[2][8];
  __shared__ int cnt[64];
  __shared__ int not_identity;
  if (threadIdx.x == 0) not_identity = (G != H) ? 1 : 0;
  for (int i = threadIdx.x; i < 64; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < G; i += blockDim.x) {
    const int h = gate_to_head[i];
    g2h[i] = h;
    if (h != i) not_identity = 1;
  }
  __syncthreads();
  const bool identity = not_identity == 0;  // gate g feeds head g: no scatter needed
  const int k = min(k_dev ? k_dev[0] : k_host, kmax);
  const int64_t tok = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  float score_sum = 0.f, ent = 0.f;
  uint64_t bits = 0;
  if (tok < n) {
    float hp[HT];
#pragma unroll
    for (int h = 0; h < HT; ++h) hp[h] = 0.f;
    const float* gp = gate_probs + tok * G;
    if (identity) {
#pragma unroll
      for (int h = 0; h < HT; h += 4) {
        if (h + 3 < G && (G % 4) == 0) {
          const float4 p4 = *reinterpret_cast<const float4*>(gp + h);
          hp[h] = p4.x; hp[h + 1] = p4.y; hp[h + 2] = p4.z; hp[h + 3] = p4.w;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (h + e < G) hp[h + e] = gp[h + e];
        }
      }
#pragma unroll
      for (int h = 0; h < HT; ++h)
        if (h < G) ent -= logf(fmaxf(hp[h], 1e-9f)) * hp[h];
    } else {
      for (int g = 0; g < G; ++g) {
        const float p = gp[g];
        ent -= logf(fmaxf(p, 1e-9f)) * p;
        const int h = g2h[g];
#pragma unroll
        for (int hh = 0; hh < HT; ++hh) hp[hh] += hh == h ? p : 0.f;  // static register indexing
      }
    }
    if (HT <= 32 && (kmax & 3) == 0) {
      // picks kept in registers (statically indexed) and written as 16-byte vectors: scalar stores of a token's row
      // would each dirty a separate 32-byte sector
      int ti[HT];
      float tsc[HT];
#pragma unroll
      for (int j = 0; j < HT; ++j) {
        int best = -1;
        float bv = -INFINITY;
        if (j < k) {
#pragma unroll
          for (int h = 0; h < HT; ++h)
            if (h < H && !((bits >> h) & 1ull) && hp[h] > bv) {
              bv = hp[h];
              best = h;
            }
          if (best >= 0) {
            bits |= 1ull << best;
            score_sum += bv;
          }
        }
        ti[j] = best;
        tsc[j] = best >= 0 ? bv : 0.f;
      }
#pragma unroll
      for (int j = 0; j < HT; j += 4)
        if (j < kmax) {
          if (top_idx) *reinterpret_cast<int4*>(top_idx + tok * kmax + j) = make_int4(ti[j], ti[j + 1], ti[j + 2], ti[j + 3]);
          if (top_score)
            *reinterpret_cast<float4*>(top_score + tok * kmax + j) = make_float4(tsc[j], tsc[j + 1], tsc[j + 2], tsc[j + 3]);
        }
    } else {
      for (int j = 0; j < kmax; ++j) {
        int best = -1;
        float bv = -INFINITY;
        if (j < k) {
#pragma unroll
          for (int h = 0; h < HT; ++h)
            if (h < H && !((bits >> h) & 1ull) && hp[h] > bv) {
              bv = hp[h];
              best = h;
            }
          if (best >= 0) {
            bits |= 1ull << best;
            score_sum += bv;
          }
        }
        if (top_idx) top_idx[tok * kmax + j] = best;
        if (top_score) top_score[tok * kmax + j] = best >= 0 ? bv : 0.f;
      }
    }
    if (token_mask && !token_mask[tok]) bits = 0;
    head_bits[tok] = bits;
  }
  if (seg_counts) {
    for (int h = 0; h < H; ++h) {
      const unsigned bal = __ballot_sync(0xffffffffu, (bits >> h) & 1ull);
      if ((threadIdx.x & 31) == 0 && bal) atomicAdd(&cnt[h], __popc(bal));
    }
  }
  if (stat_partials) {
    score_sum = warp_sum(score_sum);
    ent = warp_sum(ent);
    if ((threadIdx.x & 31) == 0) {
      red[0][threadIdx.x >> 5] = score_sum;
      red[1][threadIdx.x >> 5] = ent;
    }
  }
  __syncthreads();
  if (stat_partials && threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int w = 0; w < 8; ++w) {
      a += red[0][w];
      b += red[1][w];
    }
    stat_partials[blockIdx.x] = a;
    stat_partials[gridDim.x + blockIdx.x] = b;
  }
  if (seg_counts) {
    const int64_t t0 = (int64_t)blockIdx.x * 256;
    const int b = (int)(t0 / T), seg = (int)((t0 % T) / 256);
    for (int h = threadIdx.x; h < H; h += blockDim.x) seg_counts[((int64_t)b * H + h) * nseg + seg] = cnt[h];
  }
}

static void launch_head_select(const float* gate_probs, int64_t n, int G, const int32_t* gate_to_head, int H, int k_host,
                               const int32_t* k_dev, int kmax, const uint8_t* token_mask, uint64_t* head_bits,
                               int32_t* top_idx, float* top_score, float* stat_partials, int T, int nseg,
                               int32_t* seg_counts, cudaStream_t st) {
  const unsigned grid = (unsigned)ceil_div(n, 256);
  if (H <= 16)
    head_select_kernel<16><<<grid, 256, 0, st>>>(gate_probs, n, G, gate_to_head, H, k_host, k_dev, kmax, token_mask,
                                                 head_bits, top_idx, top_score, stat_partials, T, nseg, seg_counts);
  else if (H <= 32)
    head_select_kernel<32><<<grid, 256, 0, st>>>(gate_probs, n, G, gate_to_head, H, k_host, k_dev, kmax, token_mask,
                                                 head_bits, top_idx, top_score, stat_partials, T, nseg, seg_counts);
  else
    head_select_kernel<64><<<grid, 256, 0, st>>>(gate_probs, n, G, gate_to_head, H, k_host, k_dev, kmax, token_mask,
                                                 head_bits, top_idx, top_score, stat_partials, T, nseg, seg_counts);
}

// ---------------------------------------------------------------------------------------------
// Row packing.  Segment = 256 consecutive tokens of one batch element.
// seg_counts[(b*H + h) * nseg + seg] = rows of head h in the segment; an exclusive scan in that order
// gives every (bh, seg) its first output slot, so rows come out grouped by bh and token-ascending.
// ---------------------------------------------------------------------------------------------
constexpr int PK_SEG = 256;

template <bool kFromBits>
__device__ __forceinline__ uint64_t load_bits(const void* src, int heads_per_batch, int b, int T, int t) {
  if (kFromBits) return reinterpret_cast<const uint64_t*>(src)[(int64_t)b * T + t];
  // uint8 mask (heads, T) with a single "batch": bit h set when mask[h][t] != 0 (heads <= 64 per pass)
  const uint8_t* m = reinterpret_cast<const uint8_t*>(src);
  uint64_t bits = 0;
  for (int h = 0; h < heads_per_batch; ++h) bits |= (uint64_t)(m[((int64_t)b * heads_per_batch + h) * T + t] != 0) << h;
  return bits;
}

template <bool kFromBits>
__global__ void __launch_bounds__(PK_SEG) pack_count_kernel(const void* __restrict__ src, int T, int H, int nseg,
                                                            int32_t* __restrict__ seg_counts) {
  __shared__ int cnt[64];
  const int seg = blockIdx.x, b = blockIdx.y;
  for (int i = threadIdx.x; i < 64; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const int t = seg * PK_SEG + threadIdx.x;
  const uint64_t bits = t < T ? load_bits<kFromBits>(src, H, b, T, t) : 0ull;
  for (int h = 0; h < H; ++h) {
    const unsigned bal = __ballot_sync(0xffffffffu, (bits >> h) & 1ull);
    if ((threadIdx.x & 31) == 0 && bal) atomicAdd(&cnt[h], __popc(bal));
  }
  __syncthreads();
  for (int h = threadIdx.x; h < H; h += blockDim.x) seg_counts[((int64_t)b * H + h) * nseg + seg] = cnt[h];
}

__global__ void __launch_bounds__(1024) pack_scan_kernel(int32_t* __restrict__ seg_counts, int64_t n_entries,
                                                         int nseg, int32_t* __restrict__ row_offsets, int n_heads) {
  // single CTA, in-place exclusive scan; row_offsets[bh] = scanned value at (bh, seg 0)
  __shared__ int tmp[64];
  int running = 0;
  for (int64_t base = 0; base < n_entries; base += blockDim.x) {
    const int64_t i = base + threadIdx.x;
    const int v = i < n_entries ? seg_counts[i] : 0;
    int tot;
    const int ex = block_exclusive_scan(v, tmp, &tot);
    if (i < n_entries) {
      seg_counts[i] = running + ex;
      if (i % nseg == 0) row_offsets[i / nseg] = running + ex;
    }
    running += tot;
  }
  if (threadIdx.x == 0) {
    row_offsets[n_heads] = running;
    seg_counts[n_entries] = running;
  }
}

template <bool kFromBits>
__global__ void __launch_bounds__(PK_SEG) pack_fill_kernel(const void* __restrict__ src, int T, int H, int nseg,
                                                           const int32_t* __restrict__ seg_offsets,
                                                           int32_t* __restrict__ token_idx, int64_t capacity) {
  __shared__ int wcnt[PK_SEG / 32][64];
  const int seg = blockIdx.x, b = blockIdx.y;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int t = seg * PK_SEG + threadIdx.x;
  const uint64_t bits = t < T ? load_bits<kFromBits>(src, H, b, T, t) : 0ull;
  for (int h = 0; h < H; ++h) {
    const unsigned bal = __ballot_sync(0xffffffffu, (bits >> h) & 1ull);
    if (lane == 0) wcnt[w][h] = __popc(bal);
  }
  __syncthreads();
  for (int h = 0; h < H; ++h) {
    const unsigned bal = __ballot_sync(0xffffffffu, (bits >> h) & 1ull);
    if ((bits >> h) & 1ull) {
      int before = 0;
      for (int ww = 0; ww < w; ++ww) before += wcnt[ww][h];
      const int64_t pos = (int64_t)seg_offsets[((int64_t)b * H + h) * nseg + seg] + before +
                          __popc(bal & ((1u << lane) - 1u));
      if (pos < capacity) token_idx[pos] = t;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Ordered compaction of a byte mask
// ---------------------------------------------------------------------------------------------
constexpr int CM_THREADS = 256;
constexpr int CM_PER_THREAD = 8;
constexpr int CM_BLOCK = CM_THREADS * CM_PER_THREAD;  // indices per CTA

__global__ void __launch_bounds__(CM_THREADS) compact_count_kernel(const uint8_t* __restrict__ mask, int64_t n,
                                                                   int32_t* __restrict__ block_counts) {
  __shared__ int tmp[33];
  const int64_t base = (int64_t)blockIdx.x * CM_BLOCK + threadIdx.x * CM_PER_THREAD;
  int c = 0;
#pragma unroll
  for (int j = 0; j < CM_PER_THREAD; ++j)
    if (base + j < n) c += mask[base + j] ? 1 : 0;
  const int tot = block_sum_int(c, tmp);
  if (threadIdx.x == 0) block_counts[blockIdx.x] = tot;
}

__global__ void __launch_bounds__(CM_THREADS) compact_fill_kernel(const uint8_t* __restrict__ mask, int64_t n,
                                                                  int64_t capacity,
                                                                  const int32_t* __restrict__ block_counts,
                                                                  int64_t* __restrict__ kept_idx,
                                                                  int32_t* __restrict__ slot_of,
                                                                  int32_t* __restrict__ count) {
  __shared__ int tmp[33];
  __shared__ int64_t sh_prefix, sh_total;
  // this CTA's first slot and the grand total, summed in a fixed order from the per-CTA counts
  int64_t before = 0, all = 0;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += CM_THREADS) {
    const int c = block_counts[i];
    all += c;
    if (i < (int)blockIdx.x) before += c;
  }
  if (threadIdx.x == 0) sh_prefix = 0, sh_total = 0;
  __syncthreads();
  atomicAdd(reinterpret_cast<unsigned long long*>(&sh_prefix), (unsigned long long)before);
  atomicAdd(reinterpret_cast<unsigned long long*>(&sh_total), (unsigned long long)all);
  __syncthreads();
  const int64_t prefix = sh_prefix, total = sh_total;
  const int64_t base = (int64_t)blockIdx.x * CM_BLOCK + threadIdx.x * CM_PER_THREAD;
  uint32_t bits = 0;
  int c = 0;
#pragma unroll
  for (int j = 0; j < CM_PER_THREAD; ++j)
    if (base + j < n && mask[base + j]) bits |= 1u << j, ++c;
  int blk_total;
  int64_t slot = prefix + block_exclusive_scan(c, tmp, &blk_total);
#pragma unroll
  for (int j = 0; j < CM_PER_THREAD; ++j)
    if ((bits >> j) & 1u) {
      if (slot < capacity) kept_idx[slot] = base + j;
      if (slot_of) slot_of[base + j] = (int32_t)min(slot, (int64_t)0x7fffffff);
      ++slot;
    }
  // padding of the tail, spread over the grid
  for (int64_t i = total + (int64_t)blockIdx.x * CM_THREADS + threadIdx.x; i < capacity;
       i += (int64_t)gridDim.x * CM_THREADS)
    kept_idx[i] = n;
  if (blockIdx.x == 0 && threadIdx.x == 0) count[0] = (int32_t)min(total, (int64_t)0x7fffffff);
}

}  // namespace aspa

using namespace aspa;
static_assert(ASPA_TOKEN_COMPACT_MAX_T == CL_MAX * CL_KEYS_PER_CTA, "header constant out of step with the cluster kernels");

extern "C" int aspa_token_select(const float* importance, int B, int T, int need, float threshold, int guard,
                                 uint8_t* token_mask, int32_t* kept, void* stream) {
  ASPA_CHECK_ARG(importance && token_mask && kept, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0, "bad sizes");
  cudaStream_t st = (cudaStream_t)stream;
  if (T <= 4096) {
    token_select_regs_kernel<4><<<B, 1024, 0, st>>>(importance, T, need, threshold, guard, token_mask, kept);
  } else if (T <= CL_MAX * CL_KEYS_PER_CTA) {
    int csize = 1;
    while (csize * CL_KEYS_PER_CTA < T) csize <<= 1;  // 1, 2, 4 or 8 CTAs; surplus slots hold no keys
    const cudaError_t e = launch_clusters(token_select_cluster_kernel<CL_EPT>, B, csize, 0, st, importance, T, need, threshold,
                                          guard, token_mask, kept, (int64_t*)nullptr, (int32_t*)nullptr, 0);
    if (e != cudaSuccess) {
      set_error("aspa_token_select: cluster launch failed: %s", cudaGetErrorString(e));
      return ASPA_ERR_CUDA;
    }
  } else if (T <= CL_MAX * 32 * CL_THREADS) {  // up to 262144 tokens: 32 keys per thread over 8 CTAs
    const cudaError_t e = launch_clusters(token_select_cluster_kernel<32>, B, CL_MAX, 0, st, importance, T, need, threshold,
                                          guard, token_mask, kept, (int64_t*)nullptr, (int32_t*)nullptr, 0);
    if (e != cudaSuccess) {
      set_error("aspa_token_select: cluster launch failed: %s", cudaGetErrorString(e));
      return ASPA_ERR_CUDA;
    }
  } else {
    token_select_kernel<<<B, 1024, 0, st>>>(importance, T, need, threshold, guard, token_mask, kept);
  }
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_token_select_compact(const float* importance, int B, int T, int need, float threshold, int guard,
                                         uint8_t* token_mask, int32_t* kept, int64_t* kept_idx, int32_t* slot_of,
                                         int slots_per_row, void* stream) {
  ASPA_CHECK_ARG(importance && token_mask && kept && kept_idx && slot_of, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && slots_per_row > 0, "bad sizes");
  ASPA_CHECK_ARG(T <= ASPA_TOKEN_COMPACT_MAX_T, "rows longer than ASPA_TOKEN_COMPACT_MAX_T: use aspa_token_select + aspa_compact_mask");
  ASPA_CHECK_ARG((int64_t)B * std::max(T, slots_per_row) < ((int64_t)1 << 31), "slot numbers must fit 31 bits");
  cudaStream_t st = (cudaStream_t)stream;
  int csize = 1;
  while (csize * CL_KEYS_PER_CTA < T) csize <<= 1;
  const cudaError_t e = launch_clusters(token_select_cluster_kernel<CL_EPT>, B, csize, 0, st, importance, T, need, threshold, guard,
                                        token_mask, kept, kept_idx, slot_of, slots_per_row);
  if (e != cudaSuccess) {
    set_error("aspa_token_select_compact: cluster launch failed: %s", cudaGetErrorString(e));
    return ASPA_ERR_CUDA;
  }
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_head_budget(const float* gate_probs, int64_t n, int G, const int32_t* gate_to_head, int H,
                                double top_p, int dense_k, int h_active_min, int linear_head_k, double alpha,
                                float* scratch, int32_t* k_out, void* stream) {
  ASPA_CHECK_ARG(gate_probs && gate_to_head && scratch && k_out, "null pointer");
  ASPA_CHECK_ARG(n > 0 && G > 0 && G <= 128 && H > 0 && H <= 64, "bad sizes (G <= 128, H <= 64)");
  const int64_t nblk = ceil_div(n, 1024);
  head_colsum_kernel<<<(unsigned)nblk, 256, 0, (cudaStream_t)stream>>>(gate_probs, n, G, gate_to_head, H, scratch);
  ASPA_CHECK_LAUNCH();
  head_budget_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(scratch, nblk, H, (double)n, top_p, dense_k, h_active_min,
                                                          linear_head_k, alpha, k_out);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_head_select(const float* gate_probs, int64_t n, int G, const int32_t* gate_to_head, int H,
                                int k_host, const int32_t* k_dev, int kmax, const uint8_t* token_mask,
                                uint64_t* head_bits, int32_t* top_idx, float* top_score, float* stat_partials,
                                void* stream) {
  ASPA_CHECK_ARG(gate_probs && gate_to_head && head_bits, "null pointer");
  ASPA_CHECK_ARG(n > 0 && G > 0 && G <= 128 && H > 0 && H <= 64 && kmax > 0 && kmax <= H, "bad sizes");
  launch_head_select(gate_probs, n, G, gate_to_head, H, k_host, k_dev, kmax, token_mask, head_bits, top_idx, top_score,
                     stat_partials, 0, 0, nullptr, (cudaStream_t)stream);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_head_select_pack(const float* gate_probs, int B, int T, int G, const int32_t* gate_to_head, int H,
                                     int k_host, const int32_t* k_dev, int kmax, const uint8_t* token_mask,
                                     uint64_t* head_bits, int32_t* top_idx, float* top_score, float* stat_partials,
                                     int32_t* seg_scratch, int32_t* row_offsets, int32_t* token_idx, int64_t capacity,
                                     void* stream) {
  ASPA_CHECK_ARG(gate_probs && gate_to_head && head_bits && seg_scratch && row_offsets && token_idx, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && G > 0 && G <= 128 && H > 0 && H <= 64 && kmax > 0 && kmax <= H, "bad sizes");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t n = (int64_t)B * T;
  const int nseg = (int)ceil_div(T, PK_SEG);
  const bool fused = T % PK_SEG == 0;  // a 256-token CTA of the head choice is then exactly one packing segment
  launch_head_select(gate_probs, n, G, gate_to_head, H, k_host, k_dev, kmax, token_mask, head_bits, top_idx, top_score,
                     stat_partials, T, nseg, fused ? seg_scratch : nullptr, st);
  ASPA_CHECK_LAUNCH();
  const dim3 grid(nseg, B);
  if (!fused) pack_count_kernel<true><<<grid, PK_SEG, 0, st>>>(head_bits, T, H, nseg, seg_scratch);
  pack_scan_kernel<<<1, 1024, 0, st>>>(seg_scratch, (int64_t)B * H * nseg, nseg, row_offsets, B * H);
  pack_fill_kernel<true><<<grid, PK_SEG, 0, st>>>(head_bits, T, H, nseg, seg_scratch, token_idx, capacity);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int64_t aspa_pack_rows_scratch(int B, int H, int T) {
  return (int64_t)B * H * ceil_div(T, PK_SEG) + 1;
}

template <bool kFromBits>
static int pack_impl(const void* src, int B, int T, int H, int32_t* seg_scratch, int32_t* row_offsets,
                     int32_t* token_idx, int64_t capacity, cudaStream_t st) {
  const int nseg = (int)ceil_div(T, PK_SEG);
  const dim3 grid(nseg, B);
  pack_count_kernel<kFromBits><<<grid, PK_SEG, 0, st>>>(src, T, H, nseg, seg_scratch);
  pack_scan_kernel<<<1, 1024, 0, st>>>(seg_scratch, (int64_t)B * H * nseg, nseg, row_offsets, B * H);
  pack_fill_kernel<kFromBits><<<grid, PK_SEG, 0, st>>>(src, T, H, nseg, seg_scratch, token_idx, capacity);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("pack_rows: launch failed: %s", cudaGetErrorString(e));
    return ASPA_ERR_CUDA;
  }
  return ASPA_OK;
}

extern "C" int aspa_pack_rows(const uint64_t* head_bits, int B, int T, int H, int32_t* seg_scratch,
                              int32_t* row_offsets, int32_t* token_idx, int64_t capacity, void* stream) {
  ASPA_CHECK_ARG(head_bits && seg_scratch && row_offsets && token_idx, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && H > 0 && H <= 64, "bad sizes (H <= 64)");
  return pack_impl<true>(head_bits, B, T, H, seg_scratch, row_offsets, token_idx, capacity, (cudaStream_t)stream);
}

extern "C" int aspa_pack_mask(const uint8_t* mask, int heads, int T, int32_t* seg_scratch, int32_t* row_offsets,
                              int32_t* token_idx, int64_t capacity, void* stream) {
  ASPA_CHECK_ARG(mask && seg_scratch && row_offsets && token_idx, "null pointer");
  ASPA_CHECK_ARG(heads > 0 && T > 0, "bad sizes");
  // heads may exceed 64: treat every group of <= 64 heads as one "batch" of the bit-mask packer.
  // Groups must be equal-sized for the (b*H + h) indexing, so use the largest divisor of heads <= 64.
  int hp = 1;
  for (int d = 1; d <= 64 && d <= heads; ++d)
    if (heads % d == 0) hp = d;
  return pack_impl<false>(mask, heads / hp, T, hp, seg_scratch, row_offsets, token_idx, capacity,
                          (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Row packing for callers that must not allocate.
//
// Some hosts of this library cannot hand it scratch memory at call time: a serving loop that sized
// its device arena once at start-up and forbids allocator calls on the request path (an allocation
// may synchronise the device or fragment the arena), or a foreign-language binding that has no CUDA
// allocator of its own and only passes through the input and output buffers it was given.  For them
// the segment-count scratch of the packer lives in a fixed device array inside the library: 1 MiB
// per GPU that loads the library, held until the process exits.
//
// The array's name is only a host-side handle here, not a device address.  The address is looked up
// once per device with cudaGetSymbolAddress (that device being current) and cached.
// ---------------------------------------------------------------------------------------------
namespace aspa {
constexpr int64_t PACK_STATIC_INTS = 262144;  // 1 MiB of int32
static __device__ __align__(256) int32_t g_pack_static_scratch[PACK_STATIC_INTS];

constexpr int PACK_STATIC_MAX_DEVICES = 64;
static int32_t* g_pack_static_ptr[PACK_STATIC_MAX_DEVICES] = {nullptr};
static std::mutex g_pack_static_mutex;

// Device address of the static scratch on the current device; nullptr (with the error set) on failure.
static int32_t* pack_static_scratch_for_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= PACK_STATIC_MAX_DEVICES) {
    set_error("aspa_pack_rows_static: cannot identify the current device (%s)",
              e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_pack_static_mutex);
  if (g_pack_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_pack_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("aspa_pack_rows_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    g_pack_static_ptr[dev] = static_cast<int32_t*>(p);
  }
  return g_pack_static_ptr[dev];
}
}  // namespace aspa

extern "C" int64_t aspa_pack_rows_static_capacity(void) { return aspa::PACK_STATIC_INTS; }

extern "C" int aspa_pack_rows_static(const uint64_t* head_bits, int B, int T, int H, int32_t* row_offsets,
                                     int32_t* token_idx, int64_t capacity, void* stream) {
  ASPA_CHECK_ARG(head_bits && row_offsets && token_idx, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && H > 0 && H <= 64, "bad sizes (H <= 64)");
  const int64_t need = aspa_pack_rows_scratch(B, H, T);
  if (need > PACK_STATIC_INTS) {
    set_error("aspa_pack_rows_static: B*H*ceil(T/256)+1 = %lld scratch entries exceed the built-in %lld; "
              "use aspa_pack_rows with caller-provided scratch",
              (long long)need, (long long)PACK_STATIC_INTS);
    return ASPA_ERR_ARG;
  }
  int32_t* scratch = pack_static_scratch_for_current_device();
  if (scratch == nullptr) return ASPA_ERR_CUDA;
  // Nothing in the scratch has to start at zero: the count pass writes every entry the scan reads.
  return pack_impl<true>(head_bits, B, T, H, scratch, row_offsets, token_idx, capacity, (cudaStream_t)stream);
}

extern "C" int64_t aspa_compact_mask_scratch(int64_t n) { return (int64_t)sizeof(int32_t) * std::max<int64_t>(1, ceil_div(n, CM_BLOCK)); }

extern "C" int aspa_compact_mask(const uint8_t* mask, int64_t n, int64_t capacity, int64_t* kept_idx, int32_t* slot_of,
                                 int32_t* count, void* scratch, void* stream) {
  ASPA_CHECK_ARG(mask && kept_idx && count && scratch, "null pointer");
  ASPA_CHECK_ARG(n > 0 && n < ((int64_t)1 << 31) && capacity >= 0, "bad sizes");
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned nblk = (unsigned)ceil_div(n, CM_BLOCK);
  int32_t* counts = reinterpret_cast<int32_t*>(scratch);
  compact_count_kernel<<<nblk, CM_THREADS, 0, st>>>(mask, n, counts);
  ASPA_CHECK_LAUNCH();
  compact_fill_kernel<<<nblk, CM_THREADS, 0, st>>>(mask, n, capacity, counts, kept_idx, slot_of, count);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
