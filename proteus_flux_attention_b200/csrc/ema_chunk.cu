// Prototype EMA update, chunk promotion (nucleus + top-budget) and the global merge of the chunked
// shortlist pipeline.
#include "cluster.cuh"
#include "common.cuh"
#include "mma.cuh"

namespace aspa {

// ------------------------------------------------------------------------------------------------
// Prototype EMA: weighted[g][c] = sum_t probs[t][g] * x[t][c]
// ------------------------------------------------------------------------------------------------
constexpr int EMA_TOK = 512;   // tokens per CTA
constexpr int EMA_CH = 128;    // channels per CTA (one per thread)

template <typename T, int GT>
__global__ void __launch_bounds__(EMA_CH) ema_partial_kernel(const T* __restrict__ x, int64_t n, int C,
                                                             const float* __restrict__ gate_probs, int G,
                                                             float* __restrict__ part_w /*[nchunk][G][C]*/,
                                                             float* __restrict__ part_c /*[nchunk][G]*/) {
  __shared__ float ps[64][GT];  // 64 tokens of gate probs at a time
  const int chunk = blockIdx.x;
  const int c = blockIdx.y * EMA_CH + threadIdx.x;
  const int64_t t0 = (int64_t)chunk * EMA_TOK;
  const int64_t t1 = min(n, t0 + EMA_TOK);
  float acc[GT];
  float cnt[GT];
#pragma unroll
  for (int g = 0; g < GT; ++g) acc[g] = 0.f, cnt[g] = 0.f;
  for (int64_t tb = t0; tb < t1; tb += 64) {
    const int nt = (int)min((int64_t)64, t1 - tb);
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * GT; i += EMA_CH) {
      const int tt = i / GT, g = i % GT;
      ps[tt][g] = (tt < nt && g < G) ? gate_probs[(tb + tt) * G + g] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float xv = c < C ? ld_as_float<T>(x, (tb + tt) * C + c) : 0.f;
#pragma unroll
      for (int g = 0; g < GT; ++g) acc[g] = fmaf(ps[tt][g], xv, acc[g]);
    }
    if (blockIdx.y == 0 && threadIdx.x == 0) {
      for (int tt = 0; tt < nt; ++tt)
#pragma unroll
        for (int g = 0; g < GT; ++g) cnt[g] += ps[tt][g];
    }
  }
  if (c < C) {
#pragma unroll
    for (int g = 0; g < GT; ++g)
      if (g < G) part_w[((int64_t)chunk * G + g) * C + c] = acc[g];
  }
  if (blockIdx.y == 0 && threadIdx.x == 0) {
#pragma unroll
    for (int g = 0; g < GT; ++g)
      if (g < G) part_c[(int64_t)chunk * G + g] = cnt[g];
  }
}

// The same partial sums on the tensor cores (bf16 activations): W[g][c] = sum_t probs[t][g] * x[t][c] is a GEMM with
// M = gates, N = channels, K = tokens.  The fp32 probabilities are split into three bf16 terms (hi + mid + lo), so
// every product is exact and the fp32 accumulation carries full precision; x is used as it is.
// CTA = 8 warps: a chunk of ETC_TOK tokens x 256 channels (32 per warp); token steps of 32 arrive by cp.async in a
// 3-stage ring; B fragments come from ldmatrix.trans on the staged (token-major) tile.
constexpr int ETC_TOK = 2048;    // tokens per CTA
constexpr int ETC_STEP = 32;     // tokens per pipeline stage
constexpr int ETC_CH = 256;      // channels per CTA
constexpr int ETC_STAGES = 3;
constexpr int ETC_X_BYTES = ETC_STEP * ETC_CH * 2;   // 16 KB

template <int MT>  // MT = ceil(G / 16) m-tiles of 16 gates
__global__ void __launch_bounds__(256) ema_partial_tc_kernel(const __nv_bfloat16* __restrict__ x, int64_t n, int C,
                                                             const float* __restrict__ gate_probs, int G, int tok_per_cta,
                                                             float* __restrict__ part_w, float* __restrict__ part_c) {
  extern __shared__ __align__(128) unsigned char etc_smem[];
  unsigned char* xs = etc_smem;                                              // ETC_STAGES x [32 tokens][512 B], swizzled
  float* ps = reinterpret_cast<float*>(etc_smem + ETC_STAGES * ETC_X_BYTES);  // ETC_STAGES x [32 tokens][MT*16]
  constexpr int GP = MT * 16;
  uint32_t* as_ = reinterpret_cast<uint32_t*>(ps + ETC_STAGES * ETC_STEP * GP);  // [k16][m][term][lane] x 4 words: A fragments of the step
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, c0 = blockIdx.y * ETC_CH;
  const int64_t t_begin = (int64_t)chunk * tok_per_cta;
  const int64_t t_end = min(n, t_begin + tok_per_cta);
  const int nsteps = (int)((t_end - t_begin + ETC_STEP - 1) / ETC_STEP);

  auto issue = [&](int step) {
    if (step < nsteps) {
      const int slot = step % ETC_STAGES;
      const int64_t tb = t_begin + (int64_t)step * ETC_STEP;
      unsigned char* xd = xs + slot * ETC_X_BYTES;
      // 32 tokens x 32 chunks of 16 B; chunk c of token r lives at chunk (c ^ (r & 7)) of its 512-byte row
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int idx = tid + 256 * i;
        const int r = idx >> 5, ch = idx & 31;
        const int64_t t = tb + r;
        const bool ok = t < t_end && c0 + ch * 8 < C;
        const __nv_bfloat16* src = x + (ok ? t : t_begin) * C + (ok ? c0 + ch * 8 : 0);
        cp_async16(smem_u32(xd + r * 512 + ((ch ^ (r & 7)) << 4)), src, ok ? 16 : 0);
      }
      float* pd = ps + slot * ETC_STEP * GP;
      for (int idx = tid; idx < ETC_STEP * GP / 4; idx += 256) {   // 16-byte pieces of the probability rows
        const int r = idx / (GP / 4), g4 = (idx % (GP / 4)) * 4;
        const int64_t t = tb + r;
        const bool ok = t < t_end && g4 + 3 < G && (G % 4) == 0;
        if (ok || (t < t_end && g4 < G)) {
          if (ok) {
            cp_async16(smem_u32(pd + r * GP + g4), gate_probs + t * G + g4, 16);
          } else {   // ragged gate count: plain loads
            for (int e = 0; e < 4; ++e) pd[r * GP + g4 + e] = g4 + e < G ? gate_probs[t * G + g4 + e] : 0.f;
          }
        } else {
          *reinterpret_cast<float4*>(pd + r * GP + g4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
    }
    cp_async_commit();
  };

  float acc[MT][4][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[m][j][e] = 0.f;
  float cnt = 0.f;   // thread g < G of the first channel group sums the probabilities of gate g, in token order

#pragma unroll
  for (int s_ = 0; s_ < ETC_STAGES - 1; ++s_) issue(s_);
  const int gq = lane >> 2, q = lane & 3;
  for (int step = 0; step < nsteps; ++step) {
    cp_async_wait<ETC_STAGES - 2>();
    __syncthreads();
    issue(step + ETC_STAGES - 1);
    const unsigned char* xd = xs + (step % ETC_STAGES) * ETC_X_BYTES;
    const float* pd = ps + (step % ETC_STAGES) * ETC_STEP * GP;
    if (blockIdx.y == 0 && tid < G) {
      for (int r = 0; r < ETC_STEP; ++r) cnt += pd[r * GP + tid];
    }
    // A = probs^T as bf16 fragments, three terms each (hi + mid + lo carry the fp32 probability): every warp needs
    // the same ones, so they are split ONCE per step into shared memory - one thread per (k16, m, lane) fragment -
    // instead of by each of the eight warps (the splitting was three quarters of the kernel's instructions).
    if (tid < (ETC_STEP / 16) * MT * 32) {
      const int fl = tid & 31, fm = (tid >> 5) % MT, fk = tid / (32 * MT);
      const int fgq = fl >> 2, fq = fl & 3;
      const int g0 = fm * 16 + fgq, tk = fk * 16 + 2 * fq;
      float pv[8];
      pv[0] = pd[(tk) * GP + g0];          pv[1] = pd[(tk + 1) * GP + g0];
      pv[2] = pd[(tk) * GP + g0 + 8];      pv[3] = pd[(tk + 1) * GP + g0 + 8];
      pv[4] = pd[(tk + 8) * GP + g0];      pv[5] = pd[(tk + 9) * GP + g0];
      pv[6] = pd[(tk + 8) * GP + g0 + 8];  pv[7] = pd[(tk + 9) * GP + g0 + 8];
#pragma unroll
      for (int term = 0; term < 3; ++term) {
        uint32_t af[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float h0 = bf16_round(pv[2 * i]), h1 = bf16_round(pv[2 * i + 1]);
          pv[2 * i] -= h0;       // exact: what this term does not represent
          pv[2 * i + 1] -= h1;
          af[i] = pack_bf16(h0, h1);
        }
        *reinterpret_cast<uint4*>(as_ + (((fk * MT + fm) * 3 + term) * 32 + fl) * 4) = make_uint4(af[0], af[1], af[2], af[3]);
      }
    }
    __syncthreads();
#pragma unroll
    for (int k16 = 0; k16 < ETC_STEP / 16; ++k16) {
      // B fragments: this warp's 32 channels = chunks 4*warp .. 4*warp+3, two n-tiles per ldmatrix
      uint32_t bf[4][2];
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        const int r = k16 * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        const int ch = warp * 4 + jp * 2 + (lane >> 4);
        ldmatrix_x4_trans(smem_u32(xd + r * 512 + ((ch ^ (r & 7)) << 4)), bf[2 * jp][0], bf[2 * jp][1], bf[2 * jp + 1][0],
                          bf[2 * jp + 1][1]);
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
#pragma unroll
        for (int term = 0; term < 3; ++term) {
          const uint4 a4 = *reinterpret_cast<const uint4*>(as_ + (((k16 * MT + m) * 3 + term) * 32 + lane) * 4);
          const uint32_t af[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16(acc[m][j], af, bf[j][0], bf[j][1]);
        }
      }
    }
  }
  cp_async_wait<0>();
  // partial sums: part_w[(chunk*G + g)*C + c]
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + warp * 32 + j * 8 + 2 * q;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int g = m * 16 + gq + 8 * half;
        if (g < G && c < C)
          *reinterpret_cast<float2*>(part_w + ((int64_t)chunk * G + g) * C + c) =
              make_float2(acc[m][j][2 * half], acc[m][j][2 * half + 1]);
      }
    }
  if (blockIdx.y == 0 && tid < G) part_c[(int64_t)chunk * G + tid] = cnt;
}

__global__ void __launch_bounds__(256) ema_apply_kernel(const float* __restrict__ part_w,
                                                        const float* __restrict__ part_c, int64_t nchunk, int C,
                                                        int G, float decay, float om, float* __restrict__ protos,
                                                        float* __restrict__ usage, float* __restrict__ conf,
                                                        int32_t* __restrict__ updated) {
  // grid (ceil(C/256), G).  Fixed summation order over chunks.
  const int g = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  __shared__ float count_s;
  if (threadIdx.x == 0) {
    float cs = 0.f;
    for (int64_t k = 0; k < nchunk; ++k) cs += part_c[k * G + g];
    count_s = cs;
  }
  __syncthreads();
  const float count = count_s;
  const bool on = count > 1e-6f;
  if (c < C && on) {
    float w = 0.f;
    for (int64_t k = 0; k < nchunk; ++k) w += part_w[(k * G + g) * C + c];
    const float mean = __fdiv_rn(w, count);
    const int64_t i = (int64_t)g * C + c;
    protos[i] = __fadd_rn(__fmul_rn(protos[i], decay), __fmul_rn(mean, om));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    float u = __fmul_rn(usage[g], decay), cf = __fmul_rn(conf[g], decay);
    if (on) {
      u = __fadd_rn(u, __fmul_rn(count, om));
      cf = __fadd_rn(cf, om);
      if (updated) atomicAdd(updated, 1);
    }
    usage[g] = u;
    conf[g] = cf;
  }
}

// ------------------------------------------------------------------------------------------------
// Chunk promotion
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float safe_score(const float* imp, const uint8_t* mask, int i) {
  float s = imp[i];
  if (mask && !mask[i]) s = -INFINITY;
  return isfinite(s) ? s : -1e9f;
}

__device__ void bitonic_u64(unsigned long long* a, int n) {
  for (int k = 2; k <= n; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const unsigned long long x = a[i], y = a[ixj];
          if ((x > y) == ((i & k) == 0)) {
            a[i] = y;
            a[ixj] = x;
          }
        }
      }
      __syncthreads();
    }
}

__global__ void __launch_bounds__(1024) chunk_select_kernel(const float* __restrict__ imp,
                                                            const uint8_t* __restrict__ mask, int T, int budget,
                                                            float top_p, int64_t offset, int P2,
                                                            float* __restrict__ out_scores,
                                                            int64_t* __restrict__ out_idx,
                                                            int32_t* __restrict__ out_count) {
  extern __shared__ unsigned long long keys[];  // [P2] sort keys, then reused
  __shared__ int hist[256];
  __shared__ int sh[4];
  __shared__ int scan_tmp[33];
  __shared__ float redf[33];
  const int limit = min(budget, T);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // any finite score at all?  max and softmax denominator over the safe scores
  float mx = -INFINITY;
  int nfinite = 0;
  for (int i = tid; i < T; i += blockDim.x) {
    float raw = imp[i];
    if (mask && !mask[i]) raw = -INFINITY;
    nfinite += isfinite(raw) ? 1 : 0;
    mx = fmaxf(mx, isfinite(raw) ? raw : -1e9f);
  }
  mx = warp_max(mx);
  if (lane == 0) redf[warp] = mx;
  __syncthreads();
  if (tid == 0) {
    float m = redf[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, redf[w]);
    redf[32] = m;
  }
  __syncthreads();
  mx = redf[32];
  int tot_fin;
  block_exclusive_scan(nfinite, scan_tmp, &tot_fin);
  if (tot_fin == 0 || limit <= 0) {
    if (tid == 0) out_count[0] = 0;
    return;
  }
  float sum = 0.f;
  for (int i = tid; i < T; i += blockDim.x) sum += expf(safe_score(imp, mask, i) - mx);
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) redf[warp] = sum;
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += redf[w];
    redf[32] = s;
  }
  __syncthreads();
  sum = redf[32];

  // radix select of the `limit` best safe scores, ties to the lowest index
  uint32_t prefix = 0, pmask = 0;
  int remaining = limit;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < T; i += blockDim.x) {
      const uint32_t k = float_key(safe_score(imp, mask, i));
      if ((k & pmask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
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
    pmask |= 255u << shift;
    remaining = sh[1];
    __syncthreads();
  }
  for (int i = tid; i < P2; i += blockDim.x) keys[i] = ~0ull;
  __syncthreads();
  int ties_seen = 0, written = 0;
  for (int base = 0; base < T; base += blockDim.x) {
    const int i = base + tid;
    uint32_t k = 0;
    bool gt = false, tie = false;
    if (i < T) {
      k = float_key(safe_score(imp, mask, i));
      gt = k > prefix;
      tie = k == prefix;
    }
    int tt, to;
    const int rank_t = block_exclusive_scan(tie ? 1 : 0, scan_tmp, &tt);
    const bool on = gt || (tie && ties_seen + rank_t < remaining);
    const int pos = block_exclusive_scan(on ? 1 : 0, scan_tmp, &to);
    if (on) keys[written + pos] = ((unsigned long long)(~k) << 32) | (unsigned)i;
    written += to;
    ties_seen += tt;
  }
  __syncthreads();
  bitonic_u64(keys, P2);
  // cumulative softmax mass over the sorted picks (parallel scan, limit <= P2)
  int keep = limit;
  if (top_p < 1.0f) {
    float running = 0.f;
    int below = 0;
    for (int base = 0; base < limit; base += blockDim.x) {
      const int i = base + tid;
      float pr = 0.f;
      if (i < limit) {
        const float sc = key_float(~(uint32_t)(keys[i] >> 32));
        pr = __fdiv_rn(expf(sc - mx), sum);
      }
      // inclusive scan of pr across the block
      float inc = pr;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      __syncthreads();
      if (lane == 31) redf[warp] = inc;
      __syncthreads();
      if (warp == 0) {
        float w = lane < (int)(blockDim.x >> 5) ? redf[lane] : 0.f;
        float winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, winc, o);
          if (lane >= o) winc += t;
        }
        redf[lane] = winc - w;
        if (lane == 31) redf[32] = winc;
      }
      __syncthreads();
      const float mass = running + redf[warp] + inc;
      int tb;
      block_exclusive_scan((i < limit && mass < top_p) ? 1 : 0, scan_tmp, &tb);
      below += tb;
      running += redf[32];
      __syncthreads();
    }
    keep = below;
    if (keep < T) keep += 1;
    keep = max(1, keep);
    keep = min(limit, keep);
  }
  // masked / non-finite picks sort last (their safe score is -1e9): drop them
  int nvalid = 0;
  for (int base = 0; base < keep; base += blockDim.x) {
    const int i = base + tid;
    bool ok = false;
    int idx = 0;
    float raw = 0.f;
    if (i < keep) {
      idx = (int)(keys[i] & 0xffffffffu);
      raw = imp[idx];
      ok = isfinite(raw) && !(mask && !mask[idx]);
    }
    int tv;
    const int pos = block_exclusive_scan(ok ? 1 : 0, scan_tmp, &tv);
    if (ok) {
      out_scores[nvalid + pos] = raw;
      out_idx[nvalid + pos] = (int64_t)idx + offset;
    }
    nvalid += tv;
  }
  if (tid == 0) out_count[0] = nvalid;
}

// Chunk promotion with the chunk's keys spread over a cluster (8 keys per thread, 8192 tokens per CTA, up to 8
// CTAs).  Every CTA places its picks straight into the sort buffer of CTA 0 through distributed shared memory;
// CTA 0 then sorts them, applies the nucleus cut and writes the result.
__global__ void __launch_bounds__(CL_THREADS) chunk_select_cluster_kernel(const float* __restrict__ imp,
                                                                          const uint8_t* __restrict__ mask, int T,
                                                                          int budget, float top_p, int64_t offset,
                                                                          int P2, float* __restrict__ out_scores,
                                                                          int64_t* __restrict__ out_idx,
                                                                          int32_t* __restrict__ out_count,
                                                                          const int32_t* __restrict__ slot_dev,
                                                                          const int64_t* __restrict__ slot_offsets) {
  extern __shared__ unsigned long long keys64[];  // [P2], used in CTA 0
  if (slot_dev != nullptr) {  // record slot and index offset come from device memory (the launch may be a graph node)
    const int slot = slot_dev[0];
    offset = slot_offsets[slot];
    out_scores += (int64_t)slot * budget;
    out_idx += (int64_t)slot * budget;
    out_count += slot;
  }
  __shared__ ClusterScratch cs;
  __shared__ float redf[33];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int limit = min(budget, T);
  const int base = rank * CL_KEYS_PER_CTA + tid * CL_EPT;
  int parity = 0;
  uint32_t keys[CL_EPT];
  uint32_t stat[2] = {0u, 0u};  // finite scores, largest key
  const bool vec_ok = (T % 4 == 0);
#pragma unroll
  for (int j = 0; j < CL_EPT; j += 4) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t mw = 0x01010101u;
    if (vec_ok && base + j + 3 < T) {
      const float4 f = *reinterpret_cast<const float4*>(imp + base + j);
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      if (mask) mw = *reinterpret_cast<const uint32_t*>(mask + base + j);
    } else {
      mw = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (base + j + e < T) {
          v[e] = imp[base + j + e];
          mw |= ((!mask || mask[base + j + e]) ? 1u : 0u) << (8 * e);
        }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      keys[j + e] = 0;
      if (base + j + e < T) {
        const float raw = ((mw >> (8 * e)) & 0xffu) ? v[e] : -INFINITY;
        const bool fin = isfinite(raw);
        stat[0] += fin ? 1u : 0u;
        keys[j + e] = max(float_key(fin ? raw : -1e9f), 1u);
        stat[1] = max(stat[1], keys[j + e]);
      }
    }
  }
  if (rank == 0)
    for (int i = tid; i < P2; i += CL_THREADS) keys64[i] = ~0ull;
  {
    uint32_t fin[1] = {stat[0]}, top[1] = {stat[1]};
    cluster_reduce<1, OpAdd>(fin, cs, parity);
    cluster_reduce<1, OpMax>(top, cs, parity);
    stat[0] = fin[0];
    stat[1] = top[0];
  }
  if (stat[0] == 0u || limit <= 0) {  // uniform over the cluster
    if (rank == 0 && tid == 0) out_count[0] = 0;
    return;
  }
  const float mx = key_float(stat[1]);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < CL_EPT; ++j)
    if (keys[j] != 0) sum += expf(key_float(keys[j]) - mx);
  sum = cluster_sum_float(sum, cs, parity);

  const uint32_t thr = cluster_kth_largest<CL_EPT>(keys, limit, cs, parity);
  uint32_t ge[2] = {0u, 0u}, lower[2];
#pragma unroll
  for (int j = 0; j < CL_EPT; ++j) {
    ge[0] += keys[j] > thr ? 1u : 0u;
    ge[1] += (keys[j] == thr && keys[j] != 0) ? 1u : 0u;
  }
  const int my_eq = (int)ge[1];
  cluster_reduce<2, OpAdd>(ge, cs, parity, lower);
  const int take = limit - (int)ge[0];
  int n_eq;
  int tie_rank = (int)lower[1] + block_exclusive_scan(my_eq, cs.scan_tmp, &n_eq);
  // picks of this thread, then their first slot in CTA 0's buffer (slot order is irrelevant: sorted below)
  uint32_t mine[1] = {0u}, mine_lower[1];
  {
    int tr = tie_rank;
#pragma unroll
    for (int j = 0; j < CL_EPT; ++j) {
      if (keys[j] > thr) ++mine[0];
      else if (keys[j] == thr && keys[j] != 0) mine[0] += (tr++ < take) ? 1u : 0u;
    }
  }
  int cta_picks;
  const int in_cta = block_exclusive_scan((int)mine[0], cs.scan_tmp, &cta_picks);
  mine[0] = (tid == 0) ? (uint32_t)cta_picks : 0u;
  cluster_reduce<1, OpAdd>(mine, cs, parity, mine_lower);
  int slot = (int)mine_lower[0] + in_cta;
  unsigned long long* dst = cluster.map_shared_rank(keys64, 0);
#pragma unroll
  for (int j = 0; j < CL_EPT; ++j) {
    bool on = keys[j] > thr;
    if (keys[j] == thr && keys[j] != 0) on = tie_rank++ < take;
    if (on && slot < P2) dst[slot++] = ((unsigned long long)(~keys[j]) << 32) | (unsigned)(base + j);
  }
  cluster.sync();
  if (rank != 0) return;
  bitonic_u64(keys64, P2);
  int keep = limit;
  if (top_p < 1.0f) {
    float running = 0.f;
    int below = 0;
    for (int b0 = 0; b0 < limit; b0 += CL_THREADS) {
      const int i = b0 + tid;
      float pr = 0.f;
      if (i < limit) pr = __fdiv_rn(expf(key_float(~(uint32_t)(keys64[i] >> 32)) - mx), sum);
      float inc = pr;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      __syncthreads();
      if (lane == 31) redf[warp] = inc;
      __syncthreads();
      if (warp == 0) {
        const float w = redf[lane];
        float winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float t = __shfl_up_sync(0xffffffffu, winc, o);
          if (lane >= o) winc += t;
        }
        redf[lane] = winc - w;
        if (lane == 31) redf[32] = winc;
      }
      __syncthreads();
      const float mass = running + redf[warp] + inc;
      int nb;
      block_exclusive_scan((i < limit && mass < top_p) ? 1 : 0, cs.scan_tmp, &nb);
      below += nb;
      running += redf[32];
      __syncthreads();
    }
    keep = below;
    if (keep < T) keep += 1;
    keep = min(limit, max(1, keep));
  }
  int nvalid = 0;
  for (int b0 = 0; b0 < keep; b0 += CL_THREADS) {
    const int i = b0 + tid;
    bool ok = false;
    int idx = 0;
    float raw = 0.f;
    if (i < keep) {
      idx = (int)(keys64[i] & 0xffffffffu);
      raw = imp[idx];
      ok = isfinite(raw) && !(mask && !mask[idx]);
    }
    int tv;
    const int pos = block_exclusive_scan(ok ? 1 : 0, cs.scan_tmp, &tv);
    if (ok) {
      out_scores[nvalid + pos] = raw;
      out_idx[nvalid + pos] = (int64_t)idx + offset;
    }
    nvalid += tv;
  }
  if (tid == 0) out_count[0] = nvalid;
}

// ------------------------------------------------------------------------------------------------
// Global merge
// ------------------------------------------------------------------------------------------------
__global__ void merge_scatter_kernel(const float* __restrict__ scores, const int64_t* __restrict__ indices,
                                     int64_t n, int64_t seq_len, uint32_t* __restrict__ table) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t idx = indices[i];
  if (idx < 0 || idx >= seq_len) return;
  // a duplicated index is represented by its lowest score; key 0 is reserved for "absent"
  atomicMin(&table[idx], max(float_key(scores[i]), 1u));
}

__global__ void __launch_bounds__(1024) merge_select_kernel(const uint32_t* __restrict__ table, int64_t seq_len,
                                                            int max_tokens, int64_t* __restrict__ keep_idx,
                                                            float* __restrict__ keep_scores,
                                                            int32_t* __restrict__ keep_count) {
  __shared__ int hist[256];
  __shared__ int sh[4];
  __shared__ int scan_tmp[33];
  const int tid = threadIdx.x;
  auto key_at = [table](int64_t i) { const uint32_t k = table[i]; return k == 0xffffffffu ? 0u : k; };
  int present = 0;
  for (int64_t i = tid; i < seq_len; i += blockDim.x) present += key_at(i) != 0u ? 1 : 0;
  int n_present;
  block_exclusive_scan(present, scan_tmp, &n_present);
  const int need = min(max_tokens, n_present);
  if (need <= 0) {
    if (tid == 0) keep_count[0] = 0;
    return;
  }
  uint32_t prefix = 0, pmask = 0;
  int remaining = need;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int64_t i = tid; i < seq_len; i += blockDim.x) {
      const uint32_t k = key_at(i);
      if (k != 0u && (k & pmask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1);
    }
    __syncthreads();
    if (tid == 0) {
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
    pmask |= 255u << shift;
    remaining = sh[1];
    __syncthreads();
  }
  int ties_seen = 0, written = 0;
  for (int64_t base = 0; base < seq_len; base += blockDim.x) {
    const int64_t i = base + tid;
    uint32_t k = 0;
    if (i < seq_len) k = key_at(i);
    const bool gt = k != 0u && k > prefix, tie = k != 0u && k == prefix;
    int tt, to;
    const int rank_t = block_exclusive_scan(tie ? 1 : 0, scan_tmp, &tt);
    const bool on = gt || (tie && ties_seen + rank_t < remaining);
    const int pos = block_exclusive_scan(on ? 1 : 0, scan_tmp, &to);
    if (on) {
      keep_idx[written + pos] = i;
      keep_scores[written + pos] = key_float(k);
    }
    written += to;
    ties_seen += tt;
  }
  if (tid == 0) keep_count[0] = written;
}

// ---- merge with every candidate in registers (n <= 32768) ------------------------------------------------------
// table64[idx] = min over candidates with that index of (score_key << 32 | position): the representative of a
// duplicated index is its lowest score (first position on equal scores), found with one atomicMin per candidate.
__global__ void merge_scatter64_kernel(const float* __restrict__ scores, const int64_t* __restrict__ indices,
                                       int64_t n, int64_t seq_len, unsigned long long* __restrict__ table) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t idx = indices[i];
  if (idx < 0 || idx >= seq_len) return;
  atomicMin(&table[idx], ((unsigned long long)max(float_key(scores[i]), 1u) << 32) | (unsigned)i);
}

__device__ void bitonic_i32(int* a, int n) {
  for (int k = 2; k <= n; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const int x = a[i], y = a[ixj];
          if ((x > y) == ((i & k) == 0)) {
            a[i] = y;
            a[ixj] = x;
          }
        }
      }
      __syncthreads();
    }
}

// Selection over the representatives with the candidates spread over a cluster (8 per thread, 8192 per CTA, up to
// 8 CTAs).  Every pick raises the byte of its sequence index in `picked`; an ordered compaction of that mask then
// yields the kept indices in ascending order (no sort).
__global__ void __launch_bounds__(CL_THREADS) merge_select_cluster_kernel(const float* __restrict__ scores,
                                                                          const int64_t* __restrict__ indices, int n,
                                                                          int64_t seq_len,
                                                                          const unsigned long long* __restrict__ table,
                                                                          int max_tokens,
                                                                          uint8_t* __restrict__ picked) {
  __shared__ ClusterScratch cs;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x;
  int parity = 0;
  uint32_t keys[CL_EPT];
  int idxs[CL_EPT];
  uint32_t reps[1] = {0u};
#pragma unroll
  for (int j = 0; j < CL_EPT; ++j) {
    const int i = rank * CL_KEYS_PER_CTA + j * CL_THREADS + tid;
    keys[j] = 0;
    idxs[j] = 0;
    if (i < n) {
      const int64_t idx = indices[i];
      if (idx >= 0 && idx < seq_len) {
        const uint32_t k = max(float_key(scores[i]), 1u);
        if (table[idx] == (((unsigned long long)k << 32) | (unsigned)i)) {
          keys[j] = k;
          idxs[j] = (int)idx;
          ++reps[0];
        }
      }
    }
  }
  cluster_reduce<1, OpAdd>(reps, cs, parity);
  const int n_rep = (int)reps[0];
  const int need = min(max_tokens, n_rep);
  if (need <= 0) return;  // uniform over the cluster
  uint32_t thr = 0;      // need == n_rep: every representative is kept
  uint32_t idx_cut = 0;  // among ties at thr: keep indices whose complement >= idx_cut
  bool all_ties = true;
  if (need < n_rep) {
    thr = cluster_kth_largest<CL_EPT>(keys, need, cs, parity);
    uint32_t ge[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < CL_EPT; ++j) {
      ge[0] += keys[j] > thr ? 1u : 0u;
      ge[1] += keys[j] == thr ? 1u : 0u;
    }
    cluster_reduce<2, OpAdd>(ge, cs, parity);
    const int take = need - (int)ge[0];
    all_ties = take >= (int)ge[1];
    if (!all_ties)  // the `take` lowest indices among the ties = the `take` largest complements
      idx_cut = cluster_kth_largest_fn<CL_EPT>([&](int j) { return keys[j] == thr ? ~(uint32_t)idxs[j] : 0u; }, take, cs,
                                               parity);
  }
#pragma unroll
  for (int j = 0; j < CL_EPT; ++j)
    if (keys[j] != 0 && (keys[j] > thr || (keys[j] == thr && (all_ties || ~(uint32_t)idxs[j] >= idx_cut))))
      picked[idxs[j]] = 1;
}

// keep_scores / keep_pos of the kept indices from the table entry of each (score key << 32 | candidate position).
__global__ void merge_emit_kernel(const int64_t* __restrict__ keep_idx, const int32_t* __restrict__ keep_count,
                                  int max_tokens, const unsigned long long* __restrict__ table,
                                  float* __restrict__ keep_scores, int64_t* __restrict__ keep_pos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= min(keep_count[0], max_tokens)) return;
  const unsigned long long e = table[keep_idx[i]];
  keep_scores[i] = key_float((uint32_t)(e >> 32));
  if (keep_pos) keep_pos[i] = (int64_t)(e & 0xffffffffull);
}

}  // namespace aspa

using namespace aspa;
static_assert(ASPA_MERGE_POS_MAX == CL_MAX * CL_KEYS_PER_CTA, "header constant out of step with the cluster kernels");

extern "C" int64_t aspa_proto_ema_scratch(int64_t n, int C, int G) {
  const int64_t nchunk = ceil_div(n, EMA_TOK);
  return (int64_t)sizeof(float) * (nchunk * G * C + nchunk * G);
}

template <typename T>
static int ema_launch(const T* x, int64_t n, int C, const float* gp, int G, float* pw, float* pc, cudaStream_t st) {
  const dim3 grid((unsigned)ceil_div(n, EMA_TOK), (unsigned)ceil_div(C, EMA_CH));
  if (G <= 8) ema_partial_kernel<T, 8><<<grid, EMA_CH, 0, st>>>(x, n, C, gp, G, pw, pc);
  else if (G <= 16) ema_partial_kernel<T, 16><<<grid, EMA_CH, 0, st>>>(x, n, C, gp, G, pw, pc);
  else if (G <= 32) ema_partial_kernel<T, 32><<<grid, EMA_CH, 0, st>>>(x, n, C, gp, G, pw, pc);
  else ema_partial_kernel<T, 64><<<grid, EMA_CH, 0, st>>>(x, n, C, gp, G, pw, pc);
  return 0;
}

extern "C" int aspa_proto_ema_update(const void* x, int x_dtype, int64_t n, int C, const float* gate_probs, int G,
                                     double decay, float* prototypes, float* usage, float* confidence, void* scratch,
                                     int32_t* updated, void* stream) {
  ASPA_CHECK_ARG(x && gate_probs && prototypes && usage && confidence && scratch, "null pointer");
  ASPA_CHECK_ARG(n > 0 && C > 0 && G > 0 && G <= 64, "bad sizes (G <= 64)");
  ASPA_CHECK_ARG(x_dtype == ASPA_F32 || x_dtype == ASPA_BF16, "x must be fp32 or bf16");
  cudaStream_t st = (cudaStream_t)stream;
  // bf16 activations with 8-element aligned rows go through the tensor cores (larger token chunks, fewer partials)
  const bool tc = x_dtype == ASPA_BF16 && C % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(gate_probs) & 15) == 0;
  // tokens per CTA of the tensor-core kernel: as many as keep at least two CTAs per SM busy (fewer partial sums to add
  // up), never fewer than the CUDA-core kernel's, for which the scratch is sized
  int etc_tok = ETC_TOK;
  while (tc && etc_tok > EMA_TOK && ceil_div(n, etc_tok) * ceil_div(C, ETC_CH) < 2 * 148) etc_tok >>= 1;
  const int64_t nchunk = ceil_div(n, tc ? etc_tok : EMA_TOK);
  float* pw = reinterpret_cast<float*>(scratch);
  float* pc = pw + nchunk * G * C;
  if (updated) cudaMemsetAsync(updated, 0, sizeof(int32_t), st);
  if (tc) {
    const int MT = (int)ceil_div(G, 16);
    const dim3 grid((unsigned)nchunk, (unsigned)ceil_div(C, ETC_CH));
    const size_t smem = ETC_STAGES * (ETC_X_BYTES + ETC_STEP * MT * 16 * sizeof(float)) + (ETC_STEP / 16) * MT * 3 * 32 * 16;
    auto launch = [&](auto kernel) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      kernel<<<grid, 256, smem, st>>>((const __nv_bfloat16*)x, n, C, gate_probs, G, etc_tok, pw, pc);
    };
    if (MT == 1) launch(ema_partial_tc_kernel<1>);
    else if (MT == 2) launch(ema_partial_tc_kernel<2>);
    else if (MT == 3) launch(ema_partial_tc_kernel<3>);
    else launch(ema_partial_tc_kernel<4>);
  } else if (x_dtype == ASPA_F32) {
    ema_launch<float>((const float*)x, n, C, gate_probs, G, pw, pc, st);
  } else {
    ema_launch<__nv_bfloat16>((const __nv_bfloat16*)x, n, C, gate_probs, G, pw, pc, st);
  }
  ASPA_CHECK_LAUNCH();
  ema_apply_kernel<<<dim3((unsigned)ceil_div(C, 256), G), 256, 0, st>>>(pw, pc, nchunk, C, G, (float)decay, (float)(1.0 - decay), prototypes, usage,
                                                                       confidence, updated);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_chunk_select(const float* importance, const uint8_t* token_mask, int T, int budget, float top_p,
                                 int64_t offset, float* out_scores, int64_t* out_idx, int32_t* out_count,
                                 void* stream) {
  ASPA_CHECK_ARG(importance && out_scores && out_idx && out_count, "null pointer");
  ASPA_CHECK_ARG(T > 0 && budget > 0, "bad sizes");
  int P2 = 2;
  while (P2 < std::min(budget, T)) P2 <<= 1;
  const size_t smem = sizeof(unsigned long long) * P2;
  ASPA_CHECK_ARG(smem <= 200 * 1024, "per-chunk budget too large (max 25600)");
  cudaStream_t st = (cudaStream_t)stream;
  if (T <= CL_MAX * CL_KEYS_PER_CTA) {
    int csize = 1;
    while (csize * CL_KEYS_PER_CTA < T) csize <<= 1;
    cudaFuncSetAttribute(chunk_select_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const cudaError_t e = launch_clusters(chunk_select_cluster_kernel, 1, csize, smem, st, importance, token_mask, T, budget,
                                          top_p, offset, P2, out_scores, out_idx, out_count, (const int32_t*)nullptr,
                                          (const int64_t*)nullptr);
    if (e != cudaSuccess) {
      set_error("aspa_chunk_select: cluster launch failed: %s", cudaGetErrorString(e));
      return ASPA_ERR_CUDA;
    }
  } else {
    cudaFuncSetAttribute(chunk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    chunk_select_kernel<<<1, 1024, smem, st>>>(importance, token_mask, T, budget, top_p, offset, P2, out_scores, out_idx,
                                               out_count);
  }
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_chunk_select_slot(const float* importance, const uint8_t* token_mask, int T, int budget, float top_p,
                                      const int32_t* slot_dev, const int64_t* slot_offsets, float* rec_scores,
                                      int64_t* rec_idx, int32_t* rec_count, void* stream) {
  ASPA_CHECK_ARG(importance && slot_dev && slot_offsets && rec_scores && rec_idx && rec_count, "null pointer");
  ASPA_CHECK_ARG(T > 0 && budget > 0, "bad sizes");
  ASPA_CHECK_ARG(T <= CL_MAX * CL_KEYS_PER_CTA, "chunks longer than 65536 tokens: use aspa_chunk_select");
  int P2 = 2;
  while (P2 < std::min(budget, T)) P2 <<= 1;
  const size_t smem = sizeof(unsigned long long) * P2;
  ASPA_CHECK_ARG(smem <= 200 * 1024, "per-chunk budget too large (max 25600)");
  cudaStream_t st = (cudaStream_t)stream;
  int csize = 1;
  while (csize * CL_KEYS_PER_CTA < T) csize <<= 1;
  cudaFuncSetAttribute(chunk_select_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const cudaError_t e = launch_clusters(chunk_select_cluster_kernel, 1, csize, smem, st, importance, token_mask, T, budget,
                                        top_p, (int64_t)0, P2, rec_scores, rec_idx, rec_count, slot_dev, slot_offsets);
  if (e != cudaSuccess) {
    set_error("aspa_chunk_select_slot: cluster launch failed: %s", cudaGetErrorString(e));
    return ASPA_ERR_CUDA;
  }
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int64_t aspa_merge_finalise_scratch(int64_t seq_len) {
  return 8 * seq_len + ((seq_len + 15) / 16) * 16 + aspa_compact_mask_scratch(seq_len);
}

extern "C" int aspa_merge_finalise(const float* scores, const int64_t* indices, int64_t n, int64_t seq_len,
                                   int max_tokens, void* table, int64_t* keep_idx, float* keep_scores,
                                   int64_t* keep_pos, int32_t* keep_count, void* stream) {
  ASPA_CHECK_ARG(scores && indices && table && keep_idx && keep_scores && keep_count, "null pointer");
  ASPA_CHECK_ARG(n >= 0 && seq_len > 0 && max_tokens > 0, "bad sizes");
  ASPA_CHECK_ARG(keep_pos == nullptr || (n > 0 && n <= ASPA_MERGE_POS_MAX && seq_len < (int64_t)1 << 31),
                 "candidate positions are only tracked for n <= ASPA_MERGE_POS_MAX");
  cudaStream_t st = (cudaStream_t)stream;
  if (n > 0 && n <= CL_MAX * CL_KEYS_PER_CTA && seq_len < (int64_t)1 << 31) {
    // scratch: [64-bit table (seq_len) | picked bytes (seq_len, rounded up to 16) | compaction block counts]
    unsigned long long* t64 = reinterpret_cast<unsigned long long*>(table);
    uint8_t* picked = reinterpret_cast<uint8_t*>(t64 + seq_len);
    void* cscratch = picked + ((seq_len + 15) / 16) * 16;
    cudaMemsetAsync(t64, 0xff, sizeof(unsigned long long) * seq_len, st);
    cudaMemsetAsync(picked, 0, (size_t)seq_len, st);
    merge_scatter64_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(scores, indices, n, seq_len, t64);
    int csize = 1;
    while ((int64_t)csize * CL_KEYS_PER_CTA < n) csize <<= 1;
    const cudaError_t e = launch_clusters(merge_select_cluster_kernel, 1, csize, 0, st, scores, indices, (int)n, seq_len,
                                          (const unsigned long long*)t64, max_tokens, picked);
    if (e != cudaSuccess) {
      set_error("aspa_merge_finalise: cluster launch failed: %s", cudaGetErrorString(e));
      return ASPA_ERR_CUDA;
    }
    ASPA_CHECK_LAUNCH();
    const int rc = aspa_compact_mask(picked, seq_len, max_tokens, keep_idx, nullptr, keep_count, cscratch, stream);
    if (rc != ASPA_OK) return rc;
    merge_emit_kernel<<<(unsigned)ceil_div(max_tokens, 256), 256, 0, st>>>(keep_idx, keep_count, max_tokens, t64, keep_scores,
                                                                            keep_pos);
    ASPA_CHECK_LAUNCH();
    return ASPA_OK;
  }
  // large candidate sets: 32-bit score table over the sequence, selected by a streaming radix select
  uint32_t* t32 = reinterpret_cast<uint32_t*>(table);
  cudaMemsetAsync(t32, 0xff, sizeof(uint32_t) * seq_len, st);
  if (n > 0) merge_scatter_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(scores, indices, n, seq_len, t32);
  merge_select_kernel<<<1, 1024, 0, st>>>(t32, seq_len, max_tokens, keep_idx, keep_scores, keep_count);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
