// Router on the 5th-generation tensor cores (bf16 activations).
//
// The skinny product  [tokens x C] . [C x N]  with
//   N = G router columns + 3*G prototype columns (the fp32 normalised prototypes split into three bf16 terms
//       hi + mid + lo, so that the sum of the three products carries fp32 precision)
// runs as tcgen05.mma (M=128, N, K=16, bf16 x bf16 -> fp32) with the accumulators in tensor memory.
//
// Persistent kernel, one CTA per SM, tiles of 128 tokens handed out round-robin.  The activation stream never waits
// for an epilogue: the accumulator is double-buffered in tensor memory and every role has its own warps.
//   warps 0..3   : norm warps — while the ring runs, sum x^2 of their own token row straight from the staged tiles
//                  (the L2 norm the cosine needs) and hand the 128 norms of a tile over through shared memory
//   warps 4..7   : epilogue group 0 (tiles 0, 2, 4, ... of this CTA, accumulator buffer 0)
//   warps 8..11  : epilogue group 1 (tiles 1, 3, 5, ..., accumulator buffer 1)
//                  read the accumulator with tcgen05.ld and run the per-token epilogue (softmaxes, prototype blend,
//                  importance) shared with the CUDA-core kernel, in registers when G is 16 or 32
//   warp 12      : TMA producer — 128x64 activation tiles and Nx64 weight tiles, 128-byte swizzle, ring of up to
//                  8 stages (as many as shared memory holds)
//   warp 13      : allocates tensor memory, issues the MMAs, commits them to the "stage free" and "accumulator
//                  ready" mbarriers, frees tensor memory at the end
// (Tried and dropped, both slower: taking the norms from the tensor cores as the diagonal of x.x^T, which costs more
// shared-memory bandwidth than the norm warps; prefetching the next tile into L2 with cp.async.bulk.prefetch.)
// x is read from HBM exactly once; the weight tiles (<= 256 KB in total) stay in L2.
// Every mbarrier wait is bounded: on expiry the kernel raises a status word, every role leaves its loop, tensor
// memory is still freed and the kernel returns.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "router_epilogue.cuh"
#include "umma.cuh"

namespace aspa {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;       // bf16 per k-block = one 128-byte swizzle row
constexpr int TC_MAX_STAGES = 8;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;   // 16 KB
constexpr int TC_THREADS = 14 * 32;
constexpr int TC_SMEM_LIMIT = 225 * 1024;

// Shared-memory plan of one CTA (all offsets from the 1024-byte aligned base).
struct TcPlan {
  int stages;        // ring depth
  int stage_bytes;   // 16 KB of activations (+ N * 128 bytes of weights when they stream through the ring)
  int w_resident;    // 1: the whole weight operand (num_k tiles of N x 64) sits in shared memory, loaded once
  int w_off;         // resident weights
  int scratch_off;   // 2 groups x 128 rows x (2G+1) floats for the shared-memory epilogue (G other than 16, 32)
  int norm_off;      // 2 x 128 floats: row norms of the tile in flight for each accumulator buffer
  int bar_off;       // mbarriers, tensor-memory slot, abort flag (256 B), then copies of conf_eps and usage_bias (2 x 256 B)
  int total;         // bytes to request (includes 1024 of alignment slack)
};

static inline bool tc_reg_epilogue(int N, int G, bool has_proto) {
  // the register epilogue expects the column layout [G | G | G | G] (N == 4G, no padding) or just [G]
  return (G == 16 || G == 32) && (!has_proto || N == 4 * G);
}

// The TMA unit turns a box into one request per 128-byte row and, measured, issues about one row every 6 cycles:
// 192 rows per k-block (128 of activations, 64 of weights) cap the stream near 14 B/clk per SM, a third of what HBM
// can deliver.  Keeping the weights resident leaves the whole request rate to the activations.
static inline TcPlan tc_plan(int N, int G, int C, bool has_proto) {
  TcPlan p;
  const int scratch = tc_reg_epilogue(N, G, has_proto) ? 0 : 2 * TC_BM * (2 * G + 1) * 4;
  const int w_bytes = N * C * 2;
  const int fixed = scratch + 2 * TC_BM * 4 + 1024 + 1024;
  p.w_resident = (TC_SMEM_LIMIT - fixed - w_bytes) / TC_A_BYTES >= 4 ? 1 : 0;
  p.stage_bytes = p.w_resident ? TC_A_BYTES : TC_A_BYTES + N * TC_BK * 2;
  p.stages = (TC_SMEM_LIMIT - fixed - (p.w_resident ? w_bytes : 0)) / p.stage_bytes;
  if (p.stages > TC_MAX_STAGES) p.stages = TC_MAX_STAGES;
  p.w_off = p.stages * p.stage_bytes;
  p.scratch_off = p.w_off + (p.w_resident ? w_bytes : 0);
  p.norm_off = p.scratch_off + scratch;
  p.bar_off = (p.norm_off + 2 * TC_BM * 4 + 15) & ~15;
  p.total = p.bar_off + 1024 + 1024;
  return p;
}

// GT = number of gates when it is 16 or 32 (epilogue in registers), 0 = any other count (epilogue through shared memory)
template <int GT>
__global__ void __launch_bounds__(TC_THREADS, 1)
router_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_xt,
                 const __grid_constant__ CUtensorMap tmap_w, const __nv_bfloat16* __restrict__ x, int64_t n,
                 const int rows_per_cta,
                 int C, int G, int N, int has_proto, const float* __restrict__ conf_eps,
                 const float* __restrict__ usage_bias, float proto_temp, float proto_threshold, float proto_span,
                 float proto_blend, float usage_boost, float* __restrict__ gate_probs,
                 float* __restrict__ importance, float* __restrict__ proto_sim, float* __restrict__ blend,
                 float* __restrict__ stat_partials, int* __restrict__ status, const TcPlan plan,
                 const uint32_t spin, const int64_t withhold_tile) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int S = plan.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + plan.bar_off);
  // barrier order: full[S], empty[S], acc_full[2], acc_empty[2], nrm_full[2], nrm_empty[2], wbar
  const uint32_t full0 = s_addr(bars), empty0 = s_addr(bars + S), acc_full0 = s_addr(bars + 2 * S),
                 acc_empty0 = s_addr(bars + 2 * S + 2), nrm_full0 = s_addr(bars + 2 * S + 4),
                 nrm_empty0 = s_addr(bars + 2 * S + 6), wbar = s_addr(bars + 2 * S + 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 9);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  float* norm_s = reinterpret_cast<float*>(smem + plan.norm_off);
  float* conf_s = reinterpret_cast<float*>(smem + plan.bar_off + 256);
  float* ub_s = conf_s + 64;
  if (threadIdx.x < 64) {
    conf_s[threadIdx.x] = (conf_eps != nullptr && (int)threadIdx.x < G) ? conf_eps[threadIdx.x] : 0.f;
    ub_s[threadIdx.x] = (usage_bias != nullptr && (int)threadIdx.x < G) ? usage_bias[threadIdx.x] : 0.f;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k = C / TC_BK;
  // This CTA's token range [cta_row0, cta_end): rows_per_cta (a multiple of 32) rows as 128-row tiles, the last of
  // them shorter when rows_per_cta is no multiple of 128 (copied with its own tensor map, tmap_xt: a shorter box costs
  // proportionally less of the stream, so every SM gets the same share of the bytes and none runs a whole tile longer).
  const int64_t cta_row0 = (int64_t)blockIdx.x * rows_per_cta;
  const int64_t cta_end = cta_row0 + rows_per_cta < n ? cta_row0 + rows_per_cta : n;
  const int tiles_per_cta = (rows_per_cta + TC_BM - 1) / TC_BM;
  const int tail_rows = rows_per_cta - (tiles_per_cta - 1) * TC_BM;            // rows of the last tile of a full range
  const int ntiles = cta_end > cta_row0 ? (int)((cta_end - cta_row0 + TC_BM - 1) / TC_BM) : 0;   // tiles of this CTA
  const uint32_t buf_cols = (uint32_t)N;   // one accumulator buffer
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2 * buf_cols) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);       // the producer's expect_tx arrival; TMA completes the bytes
      mbar_init(empty0 + 8 * s, 1 + 4);  // one MMA commit + one arrival per norm warp
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);          // MMA commit
      mbar_init(acc_empty0 + 8 * b, TC_BM);     // every thread of the epilogue group that owns the buffer
      mbar_init(nrm_full0 + 8 * b, TC_BM);      // every norm thread
      mbar_init(nrm_empty0 + 8 * b, TC_BM);     // every thread of the epilogue group
    }
    mbar_init(wbar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 13) {  // whole warp: allocate tensor memory, publish its base address in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 12) {
    // ---- TMA producer ------------------------------------------------------------------------------------
    // (this loop and the MMA loop below are single threads: every instruction in them is exposed latency, so ring
    // positions are carried, not divided out, and the abort flag is only looked at inside a wait that does not
    // succeed at once)
    if (lane == 0) {
      uint32_t issued = 0, withheld = 0xffffffffu;
      RingPos pos{0, 0u};
      bool ok = true;
      const uint32_t w_tile = (uint32_t)N * TC_BK * 2;
      const uint32_t ring0 = s_addr(smem);
      if (plan.w_resident) {  // the whole weight operand, once: num_k tiles of N x 64 on one barrier
        mbar_expect_tx(wbar, w_tile * (uint32_t)num_k);
        for (int kb = 0; kb < num_k; ++kb) tma_load_2d(s_addr(smem + plan.w_off) + kb * w_tile, &tmap_w, kb * TC_BK, 0, wbar);
      }
      for (int tile = 0; tile < ntiles && ok; ++tile) {
        const int row0 = (int)(cta_row0 + (int64_t)tile * TC_BM);
        const bool short_tile = tile == tiles_per_cta - 1 && tail_rows < TC_BM;
        const CUtensorMap* map_x = short_tile ? &tmap_xt : &tmap_x;
        const uint32_t stage_tx = (short_tile ? (uint32_t)tail_rows * TC_BK * 2 : (uint32_t)TC_A_BYTES) + (plan.w_resident ? 0u : w_tile);
        for (int kb = 0; kb < num_k; ++kb, ++issued, pos.next(S)) {
          if (!mbar_wait_abortable(empty0 + 8 * pos.s, pos.ph ^ 1u, abort_flag, spin)) { raise_abort(abort_flag, status, 1); ok = false; break; }
          if ((int64_t)blockIdx.x * tiles_per_cta + tile == withhold_tile && kb == 0) {   // test hook: this stage is never filled, its consumers must give up
            withheld = issued;
            continue;
          }
          const uint32_t a_dst = ring0 + (uint32_t)pos.s * (uint32_t)plan.stage_bytes, bar = full0 + 8 * pos.s;
          mbar_expect_tx(bar, stage_tx);
          tma_load_2d(a_dst, map_x, kb * TC_BK, row0, bar);
          if (!plan.w_resident) tma_load_2d(a_dst + TC_A_BYTES, &tmap_w, kb * TC_BK, 0, bar);
        }
      }
      if (plan.w_resident) mbar_wait(wbar, 0, spin);  // the weight copies, too, must have landed before shared memory goes away
      // Shared memory must outlive every copy this thread started.  On the normal path the consumers have already
      // waited for all of them; after an abort they may have left early, so wait here (bounded) for the last
      // copy issued into each stage.
      const uint32_t first = issued > (uint32_t)S ? issued - (uint32_t)S : 0u;
      for (uint32_t j = first; j < issued; ++j)
        if (j != withheld) mbar_wait(full0 + 8 * (j % (uint32_t)S), (j / (uint32_t)S) & 1u, spin);
    }
  } else if (warp == 13) {
    // ---- MMA issuer --------------------------------------------------------------------------------------
    if (lane == 0) {
      // instruction descriptor: D fp32, A/B bf16, both K-major, N/8 at bit 17, M/16 at bit 24
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      // operand descriptors by 64-bit adds on the start-address field (16-byte units; shared memory ends below 2^18)
      const uint64_t a_desc0 = umma_desc_k_sw128(s_addr(smem));
      const uint64_t b_desc0 = umma_desc_k_sw128(plan.w_resident ? s_addr(smem + plan.w_off) : s_addr(smem) + TC_A_BYTES);
      const uint64_t stage_step = (uint64_t)(plan.stage_bytes >> 4), w_step = (uint64_t)((N * TC_BK * 2) >> 4);
      RingPos pos{0, 0u};
      uint32_t t = 0;
      bool ok = true;
      if (plan.w_resident && !mbar_wait_abortable(wbar, 0, abort_flag, spin)) { raise_abort(abort_flag, status, 8); ok = false; }
      for (int tile = 0; tile < ntiles && ok; ++tile, ++t) {
        const uint32_t buf = t & 1u, aph = (t >> 1) & 1u;
        if (!mbar_wait_abortable(acc_empty0 + 8 * buf, aph ^ 1u, abort_flag, spin)) { raise_abort(abort_flag, status, 5); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + buf * buf_cols;
        for (int kb = 0; kb < num_k; ++kb, pos.next(S)) {
          if (!mbar_wait_abortable(full0 + 8 * pos.s, pos.ph, abort_flag, spin)) { raise_abort(abort_flag, status, 2); ok = false; break; }
          const uint64_t da = a_desc0 + (uint64_t)pos.s * stage_step;
          const uint64_t db = plan.w_resident ? b_desc0 + (uint64_t)kb * w_step : b_desc0 + (uint64_t)pos.s * stage_step;
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)   // 32 bytes = 2 address units per 16-element step along K
            umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty0 + 8 * pos.s);  // arrives once the MMAs above have finished reading this stage
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);  // arrives once every MMA of the tile has landed in tensor memory
      }
    }
  } else if (warp < 4) {
    // ---- norm warps: thread r owns token row r of every tile ------------------------------------------------
    const int r = threadIdx.x;
    RingPos pos{0, 0u};
    uint32_t t = 0;
    bool ok = true;
    const unsigned char* row0 = smem + r * 128;
    for (int tile = 0; tile < ntiles && ok; ++tile, ++t) {
      float2 acc_a = make_float2(0.f, 0.f), acc_b = make_float2(0.f, 0.f);
      for (int kb = 0; kb < num_k; ++kb, pos.next(S)) {
        if (!mbar_wait_abortable(full0 + 8 * pos.s, pos.ph, abort_flag, spin)) { raise_abort(abort_flag, status, 3); ok = false; break; }
        if (has_proto) {
          const unsigned char* row = row0 + pos.s * plan.stage_bytes;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            // the swizzle only permutes 16-byte chunks inside a row; rotate the start so lanes hit different banks
            const uint4 raw = *reinterpret_cast<const uint4*>(row + (((j + r) & 7) << 4));
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
            const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
            acc_a = __ffma2_rn(f0, f0, acc_a);   // four fp32 chains, two per packed FMA
            acc_b = __ffma2_rn(f1, f1, acc_b);
            acc_a = __ffma2_rn(f2, f2, acc_a);
            acc_b = __ffma2_rn(f3, f3, acc_b);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * pos.s);
      }
      if (!ok) break;
      const uint32_t buf = t & 1u, nph = (t >> 1) & 1u;
      if (!mbar_wait_abortable(nrm_empty0 + 8 * buf, nph ^ 1u, abort_flag, spin)) { raise_abort(abort_flag, status, 6); break; }
      norm_s[buf * TC_BM + r] = (acc_a.x + acc_a.y) + (acc_b.x + acc_b.y);
      mbar_arrive(nrm_full0 + 8 * buf);  // release: the store above is visible to whoever observes the phase flip
    }
  } else {
    // ---- epilogue groups ---------------------------------------------------------------------------------
    const int grp = (warp - 4) >> 2;          // accumulator buffer of this group
    const int r = threadIdx.x - 128 - grp * TC_BM;   // row of the tile = lane of tensor memory
    const int quarter = warp & 3;             // a warp may only touch tensor-memory lanes [32*(warp%4), +32)
    const int stride = 2 * G + 1;
    float* row = reinterpret_cast<float*>(smem + plan.scratch_off) + (grp * TC_BM + r) * stride;
    const int64_t nb = (n + 31) / 32;         // statistics: one partial per 32 tokens
    uint32_t t = 0;
    for (int tile = 0; tile < ntiles; ++tile, ++t) {
      if ((int)(t & 1u) != grp) continue;
      const uint32_t ph = (t >> 1) & 1u;
      if (!mbar_wait_abortable(acc_full0 + 8 * grp, ph, abort_flag, spin)) { raise_abort(abort_flag, status, 4); break; }
      if (!mbar_wait_abortable(nrm_full0 + 8 * grp, ph, abort_flag, spin)) { raise_abort(abort_flag, status, 7); break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)grp * buf_cols;
      const int64_t tok = cta_row0 + (int64_t)tile * TC_BM + r;
      const bool mine = tok < cta_end;   // rows past the range belong to the next CTA (or lie beyond n)
      float st_sim = 0.f, st_bs = 0.f;
      if (GT > 0) {
        constexpr int GR = GT > 0 ? GT : 16;
        float lg[GR], pd[GR];
#pragma unroll
        for (int c0 = 0; c0 < GR; c0 += 16) {
          float v[16];
          tmem_ld16(t_row + (uint32_t)c0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) lg[c0 + i] = v[i];
        }
#pragma unroll
        for (int g = 0; g < GR; ++g) pd[g] = 0.f;
        if (has_proto) {
#pragma unroll
          for (int part = 0; part < 3; ++part) {   // hi, then + mid, then + lo
#pragma unroll
            for (int c0 = 0; c0 < GR; c0 += 16) {
              float v[16];
              tmem_ld16(t_row + (uint32_t)((1 + part) * GR + c0), v);
#pragma unroll
              for (int i = 0; i < 16; ++i) pd[c0 + i] = part == 0 ? v[i] : pd[c0 + i] + v[i];
            }
          }
        }
        const float nsq = norm_s[grp * TC_BM + r];
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(acc_empty0 + 8 * grp);   // the MMA warp may overwrite this accumulator buffer
        mbar_arrive(nrm_empty0 + 8 * grp);   // the norm warps may overwrite this norm buffer
        if (mine) {
          float imp;
          router_epilogue_regs<GR>(lg, pd, true, has_proto != 0, nsq, conf_eps ? conf_s : nullptr,
                                   usage_bias ? ub_s : nullptr, proto_temp, proto_threshold, proto_span, proto_blend,
                                   usage_boost, gate_probs + tok * G, &imp, proto_sim ? proto_sim + tok : nullptr,
                                   blend ? blend + tok : nullptr, &st_sim, &st_bs);
          importance[tok] = imp;
        }
      } else {
        for (int c0 = 0; c0 < N; c0 += 16) {
          float v[16];
          tmem_ld16(t_row + (uint32_t)c0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int c = c0 + i;
            if (c < 2 * G) row[c] = v[i];                            // router logits, then the hi prototype term
            else if (c < 4 * G) row[G + (c - 2 * G) % G] += v[i];    // mid and lo terms fold into the same slot
          }
        }
        const float nsq = norm_s[grp * TC_BM + r];
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(acc_empty0 + 8 * grp);
        mbar_arrive(nrm_empty0 + 8 * grp);
        if (mine) {
          float imp;
          router_epilogue(row, 1, G, true, has_proto != 0, nsq, conf_eps ? conf_s : nullptr, usage_bias ? ub_s : nullptr,
                          proto_temp, proto_threshold, proto_span, proto_blend, usage_boost, gate_probs + tok * G, &imp,
                          proto_sim ? proto_sim + tok : nullptr, blend ? blend + tok : nullptr, &st_sim, &st_bs);
          importance[tok] = imp;
        }
      }
      if (stat_partials) {  // fixed order inside the warp: shuffle tree
        const float a = warp_sum(st_sim), b = warp_sum(st_bs), c = warp_sum(st_bs > 0.f ? 1.f : 0.f);
        const int64_t blk = (cta_row0 + (int64_t)tile * TC_BM) / 32 + quarter;   // ranges and tiles start on multiples of 32
        if (lane == 0 && blk < nb && blk * 32 < cta_end) {
          stat_partials[blk] = a;
          stat_partials[nb + blk] = b;
          stat_partials[2 * nb + blk] = c;
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 13) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// [W_router ; hi(P) ; mid(P) ; lo(P)] as bf16 rows, zero padded to N rows.
__global__ void router_wcat_kernel(const __nv_bfloat16* __restrict__ w_router, const float* __restrict__ proto_hat,
                                   int G, int C, int N, __nv_bfloat16* __restrict__ wcat) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)N * C) return;
  const int row = (int)(i / C), c = (int)(i % C);
  __nv_bfloat16 out = __float2bfloat16_rn(0.f);
  if (row < G) {
    out = w_router[(int64_t)row * C + c];
  } else if (proto_hat != nullptr && row < 4 * G) {
    const int part = (row - G) / G, g = (row - G) % G;
    const float p = proto_hat[(int64_t)g * C + c];
    const float hi = __bfloat162float(__float2bfloat16_rn(p));
    const float mid = __bfloat162float(__float2bfloat16_rn(p - hi));
    const float lo = p - hi - mid;
    out = __float2bfloat16_rn(part == 0 ? hi : (part == 1 ? mid : lo));
  }
  wcat[i] = out;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

static bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TC_BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int router_tc_columns(int G, bool has_proto) {
  const int need = has_proto ? 4 * G : G;
  return (int)ceil_div(need, 16) * 16;
}

}  // namespace aspa

using namespace aspa;

extern "C" int64_t aspa_router_tc_scratch_bytes(int C, int G, int has_proto) {
  const int N = router_tc_columns(G, has_proto != 0);
  if (C <= 0 || G <= 0 || C % TC_BK != 0 || N > 128 || G % 4 != 0) return 0;  // 0 = shape not supported
  return (int64_t)N * C * 2;
}

// Per-device launch facts, looked up once per device: SM count, and whether each kernel variant has been given its
// shared-memory limit on that device (the attribute belongs to the function on ONE device).
struct TcDeviceInfo {
  int sms;
  bool attr[3];
};
static TcDeviceInfo* tc_device_info() {
  static TcDeviceInfo info[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (info[dev].sms == 0) {
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    info[dev].sms = sms > 0 ? sms : 148;
  }
  return &info[dev];
}

static int router_tc_launch(const void* x, int64_t n, int C, const void* w_router, int G, const float* proto_hat,
                            const float* conf_eps, const float* usage_bias, float proto_temp, float proto_threshold,
                            float proto_span, float proto_blend, float usage_boost, float* gate_probs,
                            float* importance, float* proto_sim, float* blend, float* stat_partials, void* scratch,
                            int32_t* status, uint32_t spin, int64_t withhold_tile, void* stream) {
  ASPA_CHECK_ARG(x && w_router && gate_probs && importance && scratch && status, "null pointer");
  const bool has_proto = proto_hat != nullptr;
  if (aspa_router_tc_scratch_bytes(C, G, has_proto) == 0 || n < TC_BM) {
    set_error("aspa_router_fwd_tc: shape not supported (need C %% 64 == 0, G %% 4 == 0, columns <= 128, n >= 128)");
    return ASPA_ERR_UNSUPPORTED;
  }
  ASPA_CHECK_ARG((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0,
                 "x and scratch must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const int N = router_tc_columns(G, has_proto);
  __nv_bfloat16* wcat = reinterpret_cast<__nv_bfloat16*>(scratch);
  router_wcat_kernel<<<(unsigned)ceil_div((int64_t)N * C, 256), 256, 0, st>>>((const __nv_bfloat16*)w_router, proto_hat,
                                                                             G, C, N, wcat);
  ASPA_CHECK_LAUNCH();
  TcDeviceInfo* di = tc_device_info();
  ASPA_CHECK_ARG(di != nullptr, "cannot identify the current device");
  // Every SM gets the same number of rows (a multiple of 32, at least one tile): 65536 tokens on 148 SMs are 448 rows
  // each, three tiles and a half, instead of four tiles on some SMs and three on the others.
  const int64_t share = ceil_div(ceil_div(n, (int64_t)di->sms), 32) * 32;
  const int rows_per_cta = (int)std::max<int64_t>(share, TC_BM);
  const unsigned grid = (unsigned)ceil_div(n, (int64_t)rows_per_cta);
  const int tail_rows = rows_per_cta - (int)(ceil_div((int64_t)rows_per_cta, TC_BM) - 1) * TC_BM;
  CUtensorMap mx, mxt, mw;   // host-side encoding of the descriptors (no driver round trip, no device work)
  if (!make_map(&mx, x, (uint64_t)n, (uint64_t)C, TC_BM) || !make_map(&mxt, x, (uint64_t)n, (uint64_t)C, (uint32_t)tail_rows) ||
      !make_map(&mw, wcat, (uint64_t)N, (uint64_t)C, (uint32_t)N)) {
    set_error("aspa_router_fwd_tc: cuTensorMapEncodeTiled failed");
    return ASPA_ERR_CUDA;
  }
  const TcPlan plan = tc_plan(N, G, C, has_proto);
  if (plan.stages < 2) {
    set_error("aspa_router_fwd_tc: shared memory holds fewer than two ring stages for this shape");
    return ASPA_ERR_UNSUPPORTED;
  }
  auto launch = [&](auto kernel, int variant) {
    if (!di->attr[variant]) {
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_LIMIT + 2048);
      di->attr[variant] = true;
    }
    kernel<<<grid, TC_THREADS, plan.total, st>>>(mx, mxt, mw, (const __nv_bfloat16*)x, n, rows_per_cta, C, G, N, has_proto ? 1 : 0,
                                                 conf_eps, usage_bias, proto_temp, proto_threshold, proto_span, proto_blend,
                                                 usage_boost, gate_probs, importance, proto_sim, blend, stat_partials, status,
                                                 plan, spin, withhold_tile);
  };
  if (tc_reg_epilogue(N, G, has_proto) && G == 16) launch(router_tc_kernel<16>, 0);
  else if (tc_reg_epilogue(N, G, has_proto)) launch(router_tc_kernel<32>, 1);
  else launch(router_tc_kernel<0>, 2);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_router_fwd_tc(const void* x, int64_t n, int C, const void* w_router, int G,
                                  const float* proto_hat, const float* conf_eps, const float* usage_bias,
                                  float proto_temp, float proto_threshold, float proto_span, float proto_blend,
                                  float usage_boost, float* gate_probs, float* importance, float* proto_sim,
                                  float* blend, float* stat_partials, void* scratch, int32_t* status, void* stream) {
  return router_tc_launch(x, n, C, w_router, G, proto_hat, conf_eps, usage_bias, proto_temp, proto_threshold, proto_span,
                          proto_blend, usage_boost, gate_probs, importance, proto_sim, blend, stat_partials, scratch,
                          status, TC_SPIN_LIMIT, -1, stream);
}

extern "C" int aspa_router_fwd_tc_probe(const void* x, int64_t n, int C, const void* w_router, int G,
                                        const float* proto_hat, const float* conf_eps, float* gate_probs,
                                        float* importance, float* proto_sim, float* blend, void* scratch,
                                        int32_t* status, uint32_t spin_limit, int64_t withhold_tile, void* stream) {
  ASPA_CHECK_ARG(spin_limit >= 1024, "spin_limit below 1024 would time healthy waits out");
  return router_tc_launch(x, n, C, w_router, G, proto_hat, conf_eps, nullptr, 0.3f, 0.2f, 0.8f, 0.5f, 0.f, gate_probs,
                          importance, proto_sim, blend, nullptr, scratch, status, spin_limit, withhold_tile, stream);
}

extern "C" int aspa_read_status(int32_t* status, int reset, void* stream) {
  ASPA_CHECK_ARG(status != nullptr, "null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  int32_t host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    set_error("aspa_read_status: %s", cudaGetErrorString(e));
    return ASPA_ERR_CUDA;
  }
  if (host == 0) return ASPA_OK;
  if (reset) cudaMemsetAsync(status, 0, sizeof(int32_t), st);
  static const char* const who[] = {"", "the producer's wait for a free ring stage", "the MMA warp's wait for a filled stage",
                                    "a norm warp's wait for a filled stage", "an epilogue warp's wait for the accumulator",
                                    "the MMA warp's wait for a free accumulator", "a norm warp's wait for a free norm buffer",
                                    "an epilogue warp's wait for the row norms", "the MMA warp's wait for the resident weights"};
  set_error("a bounded device-side wait ran out in the tensor-core router (%s); the outputs of that call are invalid",
            host >= 1 && host <= 8 ? who[host] : "unknown wait");
  return ASPA_ERR_TIMEOUT;
}
