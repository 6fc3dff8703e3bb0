// Window attention on the 5th-generation tensor cores (head_dim 64, bf16 or int8 inputs).
//
// Same job as attn_window_kernel (attention.cu): a CTA owns consecutive packed rows of one head (or of one
// (head, token % stride) group in the anchor pass), streams the union key range of those rows through shared memory
// and keeps a per-row online softmax.  Here the tile is 128 rows x 128 keys and both products run as tcgen05.mma with
// accumulators AND the probabilities in tensor memory:
//     S_j = Q K_j^T  (M 128, N 128, K 64: four instructions, both operands from shared memory)  -> S[j & 1]
//     O  += P_j V_j  (M 128, N 64, K 128: eight instructions, A = P_j from tensor memory, B = V where it lies
//                     in shared memory, as the MN-major operand)                                -> O, accumulated
// Tensor-memory columns: S0 [0,128) S1 [128,256) S2 [256,384) O0 [384,448) O1 [448,512).  Key tile j uses score
// buffer j % 3, whose first 64 columns become P_j once the row has been read (a thread overwrites only its own lane),
// and accumulator j % 2: two softmax states and two accumulators per row (split-K over the tile parity), merged when
// the row tile ends.  Three score buffers let S_{j+3} be issued right behind P_j V_j, so a softmax warp finds its next
// tile waiting.
// Roles (twelve warps: with thirteen the register file would allow 128 registers per thread instead of 168):
//   warps 0..7  softmax.  Warp w owns tensor-memory lanes 32*(w % 4) .. +31 (one row each) and the key tiles of
//               parity w / 4, so two warps share a row but never a tile: while one exponentiates tile j the other
//               waits for S_{j+1} or writes P_{j-1}, which keeps the special-function unit busy across the latencies
//               of either.  A thread reads the 128 scores of its row once, takes their maximum, exponentiates, packs
//               to 16-bit pairs and writes them with tcgen05.st.  The softmax base moves lazily: only when the
//               maximum outgrows it by 2^8 does the thread rescale its accumulator row in tensor memory
//               (probabilities stay below 256, sums in fp32), so in steady state nobody touches O but the tensor
//               core.  A warp whose rows cannot see a key tile writes zeros for it and waits for nothing but its turn.
//   warps 8..10 producers: K and V tiles into a six-stage ring.  bf16 rows arrive by cp.async into the swizzled
//               layout; int8 rows are loaded one tile ahead into registers and widened to fp16 on the way (0x6400 | byte
//               is the half 1024 + byte, one subtraction gives the signed value: exact).  Rows may have any
//               16-byte-aligned stride (the anchor pass reads every stride-th key), which is why this is not a TMA box.
//   warp 11     allocates tensor memory, issues every tcgen05.mma and tcgen05.commit, frees tensor memory.
// int8 inputs run as fp16 x fp16 (values up to 127 and their 64-term dot products are exact in fp32 accumulation),
// P is fp16 there; bf16 inputs run as bf16 x bf16 with P in bf16.
// Every mbarrier wait is bounded; on expiry the CTA raises g_attn_tc_status, all roles leave, tensor memory is freed.
#include <cuda_fp16.h>

#include <algorithm>

#include "attn_params.cuh"
#include "common.cuh"
#include "mma.cuh"
#include "umma.cuh"

namespace aspa {

constexpr int TA_BM = 128;                 // packed rows per tile = tensor-memory lanes
constexpr int TA_BN = 128;                 // keys per tile
constexpr int TA_D = 64;
constexpr int TA_STAGES = 6;             // S_{j+3} is issued with P_j V_j: its K tile must have had three tile periods to arrive
constexpr int TA_TILE = TA_BN * 128;       // bytes of one K or V tile: 128 rows of 128 bytes
constexpr int TA_Q_BYTES = TA_BM * 128;
constexpr int TA_PROD = 3 * 32;             // producer threads
constexpr int TA_THREADS = 12 * 32;
constexpr int TA_TAIL = 4096;              // row tables (2 x 128 ints), half-row exchange (4 x 128 floats), mbarriers, flags
constexpr int TA_SMEM = 1024 + TA_Q_BYTES + TA_STAGES * 2 * TA_TILE + TA_TAIL;
constexpr uint32_t TA_TMEM_COLS = 512;
constexpr uint32_t TA_COL_O = 384;
constexpr int TA_SBUF = 3;                 // score buffers
constexpr int TA_ABSENT = -2147483647;
constexpr float TA_LAZY = 8.f;             // the softmax base follows the row maximum once it is this far (log2) behind

__device__ int g_attn_tc_status;           // non-zero after a bounded wait ran out in any CTA of any launch

#ifdef TA_TIMING
// Diagnostics build only: cycles spent per role and phase, summed over every CTA.
__device__ unsigned long long g_ta_cycles[16];
__device__ int g_ta_debug;   // bit 0: producers skip the copies; bit 1: softmax skips exponentials; bit 2: softmax skips tensor memory
#define TA_DBG(bit) ((g_ta_debug >> (bit)) & 1)
#define TA_T0() long long ta_t = clock64()
#define TA_ACC(slot) do { const long long n_ = clock64(); atomicAdd(&g_ta_cycles[slot], (unsigned long long)(n_ - ta_t)); ta_t = n_; } while (0)
#else
#define TA_DBG(bit) 0
#define TA_T0() do {} while (0)
#define TA_ACC(slot) do {} while (0)
#endif

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

// Four int8 values of `w` -> two fp16 pairs, exactly.
__device__ __forceinline__ void i8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t f = w ^ 0x80808080u;                       // byte + 128 as an unsigned byte
  const uint32_t a = __byte_perm(f, 0x64646464u, 0x4140);   // halves 1024 + f0, 1024 + f1
  const uint32_t b = __byte_perm(f, 0x64646464u, 0x4342);   // halves 1024 + f2, 1024 + f3
  const __half2 off = __half2half2(__ushort_as_half((unsigned short)0x6480));   // 1152 = 1024 + 128
  const __half2 ra = __hsub2(*reinterpret_cast<const __half2*>(&a), off);
  const __half2 rb = __hsub2(*reinterpret_cast<const __half2*>(&b), off);
  lo = *reinterpret_cast<const uint32_t*>(&ra);
  hi = *reinterpret_cast<const uint32_t*>(&rb);
}

template <typename T>
__device__ __forceinline__ uint32_t pack_p(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_p<__nv_bfloat16>(float lo, float hi) { return pack_bf16(lo, hi); }
template <>
__device__ __forceinline__ uint32_t pack_p<int8_t>(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// byte offset of 16-byte chunk `ch` of row `row` inside a 128-byte-swizzled tile of 128-byte rows
__device__ __forceinline__ int ta_swz(int row, int ch) { return row * 128 + ((ch ^ (row & 7)) << 4); }

template <typename T>
__global__ void __launch_bounds__(TA_THREADS, 1) attn_window_tc_kernel(const AttnParams p, const uint32_t spin) {
  constexpr bool kI8 = sizeof(T) == 1;
  constexpr int S = TA_STAGES;
  extern __shared__ unsigned char ta_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ta_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = smem;
  unsigned char* kv_s = smem + TA_Q_BYTES;
  unsigned char* tail = kv_s + S * 2 * TA_TILE;
  int* ts = reinterpret_cast<int*>(tail);            // per tile row: its token (anchor pass: strided position), or ABSENT
  int* grow_s = ts + TA_BM;                          // per tile row: row of the head-grouped packing (workspace row)
  float* lsum_s = reinterpret_cast<float*>(grow_s + TA_BM);   // [2][128] row sums of the two column halves, exchanged at the end
  float* msum_s = lsum_s + 2 * TA_BM;                          // [2][128] their softmax bases
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 3072);
  // kv_full[S], kv_empty[S], s_full[3], p_ready[3], o_final, pair[4]
  const uint32_t kv_full0 = s_addr(bars), kv_empty0 = s_addr(bars + S), s_full0 = s_addr(bars + 2 * S),
                 p_ready0 = s_addr(bars + 2 * S + 3), o_final = s_addr(bars + 2 * S + 6), pair0 = s_addr(bars + 2 * S + 7);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 11);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool anchor = p.an_stride > 0;
  const int astr = anchor ? p.an_stride : 1;
  const int bh = anchor ? blockIdx.y / astr : blockIdx.y;
  const int rho = anchor ? blockIdx.y % astr : 0;
  const int32_t* offs = anchor ? p.an_offsets : p.row_offsets;
  const int start = offs[blockIdx.y];
  const int cnt = offs[blockIdx.y + 1] - start;
  if ((int)blockIdx.x * TA_BM >= cnt) return;      // the whole CTA: nothing has been set up yet

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(kv_full0 + 8 * s, TA_PROD);        // every producer thread
      mbar_init(kv_empty0 + 8 * s, 1);             // one tcgen05.commit
    }
    for (int b = 0; b < TA_SBUF; ++b) {
      mbar_init(s_full0 + 8 * b, 1);
      mbar_init(p_ready0 + 8 * b, TA_BM);          // every softmax thread of the parity the tile belongs to
    }
    mbar_init(o_final, 1);
    for (int q = 0; q < 4; ++q) mbar_init(pair0 + 8 * q, 64);   // the two warps that share a lane quarter
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 11) tmem_alloc(s_addr(tmem_slot), TA_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int Tn = anchor ? (p.T - rho + astr - 1) / astr : p.T;   // keys in this pass's key space
  const int window = anchor ? p.an_window : (p.has_plan ? (p.plan.window > 0 ? p.plan.window : 1) : (Tn + 1));
  const T* qh = reinterpret_cast<const T*>(p.q) + (int64_t)bh * p.T * TA_D;
  const int64_t k_ts = p.kv.k_token * astr, v_ts = p.kv.v_token * astr;
  const T* kh = reinterpret_cast<const T*>(p.k) + (bh / p.H) * p.kv.k_batch + (bh % p.H) * p.kv.k_head + rho * p.kv.k_token;
  const T* vh = reinterpret_cast<const T*>(p.v) + (bh / p.H) * p.kv.v_batch + (bh % p.H) * p.kv.v_head + rho * p.kv.v_token;
  float sc_log2 = p.scale * 1.4426950408889634f;
  if (kI8) sc_log2 *= p.q_scale[bh] * p.k_scale[bh];
  constexpr uint32_t kFmt = kI8 ? 0u : 1u;        // operand format of kind::f16: fp16 for widened int8, bf16 otherwise
  constexpr uint32_t idesc_qk = umma_idesc_f16(kFmt, 0, 0, TA_BM, TA_BN);
  constexpr uint32_t idesc_pv = umma_idesc_f16(kFmt, 0, 1, TA_BM, TA_D);   // V as it lies: MN-major B operand

  uint32_t g_it = 0;   // key tiles this CTA has been through (every role counts the same)
  uint32_t g_rt = 0;   // row tiles with at least one key tile
  uint32_t pair_uses = 0;   // softmax warps: exchanges done over the barrier two warps of a lane quarter share
  for (int r0 = blockIdx.x * TA_BM; r0 < cnt; r0 += gridDim.x * TA_BM) {
    __syncthreads();                                  // the previous row tile is finished in every role
    if (aborted(abort_flag)) break;
    const int nrows = min(TA_BM, cnt - r0);
    if (tid < TA_BM) {
      int tv = TA_ABSENT, gr = 0;
      if (tid < nrows) {
        if (anchor) {
          tv = p.an_tok[start + r0 + tid];
          if (tv == ANCHOR_NO_KEYS) tv = -1;          // present, sees nothing
          gr = p.an_row[start + r0 + tid];
        } else {
          tv = p.token_idx[start + r0 + tid];
          gr = start + r0 + tid;
        }
      }
      ts[tid] = tv;
      grow_s[tid] = gr;
    }
    __syncthreads();
    for (int c = tid; c < TA_BM * 8; c += TA_THREADS) {   // gathered Q rows -> swizzled A operand
      const int row = c >> 3, ch = c & 7;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (ts[row] != TA_ABSENT) {
        const int64_t tq = anchor ? (int64_t)p.token_idx[grow_s[row]] : (int64_t)ts[row];
        if (kI8) {
          const uint2 raw = reinterpret_cast<const uint2*>(qh + tq * TA_D)[ch];
          i8x4_to_f16x4(raw.x, val.x, val.y);
          i8x4_to_f16x4(raw.y, val.z, val.w);
        } else {
          val = reinterpret_cast<const uint4*>(qh + tq * TA_D)[ch];
        }
      }
      *reinterpret_cast<uint4*>(q_s + ta_swz(row, ch)) = val;
    }
    fence_proxy_async();
    // rows ascend inside a group; rows without keys (negative) come first
    const int t_first = ts[0], t_last = ts[nrows - 1];
    const int lo = max(0, t_first - window + 1);
    const int kt_begin = lo / TA_BN;
    const int ntiles = t_last < 0 ? 0 : t_last / TA_BN - kt_begin + 1;
    __syncthreads();

    if (warp >= 8 && warp < 11) {
      // ---- producers ---------------------------------------------------------------------------------------
      const int pt = tid - 256;
      bool ok = true;
      if (!kI8) {
        int pending = -1;   // ring stage whose copies are committed but not yet published
        for (int i = 0; i < ntiles && ok; ++i) {
          const uint32_t it = g_it + i;
          const int s = (int)(it % S);
          const uint32_t ph = ((it / S) & 1u) ^ 1u;
          if (aborted(abort_flag)) { ok = false; break; }
          if (pending >= 0 && !mbar_test(kv_empty0 + 8 * s, ph)) {   // no free stage yet: publish what is in flight first
            cp_async_wait<0>();
            fence_proxy_async();
            mbar_arrive(kv_full0 + 8 * pending);
            pending = -1;
          }
          if (!mbar_wait(kv_empty0 + 8 * s, ph, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 1); ok = false; break;
          }
          unsigned char* ks = kv_s + s * 2 * TA_TILE;
          const int kb = (kt_begin + i) * TA_BN;
          const bool whole = kb + TA_BN <= Tn;   // every key of the tile exists: no clamping
          const T* kt_ptr = kh + (int64_t)kb * k_ts;
          const T* vt_ptr = vh + (int64_t)kb * v_ts;
#pragma unroll
          for (int c = 0; c < (TA_BN * 8 + TA_PROD - 1) / TA_PROD; ++c) {
            const int id = pt + TA_PROD * c, row = id >> 3, ch = id & 7;
            if (id < TA_BN * 8 && !TA_DBG(0)) {
              if (whole) {
                cp_async16(smem_u32(ks + ta_swz(row, ch)), kt_ptr + row * k_ts + ch * 8, 16);
                cp_async16(smem_u32(ks + TA_TILE + ta_swz(row, ch)), vt_ptr + row * v_ts + ch * 8, 16);
              } else {
                const int key = kb + row;
                const int64_t kc = min(key, Tn - 1);
                const int nbytes = key < Tn ? 16 : 0;
                cp_async16(smem_u32(ks + ta_swz(row, ch)), kh + kc * k_ts + ch * 8, nbytes);
                cp_async16(smem_u32(ks + TA_TILE + ta_swz(row, ch)), vh + kc * v_ts + ch * 8, nbytes);
              }
            }
          }
          cp_async_commit();
          if (pending >= 0) {   // the previous tile has landed once at most one group is still in flight
            cp_async_wait<1>();
            fence_proxy_async();
            mbar_arrive(kv_full0 + 8 * pending);
          }
          pending = s;
        }
        cp_async_wait<0>();   // nothing of this thread is in flight into shared memory past this point
        if (ok && pending >= 0) {
          fence_proxy_async();
          mbar_arrive(kv_full0 + 8 * pending);
        }
      } else {
        // int8: the raw rows of the next tile are in registers while this tile is widened and stored
        constexpr int NC = (TA_BN * 4 + TA_PROD - 1) / TA_PROD;   // 16-byte raw chunks per thread and tile
        uint4 nk[NC], nv[NC];
        auto fetch = [&](int i) {
          const int kb = (kt_begin + i) * TA_BN;
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            const int id = pt + TA_PROD * c, row = id >> 2, rc = id & 3;
            const int key = kb + row;
            nk[c] = nv[c] = make_uint4(0, 0, 0, 0);
            if (id < TA_BN * 4 && key < Tn) {
              nk[c] = *reinterpret_cast<const uint4*>(kh + (int64_t)key * k_ts + rc * 16);
              nv[c] = *reinterpret_cast<const uint4*>(vh + (int64_t)key * v_ts + rc * 16);
            }
          }
        };
        if (ntiles > 0) fetch(0);
        for (int i = 0; i < ntiles; ++i) {
          const uint32_t it = g_it + i;
          const int s = (int)(it % S);
          uint4 ck[NC], cv[NC];
#pragma unroll
          for (int c = 0; c < NC; ++c) { ck[c] = nk[c]; cv[c] = nv[c]; }
          if (i + 1 < ntiles) fetch(i + 1);
          if (aborted(abort_flag)) break;
          if (!mbar_wait(kv_empty0 + 8 * s, ((it / S) & 1u) ^ 1u, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 1); break;
          }
          unsigned char* ks = kv_s + s * 2 * TA_TILE;
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            const int id = pt + TA_PROD * c, row = id >> 2, rc = id & 3;
            if (id >= TA_BN * 4) continue;
            uint4 a, b;
            i8x4_to_f16x4(ck[c].x, a.x, a.y); i8x4_to_f16x4(ck[c].y, a.z, a.w);
            i8x4_to_f16x4(ck[c].z, b.x, b.y); i8x4_to_f16x4(ck[c].w, b.z, b.w);
            *reinterpret_cast<uint4*>(ks + ta_swz(row, 2 * rc)) = a;
            *reinterpret_cast<uint4*>(ks + ta_swz(row, 2 * rc + 1)) = b;
            i8x4_to_f16x4(cv[c].x, a.x, a.y); i8x4_to_f16x4(cv[c].y, a.z, a.w);
            i8x4_to_f16x4(cv[c].z, b.x, b.y); i8x4_to_f16x4(cv[c].w, b.z, b.w);
            *reinterpret_cast<uint4*>(ks + TA_TILE + ta_swz(row, 2 * rc)) = a;
            *reinterpret_cast<uint4*>(ks + TA_TILE + ta_swz(row, 2 * rc + 1)) = b;
          }
          fence_proxy_async();
          mbar_arrive(kv_full0 + 8 * s);
        }
      }
    } else if (warp == 11) {
      // ---- MMA issuer ----------------------------------------------------------------------------------------
      if (lane == 0 && ntiles > 0) {
        // Descriptors differ from one instruction to the next only in their start-address field (bits 0..13, in
        // 16-byte units, never carrying out of it: shared memory is smaller than 256 KB), so each one is a 32-bit add.
        const uint64_t q_desc = umma_desc_k_sw128(s_addr(q_s));
        const uint64_t kv_desc = umma_desc_k_sw128(s_addr(kv_s));
        bool ok = true;
        auto issue_qk = [&](int i) {     // S[it % 3] = Q K_i^T
          const uint32_t it = g_it + i;
          const int s = (int)(it % S);
          if (!mbar_wait(kv_full0 + 8 * s, (it / S) & 1u, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 2); ok = false; return;
          }
          tc_fence_after();
          const uint64_t k_desc = kv_desc + (uint64_t)(s * (2 * TA_TILE / 16));
          const uint32_t d_tmem = tmem_base + (it % TA_SBUF) * TA_BN;
#pragma unroll
          for (int k = 0; k < TA_D / 16; ++k)
            umma_f16(d_tmem, q_desc + (uint64_t)(k * 2), k_desc + (uint64_t)(k * 2), idesc_qk, k > 0 ? 1u : 0u);
          umma_commit(s_full0 + 8 * (it % TA_SBUF));
        };
        TA_T0();
        issue_qk(0);
        if (ok && ntiles > 1) issue_qk(1);
        if (ok && ntiles > 2) issue_qk(2);
        TA_ACC(0);   // prologue: first two S tiles issued (includes the wait for the first K tiles)
        for (int j = 0; j < ntiles && ok; ++j) {
          const uint32_t it = g_it + j, b = it & 1u;
          const int s = (int)(it % S);
          if (aborted(abort_flag)) { ok = false; break; }
          const uint32_t b3 = it % TA_SBUF;
          if (!mbar_wait(p_ready0 + 8 * b3, (it / TA_SBUF) & 1u, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 3); ok = false; break;
          }
          TA_ACC(1);   // MMA thread waiting for P_j
          tc_fence_after();
          const uint32_t p_tmem = tmem_base + b3 * TA_BN;               // P_j lies over the first half of S_j
          const uint64_t v_desc = kv_desc + (uint64_t)((s * 2 * TA_TILE + TA_TILE) / 16);
          const uint32_t o_tmem = tmem_base + TA_COL_O + b * TA_D;      // the accumulator of this tile parity
          const uint32_t acc0 = (j >= 2 || p.read_partial) ? 1u : 0u;
#pragma unroll
          for (int k = 0; k < TA_BN / 16; ++k)   // 16 keys per instruction: 8 columns of P, 16 rows of V
            umma_f16_ts(o_tmem, p_tmem + k * 8, v_desc + (uint64_t)(k * (16 * 128 / 16)), idesc_pv, k > 0 ? 1u : acc0);
          umma_commit(kv_empty0 + 8 * s);      // P_j V_j done: O holds the sum up to tile j, the ring stage may be refilled
          TA_ACC(2);   // issuing P V
          if (j + 3 < ntiles) issue_qk(j + 3); // into the buffer of tile j: queued behind P_j V_j, which reads it first
          TA_ACC(3);   // issuing Q K (includes the wait for the K tile)
        }
        if (ok) {
          umma_commit(o_final);                // everything issued for this row tile has finished
          if (!mbar_wait(o_final, g_rt & 1u, spin)) { atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 4); }
          TA_ACC(4);   // draining the tensor pipe at the end of the row tile
        }
      }
    } else {
      // ---- softmax warps: lane quarter q4, tile parity g; thread (q4, lane) owns row r for the key tiles of parity g --------
      const int q4 = warp & 3, h = warp >> 2;   // h: tile parity this warp serves, and the output channels 32h .. 32h+31
      const int r = q4 * 32 + lane;
      const int tr_raw = ts[r];
      const bool present = tr_raw != TA_ABSENT;
      const int tr = present ? tr_raw : -1;
      const int hi_key = tr, lo_key = tr < 0 ? 0 : max(tr - window + 1, 0);   // valid keys [lo_key, hi_key]; none if tr < 0
      const int w_last = __reduce_max_sync(0xffffffffu, tr);
      const int w_first = __reduce_min_sync(0xffffffffu, tr < 0 ? 0x7fffffff : tr);
      const bool w_any = w_last >= 0;
      const int w_lo = w_any ? max(0, w_first - window + 1) : 0;
      const uint32_t t_lane = tmem_base + ((uint32_t)(q4 * 32) << 16);
      const uint32_t t_oh = t_lane + TA_COL_O + h * TA_D;    // the accumulator row of this tile parity (64 columns)
      const int64_t gr = grow_s[r];

      float m = -INFINITY, l = 0.f;     // softmax base (log2 domain, scaled) and row sum over the tiles of this parity
      bool ok = true;
      if (p.read_partial && ntiles > 0) {
        // Start from the state an earlier pass left: it becomes the state of parity 0, parity 1 starts empty.
        // Thread (q4, h) writes channels 32h .. 32h+31 of both accumulators.
        uint32_t w[32], z[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) w[i] = z[i] = 0u;
        if (present) {
          if (h == 0) {
            const float mw = p.ws_m[gr];
            m = (mw == -INFINITY) ? -INFINITY : mw * 1.4426950408889634f;
            l = p.ws_l[gr];
          }
#pragma unroll
          for (int d = 0; d < 32; d += 2) {   // the workspace rows start on 8-byte boundaries only
            const float2 f = *reinterpret_cast<const float2*>(p.ws_o + gr * TA_D + h * 32 + d);
            w[d] = __float_as_uint(f.x); w[d + 1] = __float_as_uint(f.y);
          }
        }
        tmem_st32(t_lane + TA_COL_O + h * 32, w);
        tmem_st32(t_lane + TA_COL_O + TA_D + h * 32, z);
        tmem_wait_st();
        // both warps of a lane quarter wrote parts of both accumulators: neither may signal a P before both are done
        tc_fence_before();
        mbar_arrive(pair0 + 8 * q4);
        if (!mbar_wait(pair0 + 8 * q4, pair_uses & 1u, spin)) { atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 7); ok = false; }
        ++pair_uses;
        tc_fence_after();
      }
      TA_T0();
      for (int j = 0; j < ntiles && ok; ++j) {
        const uint32_t it = g_it + j, b = it & 1u;
        if ((int)b != h) continue;                            // the other warp of this lane quarter has this tile
        const int kb = (kt_begin + j) * TA_BN;
        const bool active = w_any && kb <= w_last && kb + TA_BN - 1 >= w_lo;   // warp-uniform
        if (aborted(abort_flag)) { ok = false; break; }
        // Every warp waits for its S_j, also one that skips the tile: S_j is issued only after P_{j-3}, which shares
        // its buffer and its barriers, was signalled by all 128 threads of the other parity, so passing this wait is
        // what tells a warp that its arrival belongs to the phase of tile j.  The tensor pipe runs in order: S_j
        // complete means P_{j-3} V_{j-3} has read its operand, so these columns may be written again.
        const uint32_t b3 = it % TA_SBUF;
        if (!mbar_wait(s_full0 + 8 * b3, (it / TA_SBUF) & 1u, spin)) {
          atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 6); ok = false; break;
        }
        const uint32_t t_p = t_lane + b3 * TA_BN;   // the 128 probabilities of this row: 64 columns over the start of S_j
        if (lane == 0 && q4 == 0) TA_ACC(5);   // softmax warp waiting for S_j
        if (TA_DBG(2)) {
          tc_fence_before();
          mbar_arrive(p_ready0 + 8 * b3);
          continue;
        }
        if (active) {
          tc_fence_after();
          // valid columns of this row inside the tile: [clo, clo + span]; an empty range is (huge, 0)
          const bool some = hi_key >= lo_key && hi_key >= kb && lo_key <= kb + TA_BN - 1;
          const int clo = some ? max(lo_key - kb, 0) : (1 << 20);
          const uint32_t span = some ? (uint32_t)(min(hi_key - kb, TA_BN - 1) - clo) : 0u;
          const bool all_full = __all_sync(0xffffffffu, some && clo == 0 && span == TA_BN - 1);
          uint32_t sv[4][32];
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) tmem_ld32_nowait(t_lane + b3 * TA_BN + c4 * 32, sv[c4]);
          tmem_wait_ld();
          if (lane == 0 && q4 == 0) TA_ACC(6);   // loading the score row from tensor memory
          if (!all_full) {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                sv[c4][i] = (uint32_t)(c4 * 32 + i - clo) <= span ? sv[c4][i] : 0xff800000u;   // -inf
          }
          float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            mx0 = fmax3(mx0, __uint_as_float(sv[0][i]), __uint_as_float(sv[0][i + 1]));
            mx1 = fmax3(mx1, __uint_as_float(sv[1][i]), __uint_as_float(sv[1][i + 1]));
            mx2 = fmax3(mx2, __uint_as_float(sv[2][i]), __uint_as_float(sv[2][i + 1]));
            mx3 = fmax3(mx3, __uint_as_float(sv[3][i]), __uint_as_float(sv[3][i + 1]));
          }
          const float m_cand = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sc_log2;
          // Lazy base: move it only when the maximum has outgrown it by 2^TA_LAZY (or there was none).
          const bool need = m_cand > m + TA_LAZY || (m == -INFINITY && m_cand > -INFINITY);
          if (__any_sync(0xffffffffu, need)) {
            // O must be at rest: P_{j-2} V_{j-2}, the last product into this accumulator, signals the ring-stage
            // barrier of its tile when it is done.  (The wait is occasional, which is safe: that barrier completes its
            // next phase S tiles later, long after this thread has signalled P_j.)
            if (j >= 2 && !mbar_wait(kv_empty0 + 8 * (int)((it - 2) % S), ((it - 2) / S) & 1u, spin)) {
              atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 8); ok = false; break;
            }
            tc_fence_after();
            const float cf = !need ? 1.f : (m == -INFINITY ? 0.f : ex2_approx(m - m_cand));
#pragma unroll 1
            for (int hh = 0; hh < 8; ++hh) {   // eight columns at a time: the score row occupies most registers
              uint32_t w[8];
              tmem_ld8(t_oh + hh * 8, w);
#pragma unroll
              for (int i = 0; i < 8; ++i) w[i] = cf == 0.f ? 0u : __float_as_uint(__uint_as_float(w[i]) * cf);
              tmem_st8(t_oh + hh * 8, w);
            }
            l *= cf;
            if (need) m = m_cand;
          }
          if (lane == 0 && q4 == 0) TA_ACC(7);   // mask, maximum, (rare) rescale
          const float base = (m == -INFINITY) ? 0.f : m;
          const float2 sc2 = make_float2(sc_log2, sc_log2), nb2 = make_float2(-base, -base);
          float2 sa = make_float2(0.f, 0.f), sb = make_float2(0.f, 0.f);
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {   // 64 keys = 32 columns of P at a time
            uint32_t pw[32];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float2 ea = __ffma2_rn(make_float2(__uint_as_float(sv[2 * c2][i]), __uint_as_float(sv[2 * c2][i + 1])), sc2, nb2);
              float2 ec = __ffma2_rn(make_float2(__uint_as_float(sv[2 * c2 + 1][i]), __uint_as_float(sv[2 * c2 + 1][i + 1])), sc2, nb2);
              if (!TA_DBG(1)) {
                ea.x = ex2_approx(ea.x); ea.y = ex2_approx(ea.y);
                ec.x = ex2_approx(ec.x); ec.y = ex2_approx(ec.y);
              }
              sa = __fadd2_rn(sa, ea);
              sb = __fadd2_rn(sb, ec);
              pw[i >> 1] = pack_p<T>(ea.x, ea.y);
              pw[16 + (i >> 1)] = pack_p<T>(ec.x, ec.y);
            }
            tmem_st32(t_p + c2 * 32, pw);
          }
          l += (sa.x + sa.y) + (sb.x + sb.y);
          if (lane == 0 && q4 == 0) TA_ACC(8);   // exponentials, packing, tcgen05.st issue
        } else {
          uint32_t pw[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) pw[i] = 0u;   // the tensor core multiplies all 128 rows: rows that see nothing add zero
          tmem_st32(t_p, pw);
          tmem_st32(t_p + 32, pw);
        }
        tmem_wait_st();
        tc_fence_before();       // the writes of P_j (and of a rescaled O) and the reads of S[b] are complete
        mbar_arrive(p_ready0 + 8 * b3);
        if (lane == 0 && q4 == 0) TA_ACC(9);   // waiting for the stores, signalling P_j
      }
      // ---- result of the row tile: merge the two parities (m, l, O)_0 and (m, l, O)_1 -----------------------------------
      if (ntiles == 0 && p.read_partial && present && h == 0) {   // no key tile at all: the state passes through
        const float mw = p.ws_m[gr];
        m = (mw == -INFINITY) ? -INFINITY : mw * 1.4426950408889634f;
        l = p.ws_l[gr];
      }
      msum_s[h * TA_BM + r] = m;
      lsum_s[h * TA_BM + r] = l;
      mbar_arrive(pair0 + 8 * q4);
      if (!mbar_wait(pair0 + 8 * q4, pair_uses & 1u, spin)) { atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 7); ok = false; }
      ++pair_uses;
      const float m_other = msum_s[(h ^ 1) * TA_BM + r], l_other = lsum_s[(h ^ 1) * TA_BM + r];
      const float m_lo = h == 0 ? m : m_other, m_hi = h == 0 ? m_other : m;
      const float l_lo = h == 0 ? l : l_other, l_hi = h == 0 ? l_other : l;
      const float m_all = fmaxf(m_lo, m_hi);
      const float a_lo = m_lo == -INFINITY ? 0.f : ex2_approx(m_lo - m_all), a_hi = m_hi == -INFINITY ? 0.f : ex2_approx(m_hi - m_all);
      const float l_tot = l_lo * a_lo + l_hi * a_hi;
      float o[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0.f;
      if (ntiles > 0) {
        if (ok && !mbar_wait(o_final, g_rt & 1u, spin)) { atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 5); ok = false; }
        if (ok) {   // channels 32h .. 32h+31 of both accumulators
          tc_fence_after();
          uint32_t w0[32], w1[32];
          tmem_ld32_nowait(t_lane + TA_COL_O + h * 32, w0);
          tmem_ld32_nowait(t_lane + TA_COL_O + TA_D + h * 32, w1);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // a weight of zero means that half never saw a key; its accumulator may hold anything then
            const float x0 = a_lo == 0.f ? 0.f : __uint_as_float(w0[i]) * a_lo;
            const float x1 = a_hi == 0.f ? 0.f : __uint_as_float(w1[i]) * a_hi;
            o[i] = x0 + x1;
          }
        }
      } else if (p.read_partial && present) {
#pragma unroll
        for (int d = 0; d < 32; d += 2) {
          const float2 f = *reinterpret_cast<const float2*>(p.ws_o + gr * TA_D + h * 32 + d);
          o[d] = f.x; o[d + 1] = f.y;
        }
      }
      mbar_arrive(pair0 + 8 * q4);   // both halves have read the exchange slots: the next row tile may overwrite them
      if (!mbar_wait(pair0 + 8 * q4, pair_uses & 1u, spin)) { atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 7); ok = false; }
      ++pair_uses;
      if (ok && present) {
        if (p.write_partial) {
          if (h == 0) {
            p.ws_m[gr] = (m_all == -INFINITY) ? -INFINITY : m_all * 0.6931471805599453f;   // natural-log domain
            p.ws_l[gr] = l_tot;
          }
#pragma unroll
          for (int d = 0; d < 32; d += 2)
            *reinterpret_cast<float2*>(p.ws_o + gr * TA_D + h * 32 + d) = make_float2(o[d], o[d + 1]);
        } else {
          float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
          if (kI8) inv *= p.v_scale[bh];
          const int tok = anchor ? p.token_idx[gr] : tr;
          const int64_t ob = out_row_base(p, bh, tok) + h * 32;
          if (p.out_dtype == ASPA_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + ob;
#pragma unroll
            for (int d = 0; d < 32; d += 8)
              *reinterpret_cast<uint4*>(dst + d) =
                  make_uint4(pack_bf16(o[d] * inv, o[d + 1] * inv), pack_bf16(o[d + 2] * inv, o[d + 3] * inv),
                             pack_bf16(o[d + 4] * inv, o[d + 5] * inv), pack_bf16(o[d + 6] * inv, o[d + 7] * inv));
          } else {
            float* dst = reinterpret_cast<float*>(p.out) + ob;
#pragma unroll
            for (int d = 0; d < 32; d += 4)
              *reinterpret_cast<float4*>(dst + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
          }
        }
      }
    }
    g_it += (uint32_t)ntiles;
    g_rt += ntiles > 0 ? 1u : 0u;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 11) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TA_TMEM_COLS);
  }
}

// one flag per device and kernel variant: the shared-memory limit is an attribute of the function on one device
static bool* ta_attr_flag(int variant) {
  static bool done[64][2] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  return &done[dev][variant];
}

bool launch_window_tc(const AttnParams& p, int qkv_dtype, int max_rows, int groups, cudaStream_t st) {
  if (p.D != TA_D || !(qkv_dtype == ASPA_BF16 || qkv_dtype == ASPA_I8) || p.cand != nullptr || p.add_mask != nullptr)
    return false;
  const dim3 grid((unsigned)ceil_div(max_rows, TA_BM), groups > 0 ? groups : p.heads);
  bool* flag = ta_attr_flag(qkv_dtype == ASPA_BF16 ? 0 : 1);
  if (flag == nullptr) return false;
  if (qkv_dtype == ASPA_BF16) {
    if (!*flag) { cudaFuncSetAttribute(attn_window_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM); *flag = true; }
    attn_window_tc_kernel<__nv_bfloat16><<<grid, TA_THREADS, TA_SMEM, st>>>(p, TC_SPIN_LIMIT);
  } else {
    if (!*flag) { cudaFuncSetAttribute(attn_window_tc_kernel<int8_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM); *flag = true; }
    attn_window_tc_kernel<int8_t><<<grid, TA_THREADS, TA_SMEM, st>>>(p, TC_SPIN_LIMIT);
  }
  return true;
}

}  // namespace aspa

using namespace aspa;

#ifdef TA_TIMING
extern "C" int aspa_attn_tc_debug(int flags) {
  cudaMemcpyToSymbol(g_ta_debug, &flags, sizeof(int));
  return ASPA_OK;
}
extern "C" int aspa_attn_tc_timing(unsigned long long* host16, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host16, g_ta_cycles, sizeof(unsigned long long) * 16);
  if (reset) {
    unsigned long long z[16] = {};
    cudaMemcpyToSymbol(g_ta_cycles, z, sizeof(z));
  }
  return ASPA_OK;
}
#endif

extern "C" int aspa_attn_tc_status(int reset, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  int host = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&host, g_attn_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    set_error("aspa_attn_tc_status: %s", cudaGetErrorString(e));
    return ASPA_ERR_CUDA;
  }
  if (host == 0) return ASPA_OK;
  if (reset) {
    const int zero = 0;
    cudaMemcpyToSymbolAsync(g_attn_tc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st);
    cudaStreamSynchronize(st);
  }
  set_error("a bounded device-side wait ran out in the tensor-core window attention (wait %d); its outputs are invalid", host);
  return ASPA_ERR_TIMEOUT;
}
