// Window attention on the 5th-generation tensor cores (head_dim 64, bf16 or int8 inputs).
//
// Same job as attn_window_kernel (attention.cu): a CTA owns consecutive packed rows of one head (or of one
// (head, token % stride) group in the anchor pass), streams the union key range of those rows through shared memory
// and keeps a per-row online softmax.  Here the tile is 128 rows x 128 keys and both products run as tcgen05.mma with
// the accumulators in tensor memory:
//     S = Q K^T   (M 128, N 128, K 64: four instructions)      -> tensor memory, double buffered
//     O_j = P V   (M 128, N 64,  K 128: eight instructions)    -> tensor memory, double buffered, one per key tile
// Roles (nine warps):
//   warps 0..3  softmax: thread r owns row r = tensor-memory lane r.  Reads S with tcgen05.ld (once for the row
//               maximum, once for the exponentials: a 128-column row does not fit the register file beside the 64
//               output accumulators), writes P as 16-bit values into a 128-byte-swizzled shared-memory operand, and
//               folds the finished O_{j-1} into its fp32 accumulators (o = o * c_{j-1} + O_{j-1}) while the tensor
//               core is busy with tile j.  A warp whose 32 rows cannot see a key tile skips it altogether.
//   warps 4..7  producers: K and V tiles into a three-stage ring.  bf16 rows arrive by cp.async into the swizzled
//               layout; int8 rows are loaded one tile ahead into registers and widened to fp16 on the way (0x6400 | byte
//               is the half 1024 + byte, one subtraction gives the signed value: exact).  Rows may have any
//               16-byte-aligned stride (the anchor pass reads every stride-th key), which is why this is not a TMA box.
//   warp 8      allocates tensor memory, issues every tcgen05.mma and tcgen05.commit, frees tensor memory.
// int8 inputs run as fp16 x fp16 (values up to 127 and their 64-term dot products are exact in fp32 accumulation),
// P is fp16 there; bf16 inputs run as bf16 x bf16 with P in bf16.  V is used where it lies, as the MN-major B operand.
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
constexpr int TA_STAGES = 3;
constexpr int TA_TILE = TA_BN * 128;       // bytes of one K or V tile: 128 rows of 128 bytes
constexpr int TA_Q_BYTES = TA_BM * 128;
constexpr int TA_P_BYTES = TA_BM * 256;    // two 64-key blocks of 128 rows x 128 bytes
constexpr int TA_THREADS = 9 * 32;
constexpr int TA_TAIL = 2048;              // row tables (2 x 128 ints), mbarriers, tensor-memory slot, abort flag
constexpr int TA_SMEM = 1024 + TA_Q_BYTES + TA_STAGES * 2 * TA_TILE + 2 * TA_P_BYTES + TA_TAIL;
constexpr uint32_t TA_TMEM_COLS = 512;     // S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384)
constexpr int TA_ABSENT = -2147483647;

__device__ int g_attn_tc_status;           // non-zero after a bounded wait ran out in any CTA of any launch

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
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
  unsigned char* p_s = kv_s + S * 2 * TA_TILE;
  unsigned char* tail = p_s + 2 * TA_P_BYTES;
  int* ts = reinterpret_cast<int*>(tail);            // per tile row: its token (anchor pass: strided position), or ABSENT
  int* grow_s = ts + TA_BM;                          // per tile row: row of the head-grouped packing (workspace row)
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail + 1024);
  const uint32_t kv_full0 = s_addr(bars), kv_empty0 = s_addr(bars + S), s_full0 = s_addr(bars + 2 * S),
                 p_ready0 = s_addr(bars + 2 * S + 2), o_full0 = s_addr(bars + 2 * S + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 6);
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
      mbar_init(kv_full0 + 8 * s, 4 * 32);         // every producer thread
      mbar_init(kv_empty0 + 8 * s, 1);             // one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full0 + 8 * b, 1);
      mbar_init(p_ready0 + 8 * b, TA_BM);          // every softmax thread
      mbar_init(o_full0 + 8 * b, 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) tmem_alloc(s_addr(tmem_slot), TA_TMEM_COLS);
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

    if (warp >= 4 && warp < 8) {
      // ---- producers ---------------------------------------------------------------------------------------
      const int pt = tid - 128;
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
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const int id = pt + 128 * c, row = id >> 3, ch = id & 7;
            const int key = kb + row;
            const int64_t kc = min(key, Tn - 1);
            const int nbytes = key < Tn ? 16 : 0;
            cp_async16(smem_u32(ks + ta_swz(row, ch)), kh + kc * k_ts + ch * 8, nbytes);
            cp_async16(smem_u32(ks + TA_TILE + ta_swz(row, ch)), vh + kc * v_ts + ch * 8, nbytes);
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
        uint4 nk[4], nv[4];
        auto fetch = [&](int i) {
          const int kb = (kt_begin + i) * TA_BN;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int id = pt + 128 * c, row = id >> 2, rc = id & 3;
            const int key = kb + row;
            nk[c] = nv[c] = make_uint4(0, 0, 0, 0);
            if (key < Tn) {
              nk[c] = *reinterpret_cast<const uint4*>(kh + (int64_t)key * k_ts + rc * 16);
              nv[c] = *reinterpret_cast<const uint4*>(vh + (int64_t)key * v_ts + rc * 16);
            }
          }
        };
        if (ntiles > 0) fetch(0);
        for (int i = 0; i < ntiles; ++i) {
          const uint32_t it = g_it + i;
          const int s = (int)(it % S);
          uint4 ck[4], cv[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) { ck[c] = nk[c]; cv[c] = nv[c]; }
          if (i + 1 < ntiles) fetch(i + 1);
          if (aborted(abort_flag)) break;
          if (!mbar_wait(kv_empty0 + 8 * s, ((it / S) & 1u) ^ 1u, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 1); break;
          }
          unsigned char* ks = kv_s + s * 2 * TA_TILE;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int id = pt + 128 * c, row = id >> 2, rc = id & 3;
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
    } else if (warp == 8) {
      // ---- MMA issuer ----------------------------------------------------------------------------------------
      if (lane == 0 && ntiles > 0) {
        const uint32_t q_addr = s_addr(q_s);
        bool ok = true;
        auto issue_qk = [&](int i) {     // S[it & 1] = Q K_i^T
          const uint32_t it = g_it + i;
          const int s = (int)(it % S);
          if (!mbar_wait(kv_full0 + 8 * s, (it / S) & 1u, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 2); ok = false; return;
          }
          tc_fence_after();
          const uint32_t k_addr = s_addr(kv_s + s * 2 * TA_TILE);
          const uint32_t d_tmem = tmem_base + (it & 1u) * TA_BN;
#pragma unroll
          for (int k = 0; k < TA_D / 16; ++k)
            umma_f16(d_tmem, umma_desc_k_sw128(q_addr + k * 32), umma_desc_k_sw128(k_addr + k * 32), idesc_qk, k > 0 ? 1u : 0u);
          umma_commit(s_full0 + 8 * (it & 1u));
        };
        issue_qk(0);
        if (ok && ntiles > 1) issue_qk(1);
        for (int j = 0; j < ntiles && ok; ++j) {
          const uint32_t it = g_it + j, b = it & 1u;
          const int s = (int)(it % S);
          if (aborted(abort_flag)) { ok = false; break; }
          if (!mbar_wait(p_ready0 + 8 * b, (it >> 1) & 1u, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 3); ok = false; break;
          }
          tc_fence_after();
          const uint32_t p_addr = s_addr(p_s + b * TA_P_BYTES);
          const uint32_t v_addr = s_addr(kv_s + s * 2 * TA_TILE + TA_TILE);
          const uint32_t d_tmem = tmem_base + 2 * TA_BN + b * TA_D;
#pragma unroll
          for (int k = 0; k < TA_BN / 16; ++k)   // 16 keys per instruction: 32 bytes along a P row, 16 rows of V
            umma_f16(d_tmem, umma_desc_k_sw128(p_addr + (k >> 2) * (TA_BM * 128) + (k & 3) * 32),
                     umma_desc_k_sw128(v_addr + k * 16 * 128), idesc_pv, k > 0 ? 1u : 0u);
          umma_commit(o_full0 + 8 * b);        // O_j complete (and every earlier instruction)
          umma_commit(kv_empty0 + 8 * s);      // K_j and V_j have been read: the stage may be refilled
          if (j + 2 < ntiles) issue_qk(j + 2); // S[b] was read by the softmax warps before they signalled P_j
        }
        if (ok) {   // nothing may still be running when shared or tensor memory is reused
          const uint32_t last = g_it + ntiles - 1;
          if (!mbar_wait(o_full0 + 8 * (last & 1u), (last >> 1) & 1u, spin)) {
            atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 4);
          }
        }
      }
    } else {
      // ---- softmax warps: thread r owns row r ----------------------------------------------------------------------
      const int r = tid;
      const int tr_raw = ts[r];
      const bool present = tr_raw != TA_ABSENT;
      const int tr = present ? tr_raw : -1;
      const int hi_key = tr, lo_key = tr < 0 ? 0 : max(tr - window + 1, 0);   // valid keys [lo_key, hi_key]; none if tr < 0
      const int w_last = __reduce_max_sync(0xffffffffu, tr);
      const int w_first = __reduce_min_sync(0xffffffffu, tr < 0 ? 0x7fffffff : tr);
      const bool w_any = w_last >= 0;
      const int w_lo = w_any ? max(0, w_first - window + 1) : 0;
      const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
      const int64_t gr = grow_s[r];

      float m = -INFINITY, l = 0.f;
      float o[TA_D];
#pragma unroll
      for (int d = 0; d < TA_D; ++d) o[d] = 0.f;
      if (p.read_partial && present) {
        const float mw = p.ws_m[gr];
        m = (mw == -INFINITY) ? -INFINITY : mw * 1.4426950408889634f;
        l = p.ws_l[gr];
#pragma unroll
        for (int d = 0; d < TA_D; d += 2) {   // the workspace rows start on 8-byte boundaries only
          const float2 f = *reinterpret_cast<const float2*>(p.ws_o + gr * TA_D + d);
          o[d] = f.x; o[d + 1] = f.y;
        }
      }
      float c_prev = 1.f;
      bool prev_active = false, ok = true;
      auto fold = [&](uint32_t itp) {   // o = o * c_prev + O_{itp}
        const uint32_t bp = itp & 1u;
        if (!mbar_wait(o_full0 + 8 * bp, (itp >> 1) & 1u, spin)) {
          atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 5); ok = false; return;
        }
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float v[32];
          tmem_ld32(t_lane + 2 * TA_BN + bp * TA_D + h * 32, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[h * 32 + i] = fmaf(o[h * 32 + i], c_prev, v[i]);
        }
      };
      for (int j = 0; j < ntiles && ok; ++j) {
        const uint32_t it = g_it + j, b = it & 1u;
        const int kb = (kt_begin + j) * TA_BN;
        const bool active = w_any && kb <= w_last && kb + TA_BN - 1 >= w_lo;   // warp-uniform
        float c_j = 1.f;
        if (aborted(abort_flag)) { ok = false; break; }
        // Every warp waits for S_j, also one that skips the tile: S_j is issued only after P_{j-2} was signalled by all
        // 128 threads, so passing this wait is what tells a warp that its next arrival on that barrier belongs to the
        // phase of tile j and not to the one of tile j-2 (a warp running ahead would be counted twice in one phase).
        if (!mbar_wait(s_full0 + 8 * b, (it >> 1) & 1u, spin)) {
          atomicExch(abort_flag, 1); atomicExch(&g_attn_tc_status, 6); ok = false; break;
        }
        if (active) {
          tc_fence_after();
          const uint32_t t_s = t_lane + b * TA_BN;
          // valid columns of this row inside the tile: [clo, clo + span]; an empty range is (huge, 0)
          const bool some = hi_key >= lo_key && hi_key >= kb && lo_key <= kb + TA_BN - 1;
          const int clo = some ? max(lo_key - kb, 0) : (1 << 20);
          const uint32_t span = some ? (uint32_t)(min(hi_key - kb, TA_BN - 1) - clo) : 0u;
          const bool all_full = __all_sync(0xffffffffu, some && clo == 0 && span == TA_BN - 1);
          unsigned chunk_live = 0;
          float mx = -INFINITY;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const bool live = all_full || __any_sync(0xffffffffu, some && clo <= c4 * 32 + 31 && clo + (int)span >= c4 * 32);
            if (!live) continue;
            chunk_live |= 1u << c4;
            float v[32];
            tmem_ld32(t_s + c4 * 32, v);
            if (all_full) {
#pragma unroll
              for (int i = 0; i < 32; ++i) mx = fmaxf(mx, v[i]);
            } else {
              const int cb = c4 * 32 - clo;
#pragma unroll
              for (int i = 0; i < 32; ++i) mx = fmaxf(mx, (uint32_t)(cb + i) <= span ? v[i] : -INFINITY);
            }
          }
          const float m_new = fmaxf(m, mx * sc_log2);
          c_j = (m == -INFINITY) ? 0.f : ex2_approx(m - m_new);
          const float base = (m_new == -INFINITY) ? 0.f : m_new;
          unsigned char* prow = p_s + b * TA_P_BYTES + r * 128;
          float sum = 0.f;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t w[16];
            if (chunk_live & (1u << c4)) {
              float v[32];
              tmem_ld32(t_s + c4 * 32, v);
              const int cb = c4 * 32 - clo;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                float sv = fmaf(v[i], sc_log2, -base);
                if (!all_full) sv = (uint32_t)(cb + i) <= span ? sv : -INFINITY;
                v[i] = ex2_approx(sv);
                sum += v[i];
              }
#pragma unroll
              for (int i = 0; i < 16; ++i) w[i] = pack_p<T>(v[2 * i], v[2 * i + 1]);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i) w[i] = 0u;
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {   // 16-byte chunk cc of the 256-byte P row: block cc / 8, chunk cc % 8
              const int cc = c4 * 4 + q4;
              *reinterpret_cast<uint4*>(prow + (cc >> 3) * (TA_BM * 128) + (((cc & 7) ^ (r & 7)) << 4)) =
                  make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
            }
          }
          l = l * c_j + sum;
          m = m_new;
        }
        fence_proxy_async();     // P of this row (if written) is visible to the tensor core's reads
        tc_fence_before();       // ... and this thread's reads of S[b] are complete
        mbar_arrive(p_ready0 + 8 * b);
        if (prev_active) fold(it - 1);
        c_prev = c_j;
        prev_active = active;
      }
      if (ok && prev_active) fold(g_it + ntiles - 1);
      if (ok && present) {
        if (p.write_partial) {
          p.ws_m[gr] = (m == -INFINITY) ? -INFINITY : m * 0.6931471805599453f;   // natural-log domain
          p.ws_l[gr] = l;
#pragma unroll
          for (int d = 0; d < TA_D; d += 2)
            *reinterpret_cast<float2*>(p.ws_o + gr * TA_D + d) = make_float2(o[d], o[d + 1]);
        } else {
          float inv = l > 0.f ? 1.f / l : 0.f;
          if (kI8) inv *= p.v_scale[bh];
          const int tok = anchor ? p.token_idx[gr] : tr;
          const int64_t ob = out_row_base(p, bh, tok);
          if (p.out_dtype == ASPA_BF16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + ob;
#pragma unroll
            for (int d = 0; d < TA_D; d += 8)
              *reinterpret_cast<uint4*>(dst + d) =
                  make_uint4(pack_bf16(o[d] * inv, o[d + 1] * inv), pack_bf16(o[d + 2] * inv, o[d + 3] * inv),
                             pack_bf16(o[d + 4] * inv, o[d + 5] * inv), pack_bf16(o[d + 6] * inv, o[d + 7] * inv));
          } else {
            float* dst = reinterpret_cast<float*>(p.out) + ob;
#pragma unroll
            for (int d = 0; d < TA_D; d += 4)
              *reinterpret_cast<float4*>(dst + d) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
          }
        }
      }
    }
    g_it += (uint32_t)ntiles;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
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
