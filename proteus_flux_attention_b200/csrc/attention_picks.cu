// Prototype-pick pass of the shortlist on warp-level tensor-core tiles (head_dim 64, int8 or bf16 q / k / v).
//
// The picks of a row are a prefix of the score-sorted list of its 128-token block (aspa_proto_plan), filtered by the
// row's own window, anchors and length (reference kernels/sparse_attn.py:260-596: the dedup of the candidate
// builder).  All rows of one (head, block) pair therefore walk the SAME list: one warp takes such a pair, up to 16 of
// its rows at a time as the M dimension of mma.sync tiles, and reads every key and value row once for all of them,
// where the row kernel reads them once per row and spends about 700 CUDA-core instructions per 32 keys of one row.
//
//   int8:  S = Q K^T   mma.sync m16n8k32 s8 x s8 -> s32 (the exact integer dot the row kernel computes with dp4a)
//          O += P V    mma.sync m16n8k16 f16 x f16 -> f32, P rounded to fp16, V widened exactly from int8 to fp16
//   bf16:  both products mma.sync m16n8k16 bf16 x bf16 -> f32, P rounded to bf16 (as in the window tile kernel)
//
// No shared memory: fragments are loaded straight from global memory.  The K dimension of S (channels) and the N
// dimension of O (channels) may be permuted freely as long as both operands agree, so a thread takes the 16 contiguous
// channels [16q, 16q+16) of a key row (q = lane % 4) and the 8 contiguous channels [8g, 8g+8) of a value row
// (g = lane / 4) instead of the scattered elements the canonical fragment layout would ask for.
#include "attn_params.cuh"

namespace aspa {

constexpr int PK_WARPS = 4;
#ifndef PK_MIN_BLOCKS
#define PK_MIN_BLOCKS 5
#endif

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_f32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// bytes (lo, hi) = two int8 with their sign bits flipped -> the two values as an fp16 pair: 0x6400 | u is 1024 + u,
// and 1024 + u - 1152 = u - 128 is the signed value (exact)
__device__ __forceinline__ uint32_t flipped_bytes_to_half2(uint32_t pair_word, uint32_t sel) {
  const uint32_t w = __byte_perm(pair_word, 0x64646464u, sel);
  const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&w), __floats2half2_rn(1152.f, 1152.f));
  return *reinterpret_cast<const uint32_t*>(&v);
}

// First index in tok[0, n) (ascending) whose value is >= target; all lanes take part and get the answer.
__device__ __forceinline__ int warp_lower_bound(const int32_t* __restrict__ tok, int n, int target, int lane) {
  int lo = 0, hi = n;   // the answer lies in [lo, hi]
  while (lo < hi) {
    const int stride = (hi - lo + 31) >> 5;
    const int pos = lo + (lane + 1) * stride - 1;
    const int v = pos < hi ? tok[pos] : 0x7fffffff;
    const unsigned ge = __ballot_sync(0xffffffffu, v >= target);
    if (ge == 0u) return hi;
    const int f = __ffs(ge) - 1;
    const int top = lo + (f + 1) * stride - 1;
    lo += f * stride;
    hi = top < hi ? top : hi;
  }
  return lo;
}

struct PickRow {
  int t, loc_start, limit, tmod, alo;   // anchor groups: limit = last strided key index of the row, alo = its first
  bool present, clamp_slot, aclamps;
};

// What the rows of a warp's group share: MODE 0 the score-sorted pick list of their 128-token block (rows of one head
// and block), MODE 1 the strided key sequence K[rho + stride * i] of their residue class rho = token % stride (rows of
// one head and residue, regrouped by anchor_regroup_kernel) - the anchors t - j * stride of such rows are windows over it.
constexpr int PK_PICKS = 0, PK_ANCHORS = 1;

template <typename T, int MODE>
__global__ void __launch_bounds__(PK_WARPS * 32, sizeof(T) == 1 ? PK_MIN_BLOCKS : 4) attn_picks_tile_kernel(const AttnParams p) {
  constexpr bool I8 = sizeof(T) == 1;
  constexpr int QW = I8 ? 4 : 8;   // 32-bit words of a thread's 16 channels of a q or k row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  const int bh = blockIdx.y;
  const int PB = MODE == PK_PICKS ? p.plan.proto_block : 1;
  const int nblk = MODE == PK_PICKS ? (p.T + PB - 1) / PB : p.an_stride;   // groups per head
  const int blk = blockIdx.x * PK_WARPS + warp;                             // block of the sequence, or residue class
  if (blk >= nblk) return;
  const int start = p.row_offsets[bh];
  const int cnt = p.row_offsets[bh + 1] - start;
  if (cnt <= 0) return;
  const int32_t* toks = p.token_idx + start;
  int r_lo, r_hi;   // MODE 0: rows of the head (positions in its packing); MODE 1: positions in the regrouped arrays
  if (MODE == PK_PICKS) {
    r_lo = warp_lower_bound(toks, cnt, blk * PB, lane);
    if (r_lo >= cnt) return;
    const int span = min(cnt - r_lo, PB);   // a block holds at most PB rows of one head
    r_hi = r_lo + warp_lower_bound(toks + r_lo, span, (blk + 1) * PB, lane);
  } else {
    r_lo = p.an_offsets[bh * nblk + blk];
    r_hi = p.an_offsets[bh * nblk + blk + 1];
  }
  if (r_hi <= r_lo) return;

  const int Tn = p.T;
  const int b = bh / p.H;
  const T* qh = reinterpret_cast<const T*>(p.q) + (int64_t)bh * Tn * 64;
  const T* kh = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.kv.k_batch + (int64_t)(bh % p.H) * p.kv.k_head;
  const T* vh = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.kv.v_batch + (int64_t)(bh % p.H) * p.kv.v_head;
  const int64_t k_ts = p.kv.k_token, v_ts = p.kv.v_token;
  const float LOG2E = 1.4426950408889634f;
  const float sc2 = (I8 ? p.scale * p.q_scale[bh] * p.k_scale[bh] : p.scale) * LOG2E;   // scores in the log2 domain
  const float vscale = I8 ? p.v_scale[bh] : 1.f;
  const int32_t* plist = MODE == PK_PICKS ? p.plan.proto_lists + ((int64_t)b * nblk + blk) * p.plan.proto_list_stride : nullptr;
  const int astride = max(1, p.plan.anchor_stride);
  const int n_at = p.plan.anchor_stride > 0 ? p.plan.anchor_slots : 0;
  const bool pow2 = (astride & (astride - 1)) == 0;
  const int window = p.plan.window;

  for (int rt = r_lo; rt < r_hi; rt += 16) {
    // rows g and g + 8 of this sub-tile
    PickRow row[2];
    uint32_t qa[2][QW];
    int64_t grow[2];   // row of the head-grouped packing = workspace row
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rt + g + 8 * h;
      PickRow& R = row[h];
      R.present = r < r_hi;
      grow[h] = !R.present ? 0 : (MODE == PK_PICKS ? (int64_t)start + r : (int64_t)p.an_row[r]);
      R.t = R.present ? p.token_idx[grow[h]] : 0;
      const int n_loc = window > 0 ? min(R.t + 1, window) : 1;
      R.loc_start = R.t - n_loc + 1;
      R.tmod = pow2 ? (R.t & (astride - 1)) : (R.t % astride);
      const int j0 = R.t / astride + 1;   // the anchor slot that clamps to key 0
      const bool clamp_row = R.present && n_at > 0 && j0 <= n_at && R.tmod != 0 && R.loc_start > 0;
      if (MODE == PK_PICKS) {
        R.limit = R.present ? p.plan.proto_limit[(int64_t)b * Tn + R.t] : 0;
        R.alo = R.t - n_at * astride;
        R.aclamps = n_at > 0 && R.alo < 0;
        // the one anchor slot the 64-row tile pass leaves to this pass (the group pass takes it itself: anchors_done 2)
        R.clamp_slot = clamp_row && p.anchors_done == 1;
      } else {
        // strided key indices [alo, limit]: the last anchor outside the window back to slot n_at (an_tok holds
        // token / stride - jmin, or ANCHOR_NO_KEYS for a row whose window reaches key 0)
        R.limit = R.present ? p.an_tok[r] : ANCHOR_NO_KEYS;
        R.alo = max(0, R.t / astride - n_at);
        R.aclamps = false;
        R.clamp_slot = clamp_row;
      }
#pragma unroll
      for (int i = 0; i < QW / 4; ++i) {
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        if (R.present) w = reinterpret_cast<const uint4*>(qh + (int64_t)R.t * 64 + 16 * q)[i];
        qa[h][4 * i] = w.x; qa[h][4 * i + 1] = w.y; qa[h][4 * i + 2] = w.z; qa[h][4 * i + 3] = w.w;
      }
    }
    int max_limit = max(row[0].limit, row[1].limit);
    int min_lo = 0x7fffffff;
    if (MODE == PK_ANCHORS) min_lo = min(row[0].limit >= row[0].alo ? row[0].alo : min_lo, row[1].limit >= row[1].alo ? row[1].alo : min_lo);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      max_limit = max(max_limit, __shfl_xor_sync(0xffffffffu, max_limit, off));
      min_lo = min(min_lo, __shfl_xor_sync(0xffffffffu, min_lo, off));
    }
    // slot 0: key 0 for the rows with the clamping anchor slot; slot s >= 1: list entry s - 1, or strided key min_lo + s - 1
    const int n_slots = MODE == PK_PICKS ? max_limit + 1 : (max_limit >= min_lo ? max_limit - min_lo + 2 : 1);
    if (MODE == PK_ANCHORS && max_limit < min_lo) min_lo = 0;   // no row of the sub-tile has an anchor key

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;

    for (int s0 = 0; s0 < n_slots; s0 += 32) {
      // ---- S = Q K^T for 32 slots: n-tile nt covers slots s0 + 8 nt + (0..7); this thread loads the key of column g
      int u_own[4];
      float c[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int slot = s0 + 8 * nt + g;
        if (MODE == PK_PICKS) u_own[nt] = slot == 0 ? 0 : (slot <= max_limit ? plist[slot - 1] : -1);
        else u_own[nt] = slot == 0 ? 0 : (slot < n_slots ? blk + astride * (min_lo + slot - 1) : -1);
        const uint4* krow = reinterpret_cast<const uint4*>(kh + (int64_t)max(u_own[nt], 0) * k_ts + 16 * q);
        if (I8) {
          const uint4 kw = krow[0];
          int ci[4] = {0, 0, 0, 0};
          mma_s8(ci, qa[0][0], qa[1][0], qa[0][1], qa[1][1], kw.x, kw.y);
          mma_s8(ci, qa[0][2], qa[1][2], qa[0][3], qa[1][3], kw.z, kw.w);
          c[nt][0] = (float)ci[0]; c[nt][1] = (float)ci[1]; c[nt][2] = (float)ci[2]; c[nt][3] = (float)ci[3];
        } else {
          const uint4 k0 = krow[0], k1 = krow[1];
          const uint32_t kw[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
          c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)   // 16 channels per step: words 2 ks and 2 ks + 1 of both operands
            mma_bf16_f32(c[nt], qa[0][(2 * ks) % QW], qa[1][(2 * ks) % QW], qa[0][(2 * ks + 1) % QW], qa[1][(2 * ks + 1) % QW],
                         kw[2 * ks], kw[2 * ks + 1]);
        }
      }
      // ---- masks and scores: this thread holds columns 2q, 2q+1 of every n-tile for rows g (c0, c1) and g+8 (c2, c3)
      int ucol[4][2];
      float s[4][4];
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int u = __shfl_sync(0xffffffffu, u_own[nt], 4 * (2 * q + j));
          ucol[nt][j] = u;
          const int slot = s0 + 8 * nt + 2 * q + j;
          const int umod = pow2 ? (u & (astride - 1)) : (u >= 0 ? u % astride : 0);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const PickRow& R = row[h];
            bool ok;
            if (slot == 0) {
              ok = R.clamp_slot;
            } else if (MODE == PK_PICKS) {
              ok = R.present && slot <= R.limit && u >= 0 && u < R.loc_start;
              if (n_at > 0) ok = ok && !((umod == R.tmod && u >= R.alo) || (u == 0 && R.aclamps));
            } else {
              const int i = min_lo + slot - 1;
              ok = R.present && u >= 0 && i >= R.alo && i <= R.limit;
            }
            const float v = ok ? c[nt][2 * h + j] * sc2 : -INFINITY;
            s[nt][2 * h + j] = v;
            mx[h] = fmaxf(mx[h], v);
          }
        }
      }
      float corr[2], msafe[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h]);
        msafe[h] = m_new == -INFINITY ? 0.f : m_new;
        corr[h] = exp2f(m[h] - msafe[h]);   // 0 while the row has seen nothing
        m[h] = m_new;
        l[h] *= corr[h];
      }
      // ---- P (fp16 fragments) and the row sums
      uint32_t pa[4][2];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float p0 = exp2f(s[nt][2 * h] - msafe[h]), p1 = exp2f(s[nt][2 * h + 1] - msafe[h]);
          l[h] += p0 + p1;
          pa[nt][h] = I8 ? pack_half2(p0, p1) : pack_bf162(p0, p1);
        }
      }
      if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {   // most steps move no row's maximum
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
          o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
        }
      }
      // ---- O += P V: two k16 steps; the keys of step kk are the columns this thread already knows
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        if (I8) {
          uint2 vr[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int u = ucol[2 * kk + (i >> 1)][i & 1];   // k index 2q, 2q+1, 2q+8, 2q+9 of this step
            vr[i] = *reinterpret_cast<const uint2*>(vh + (int64_t)max(u, 0) * v_ts + 8 * g);
            vr[i].x ^= 0x80808080u;
            vr[i].y ^= 0x80808080u;
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {   // channels 8g + 4 half + (0..3): n-tiles 4 half + (0..3)
            const uint32_t k0 = half ? vr[0].y : vr[0].x, k1 = half ? vr[1].y : vr[1].x;
            const uint32_t k2 = half ? vr[2].y : vr[2].x, k3 = half ? vr[3].y : vr[3].x;
            const uint32_t lo01 = __byte_perm(k0, k1, 0x5140), hi01 = __byte_perm(k0, k1, 0x7362);   // (k0c, k1c) byte pairs
            const uint32_t lo23 = __byte_perm(k2, k3, 0x5140), hi23 = __byte_perm(k2, k3, 0x7362);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const uint32_t w01 = cc < 2 ? lo01 : hi01, w23 = cc < 2 ? lo23 : hi23;
              const uint32_t sel = (cc & 1) ? 0x4342u : 0x4140u;
              const uint32_t b0 = flipped_bytes_to_half2(w01, sel), b1 = flipped_bytes_to_half2(w23, sel);
              mma_f16(o[4 * half + cc], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1], b0, b1);
            }
          }
        } else {
          uint4 vr[4];   // channels 8g .. 8g+7 of the four value rows, two bf16 per word
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int u = ucol[2 * kk + (i >> 1)][i & 1];
            vr[i] = *reinterpret_cast<const uint4*>(vh + (int64_t)max(u, 0) * v_ts + 8 * g);
          }
#pragma unroll
          for (int cw = 0; cw < 4; ++cw) {   // word cw holds channels 8g + 2 cw and 8g + 2 cw + 1: n-tiles 2 cw, 2 cw + 1
            const uint32_t a0 = cw == 0 ? vr[0].x : cw == 1 ? vr[0].y : cw == 2 ? vr[0].z : vr[0].w;
            const uint32_t a1 = cw == 0 ? vr[1].x : cw == 1 ? vr[1].y : cw == 2 ? vr[1].z : vr[1].w;
            const uint32_t a2 = cw == 0 ? vr[2].x : cw == 1 ? vr[2].y : cw == 2 ? vr[2].z : vr[2].w;
            const uint32_t a3 = cw == 0 ? vr[3].x : cw == 1 ? vr[3].y : cw == 2 ? vr[3].z : vr[3].w;
            // (key 2q, key 2q+1) of the even channel, then of the odd one
            mma_bf16_f32(o[2 * cw], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1],
                         __byte_perm(a0, a1, 0x5410), __byte_perm(a2, a3, 0x5410));
            mma_bf16_f32(o[2 * cw + 1], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1],
                         __byte_perm(a0, a1, 0x7632), __byte_perm(a2, a3, 0x7632));
          }
        }
      }
    }

    // ---- merge with the state the window and anchor passes left, normalise, store
    float m1_in[2], l1_in[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
      m1_in[h] = row[h].present ? p.ws_m[grow[h]] : -INFINITY;
      l1_in[h] = row[h].present ? p.ws_l[grow[h]] : 0.f;
    }
    __syncwarp();   // every lane of a row has read its old maximum and sum before one of them replaces them (write_partial)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const PickRow& R = row[h];
      if (!R.present) continue;
      const int64_t gr = grow[h];
      const float m1n = m1_in[h], l1 = l1_in[h];
      const float m1 = m1n == -INFINITY ? -INFINITY : m1n * LOG2E;
      const float mm = fmaxf(m[h], m1);
      const float c1 = m1 == -INFINITY ? 0.f : exp2f(m1 - mm);
      const float c2 = m[h] == -INFINITY ? 0.f : exp2f(m[h] - mm);
      const float lt = l1 * c1 + l[h] * c2;
      float* wo = p.ws_o + gr * 64;
      if (p.write_partial) {   // another pass follows: leave the merged state (natural-log maximum, raw P.V) behind
        if (q == 0) {
          p.ws_m[gr] = mm == -INFINITY ? -INFINITY : mm * 0.6931471805599453f;
          p.ws_l[gr] = lt;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int nt = 0; nt < 8; ++nt) {
            const int ch = 8 * (2 * q + j) + nt;
            wo[ch] = wo[ch] * c1 + o[nt][2 * h + j] * c2;
          }
        }
        continue;
      }
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      const int64_t ob = out_row_base(p, bh, R.t);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const int ch = 8 * (2 * q + j) + nt;   // column 2q + j of n-tile nt is channel 8 (2q + j) + nt
          store_out(p, ob + ch, (wo[ch] * c1 + o[nt][2 * h + j] * c2) * inv * vscale);
        }
      }
    }
  }
}

// What is left when the 64-row tile passes have taken window and anchors and the plan has no prototype picks: the one
// anchor slot that clamps to key 0 (rows whose last anchor would fall below the sequence start) and the normalisation of
// the state in the workspace.  One warp per row, two channels per lane.
template <typename T>
__global__ void __launch_bounds__(256) attn_finalise_rows_kernel(const AttnParams p) {
  constexpr bool I8 = sizeof(T) == 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int start = p.row_offsets[bh];
  const int cnt = p.row_offsets[bh + 1] - start;
  const int r = blockIdx.x * 8 + warp;
  if (r >= cnt) return;
  const int64_t grow = (int64_t)start + r;
  const int t = p.token_idx[grow];
  const int b = bh / p.H;
  const int astride = max(1, p.plan.anchor_stride);
  const int n_at = p.plan.anchor_stride > 0 ? p.plan.anchor_slots : 0;
  const int n_loc = p.plan.window > 0 ? min(t + 1, p.plan.window) : 1;
  const bool clamp = p.anchors_done == 1 && n_at > 0 && t / astride + 1 <= n_at && (t % astride) != 0 && t - n_loc + 1 > 0;
  const float m1 = p.ws_m[grow], l1 = p.ws_l[grow];
  float c1 = 1.f, c2 = 0.f, lt = l1;
  float v0 = 0.f, v1 = 0.f;
  if (clamp) {   // warp-uniform
    const T* qr = reinterpret_cast<const T*>(p.q) + ((int64_t)bh * p.T + t) * 64;
    const T* k0 = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.kv.k_batch + (int64_t)(bh % p.H) * p.kv.k_head;
    const T* vr = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.kv.v_batch + (int64_t)(bh % p.H) * p.kv.v_head;
    float dot;
    if (I8) {
      const char2 a = reinterpret_cast<const char2*>(qr)[lane], kk = reinterpret_cast<const char2*>(k0)[lane];
      const char2 vv = reinterpret_cast<const char2*>(vr)[lane];
      dot = (float)((int)a.x * (int)kk.x + (int)a.y * (int)kk.y);
      v0 = (float)vv.x; v1 = (float)vv.y;
    } else {
      const float2 a = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(qr)[lane]);
      const float2 kk = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(k0)[lane]);
      const float2 vv = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(vr)[lane]);
      dot = a.x * kk.x + a.y * kk.y;
      v0 = vv.x; v1 = vv.y;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float s = dot * (I8 ? p.scale * p.q_scale[bh] * p.k_scale[bh] : p.scale);
    const float mm = fmaxf(s, m1);
    c1 = m1 == -INFINITY ? 0.f : __expf(m1 - mm);
    c2 = __expf(s - mm);
    lt = l1 * c1 + c2;
  }
  const float inv = lt > 0.f ? 1.f / lt : 0.f;
  const float vscale = I8 ? p.v_scale[bh] : 1.f;
  const float2 wo = *reinterpret_cast<const float2*>(p.ws_o + grow * 64 + 2 * lane);
  const int64_t ob = out_row_base(p, bh, t) + 2 * lane;
  store_out(p, ob, (wo.x * c1 + v0 * c2) * inv * vscale);
  store_out(p, ob + 1, (wo.y * c1 + v1 * c2) * inv * vscale);
}

void launch_finalise_rows(const AttnParams& p, int qkv_dtype, int max_rows, cudaStream_t st) {
  const dim3 grid((unsigned)ceil_div(max_rows, 8), (unsigned)p.heads);
  if (qkv_dtype == ASPA_I8) attn_finalise_rows_kernel<int8_t><<<grid, 256, 0, st>>>(p);
  else attn_finalise_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
}

// Whether the pick pass of this call can run on the tile kernel: int8 or bf16, head_dim 64, a structural plan with prototype
// lists, and no anchor slots left to this pass other than the one that clamps to key 0.
bool picks_tiles_ok(const AttnParams& p, int qkv_dtype) {
  if ((qkv_dtype != ASPA_I8 && qkv_dtype != ASPA_BF16) || p.D != 64 || !p.has_plan || p.add_mask != nullptr) return false;
  if (p.plan.proto_cap <= 0 || p.plan.proto_lists == nullptr || p.plan.proto_limit == nullptr || p.plan.proto_block <= 0) return false;
  const bool anchors = p.plan.anchor_stride > 0 && p.plan.anchor_slots > 0;
  return !anchors || p.anchors_done != 0;
}

void launch_picks_tiles(const AttnParams& p, int qkv_dtype, cudaStream_t st) {
  const int nblk = (p.T + p.plan.proto_block - 1) / p.plan.proto_block;
  const dim3 grid((unsigned)ceil_div(nblk, PK_WARPS), (unsigned)p.heads);
  if (qkv_dtype == ASPA_I8) attn_picks_tile_kernel<int8_t, PK_PICKS><<<grid, PK_WARPS * 32, 0, st>>>(p);
  else attn_picks_tile_kernel<__nv_bfloat16, PK_PICKS><<<grid, PK_WARPS * 32, 0, st>>>(p);
}

// The anchors of a call whose (head, residue) groups are too small for the 64-row tile pass: same kernel, one warp per
// group, keys = the strided sequence of the residue class.  `p` carries the regrouped rows (an_*) and says through
// write_partial whether another pass follows.
bool anchor_groups_ok(const AttnParams& p, int qkv_dtype) {
  if ((qkv_dtype != ASPA_I8 && qkv_dtype != ASPA_BF16) || p.D != 64 || !p.has_plan || p.add_mask != nullptr) return false;
  return p.plan.anchor_stride > 0 && p.plan.anchor_slots > 0;
}

void launch_anchor_groups(const AttnParams& p, int qkv_dtype, cudaStream_t st) {
  const dim3 grid((unsigned)ceil_div(p.an_stride, PK_WARPS), (unsigned)p.heads);
  if (qkv_dtype == ASPA_I8) attn_picks_tile_kernel<int8_t, PK_ANCHORS><<<grid, PK_WARPS * 32, 0, st>>>(p);
  else attn_picks_tile_kernel<__nv_bfloat16, PK_ANCHORS><<<grid, PK_WARPS * 32, 0, st>>>(p);
}

}  // namespace aspa
