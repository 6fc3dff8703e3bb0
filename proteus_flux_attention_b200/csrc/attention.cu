// Attention over packed (head, token) rows.
//
//  * attn_rows_kernel   — one warp per row, fp32 math on CUDA cores, any head_dim <= 256, any input dtype.
//                         Candidate keys come from an explicit table, from the structural shortlist plan
//                         (local window + strided anchors + prototype picks, de-duplicated on the fly) or
//                         are "every key <= t".  Also runs as the second pass that adds the gathered extras
//                         (anchors, prototype picks) to the partial softmax state of the window pass.
//  * attn_window_kernel — bf16 tensor-core pass over the contiguous local window: a CTA owns 64
//                         consecutive packed rows of one head, streams the union key range through shared
//                         memory in 64-key tiles, S = Q K^T and O += P V on mma m16n8k16 with fp32
//                         accumulation and per-row window masking (rows are sparse tokens, so 16-row MMA
//                         groups keep the masked-out fraction small).  INT8 inputs are widened to bf16 while
//                         staging (|v| <= 127 is exact in bf16, dot products of 64 such terms are exact in fp32).
#include "attn_params.cuh"
#include "common.cuh"
#include "mma.cuh"

namespace aspa {

// ------------------------------------------------------------------------------------------------
// generic kernel
// ------------------------------------------------------------------------------------------------
constexpr int GEN_WARPS = 8;
constexpr int GEN_MAXD = 256;

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ krow, const float* __restrict__ qs, int D) {
  float acc = 0.f;
  if (sizeof(T) == 2 && (D & 7) == 0) {
    const uint4* kv = reinterpret_cast<const uint4*>(krow);
    for (int c = 0; c < D / 8; ++c) {
      const uint4 raw = kv[c];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
        acc = fmaf(f.x, qs[c * 8 + 2 * i], acc);
        acc = fmaf(f.y, qs[c * 8 + 2 * i + 1], acc);
      }
    }
  } else if (sizeof(T) == 4 && (D & 3) == 0) {
    const float4* kv = reinterpret_cast<const float4*>(krow);
    for (int c = 0; c < D / 4; ++c) {
      const float4 f = kv[c];
      acc = fmaf(f.x, qs[c * 4], acc);
      acc = fmaf(f.y, qs[c * 4 + 1], acc);
      acc = fmaf(f.z, qs[c * 4 + 2], acc);
      acc = fmaf(f.w, qs[c * 4 + 3], acc);
    }
  } else if (sizeof(T) == 1 && (D & 7) == 0) {
    const uint2* kv = reinterpret_cast<const uint2*>(krow);
    for (int c = 0; c < D / 8; ++c) {
      const uint2 raw = kv[c];
      const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf((float)b[i], qs[c * 8 + i], acc);
    }
  } else {
    for (int d = 0; d < D; ++d) acc = fmaf(ld_as_float<T>(krow, d), qs[d], acc);
  }
  return acc;
}

// Elements moved by one vector load of a value row (16 bytes; 8 bytes for int8).
template <typename T> struct VecElems { static constexpr int n = 8; };
template <> struct VecElems<float> { static constexpr int n = 4; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load_vec<float>(const float* p, float (&o)[8]) {
  const float4 f = *reinterpret_cast<const float4*>(p);
  o[0] = f.x; o[1] = f.y; o[2] = f.z; o[3] = f.w;
}
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h2[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load_vec<int8_t>(const int8_t* p, float (&o)[8]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  // int8 -> fp32 without the quarter-rate I2F: flip the sign bit (s + 128 as an unsigned byte), drop the byte into the
  // mantissa of 2^23 (the float 8388608 + s + 128) and subtract 8388736.  Exact for every byte.
  const uint32_t w[2] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u};
#pragma unroll
  for (int i = 0; i < 8; ++i)
    o[i] = __uint_as_float(__byte_perm(w[i >> 2], 0x4B000000u, 0x7440u + (i & 3))) - 8388736.0f;
}

// The candidate list of one packed row as a function of the slot number: an explicit table row, the pieces of a
// structural plan (window, strided anchors, prototype picks, with the duplicates the reference's dedup removes
// skipped), or the causal / masked prefix.
struct RowCands {
  const int64_t* cand_row;
  const int32_t* plist;
  int t, Tn, n_loc, loc_start, n_anchor, n_anchor_true, n_proto, n_virtual, v_begin, astride, j0;
  bool explicit_c, planned, anchor_clamps, anchors_done;

  __device__ __forceinline__ void init(const AttnParams& p, int bh, int64_t grow, int t_, int start, int cnt) {
    t = t_; Tn = p.T;
    explicit_c = p.cand != nullptr;
    planned = !explicit_c && p.has_plan;
    n_loc = 0; loc_start = 0; n_anchor = 0; n_anchor_true = 0; n_proto = 0; n_virtual = 0; v_begin = 0;
    plist = nullptr; cand_row = nullptr;
    astride = 1; j0 = 0;
    anchor_clamps = false;
    anchors_done = p.anchors_done != 0;
    if (explicit_c) {
      long long len = p.cand_len[grow];
      n_virtual = (int)max(1LL, min(len, (long long)p.L));
      cand_row = p.cand + grow * p.L;
    } else if (planned) {
      n_loc = p.plan.window > 0 ? min(t + 1, p.plan.window) : 1;
      loc_start = t - n_loc + 1;
      astride = max(1, p.plan.anchor_stride);
      n_anchor = p.plan.anchor_stride > 0 ? p.plan.anchor_slots : 0;
      j0 = t / astride + 1;  // first anchor slot that clamps to key 0
      anchor_clamps = n_anchor > 0 && (t - (long long)n_anchor * astride) < 0;
      n_anchor_true = n_anchor;
      if (anchors_done && n_anchor > 0) n_anchor = p.anchors_done == 2 ? 0 : 1;  // at most the slot that clamps to key 0 is left to this pass
      if (p.plan.proto_cap > 0 && p.plan.proto_lists != nullptr) {
        const int b = bh / p.H;
        const int nblk = (Tn + p.plan.proto_block - 1) / p.plan.proto_block;
        plist = p.plan.proto_lists + ((int64_t)b * nblk + t / p.plan.proto_block) * p.plan.proto_list_stride;
        n_proto = p.plan.proto_limit[(int64_t)b * Tn + t];
      }
      n_virtual = n_loc + n_anchor + n_proto;
      v_begin = p.extras_only ? n_loc : 0;
    } else {
      const int max_tok = p.token_idx[start + cnt - 1];
      n_virtual = p.add_mask ? max_tok + 1 : t + 1;
    }
  }

  // key index of slot c (< n_virtual), or -1 for a slot that holds nothing
  __device__ __forceinline__ int index_of(int c) const {
    if (explicit_c) {
      const long long raw = cand_row[c];
      return (int)min(max(raw, 0LL), (long long)Tn - 1);
    }
    if (!planned) return c;
    if (c < n_loc) return loc_start + c;
    if (c < n_loc + n_anchor) {
      // after the anchor tile pass the one slot left here is the slot that clamps to key 0, if the row has it
      const int j = anchors_done ? j0 : c - n_loc + 1;
      if (j <= n_anchor_true) {
        const long long a = (long long)t - (long long)j * astride;
        if (a >= 0) {
          if (a < loc_start) return (int)a;
        } else if (j == j0 && (t % astride) != 0 && loc_start > 0) {
          return 0;
        }
      }
      return -1;
    }
    const int u = plist[c - n_loc - n_anchor];
    if (u >= 0 && u < loc_start) {
      bool is_anchor = false;
      if (n_anchor_true > 0) {
        const int dlt = t - u;
        if (dlt % astride == 0 && dlt / astride >= 1 && dlt / astride <= n_anchor_true) is_anchor = true;
        if (u == 0 && anchor_clamps) is_anchor = true;
      }
      if (!is_anchor) return u;
    }
    return -1;
  }
};

// kVec: head_dim / VecElems is a power of two <= 32, so LPR = that many lanes cover one value row with one vector
// load each and 32 / LPR candidates are accumulated per step; otherwise lanes stride over the channels one by one.
template <typename T, bool kVec>
__global__ void __launch_bounds__(GEN_WARPS * 32) attn_rows_kernel(const AttnParams p) {
  __shared__ float qs_all[GEN_WARPS][GEN_MAXD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int start = p.row_offsets[bh];
  const int cnt = p.row_offsets[bh + 1] - start;
  const int r = blockIdx.x * GEN_WARPS + warp;
  if (r >= cnt) return;
  const int64_t grow = (int64_t)start + r;
  const int t = p.token_idx[grow];
  const int D = p.D, Tn = p.T;
  const T* qh = reinterpret_cast<const T*>(p.q) + (int64_t)bh * Tn * D;
  const T* kh = reinterpret_cast<const T*>(p.k) + (bh / p.H) * p.kv.k_batch + (bh % p.H) * p.kv.k_head;
  const T* vh = reinterpret_cast<const T*>(p.v) + (bh / p.H) * p.kv.v_batch + (bh % p.H) * p.kv.v_head;
  const int64_t k_ts = p.kv.k_token, v_ts = p.kv.v_token;
  float* qs = qs_all[warp];
  for (int d = lane; d < D; d += 32) qs[d] = ld_as_float<T>(qh, (int64_t)t * D + d);
  __syncwarp();
  float sc = p.scale;
  float vscale = 1.f;
  if (sizeof(T) == 1) {
    sc *= p.q_scale[bh] * p.k_scale[bh];
    vscale = p.v_scale[bh];
  }

  RowCands rc;
  rc.init(p, bh, grow, t, start, cnt);
  const int n_virtual = rc.n_virtual, v_begin = rc.v_begin;

  float m = -INFINITY, l = 0.f;
  float acc[GEN_MAXD / 32];
#pragma unroll
  for (int i = 0; i < GEN_MAXD / 32; ++i) acc[i] = 0.f;
  constexpr int VE = VecElems<T>::n;
  const int LPR = kVec ? D / VE : 32;          // lanes per value row
  const int grp = lane / LPR, sub = lane % LPR;
  const int groups = 32 / LPR;                  // candidates accumulated per step

  for (int c0 = v_begin; c0 < n_virtual; c0 += 32) {
    const int c = c0 + lane;
    const int idx = c < n_virtual ? rc.index_of(c) : -1;
    float s = -INFINITY;
    if (idx >= 0) {
      // one key row per lane (sharing a row between lanes and reducing with shuffles was measured 20-40 % slower)
      s = dot_row<T>(kh + (int64_t)idx * k_ts, qs, D) * sc;
      if (p.add_mask) s += p.add_mask[(int64_t)t * Tn + idx];
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;  // nothing valid yet (warp-uniform)
    const float pr = (s == -INFINITY) ? 0.f : __expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : __expf(m - m_new);
    l = l * corr + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < GEN_MAXD / 32; ++i) acc[i] *= corr;
    const unsigned live = __ballot_sync(0xffffffffu, pr > 0.f);
    if (kVec && LPR == 8) {
      // head_dim 64 in bf16 / int8: eight steps of four candidates, written without branches so that the eight value
      // loads are independent instructions the scheduler can have in flight together (dead candidates: weight 0, row 0)
#pragma unroll
      for (int st = 0; st < 8; ++st) {
        const float pc = __shfl_sync(0xffffffffu, pr, st * 4 + grp);
        const int ic = max(__shfl_sync(0xffffffffu, idx, st * 4 + grp), 0);
        float vv[8];
        load_vec<T>(vh + (int64_t)ic * v_ts + sub * VE, vv);
#pragma unroll
        for (int e = 0; e < VE; ++e) acc[e] = fmaf(pc, vv[e], acc[e]);
      }
    } else if (kVec) {
      const unsigned gmask = groups == 32 ? 0xffffffffu : ((1u << groups) - 1u);
      for (int c0g = 0; c0g < 32; c0g += groups) {
        if (!((live >> c0g) & gmask)) continue;  // warp-uniform
        const float pc = __shfl_sync(0xffffffffu, pr, c0g + grp);
        const int ic = __shfl_sync(0xffffffffu, idx, c0g + grp);
        if (pc > 0.f) {
          float vv[8];
          load_vec<T>(vh + (int64_t)ic * v_ts + sub * VE, vv);
#pragma unroll
          for (int e = 0; e < VE; ++e) acc[e] = fmaf(pc, vv[e], acc[e]);
        }
      }
    } else {
      for (unsigned rem = live; rem; rem &= rem - 1) {
        const int src = __ffs(rem) - 1;
        const float pc = __shfl_sync(0xffffffffu, pr, src);
        const int ic = __shfl_sync(0xffffffffu, idx, src);
        const T* vrow = vh + (int64_t)ic * v_ts;
#pragma unroll
        for (int i = 0; i < GEN_MAXD / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < D) acc[i] = fmaf(pc, ld_as_float<T>(vrow, d), acc[i]);
        }
      }
    }
  }
  if (kVec) {  // fold the candidate groups together; lanes 0..LPR-1 end up owning channels sub*VE .. sub*VE+VE-1
    for (int off = LPR; off < 32; off <<= 1) {
#pragma unroll
      for (int e = 0; e < VE; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
    }
  }

  if (p.extras_only) {
    const float m1 = p.ws_m[grow], l1 = p.ws_l[grow];
    const float mm = fmaxf(m, m1);
    const float c1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mm);
    const float c2 = (m == -INFINITY) ? 0.f : __expf(m - mm);
    const float lt = l1 * c1 + l * c2;
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    // the window pass stores raw P.V (no value scale); acc here is raw too
    const int64_t ob = out_row_base(p, bh, t);
    if (kVec) {
      if (lane < LPR) {
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          const int d = sub * VE + e;
          store_out(p, ob + d, (p.ws_o[grow * D + d] * c1 + acc[e] * c2) * inv * vscale);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < GEN_MAXD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) store_out(p, ob + d, (p.ws_o[grow * D + d] * c1 + acc[i] * c2) * inv * vscale);
      }
    }
    return;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  const int64_t ob = out_row_base(p, bh, t);
  if (kVec) {
    if (lane < LPR) {
#pragma unroll
      for (int e = 0; e < VE; ++e) store_out(p, ob + sub * VE + e, acc[e] * inv * vscale);
    }
  } else {
#pragma unroll
    for (int i = 0; i < GEN_MAXD / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < D) store_out(p, ob + d, acc[i] * inv * vscale);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// row kernel for head_dim 64 in bf16 or int8
// ------------------------------------------------------------------------------------------------
// Same work split as attn_rows_kernel (one warp per row, 32 candidates per step, one key per lane), but the key rows
// reach the lanes through shared memory: eight lanes copy one row with cp.async (four rows per instruction, whole
// 128-byte lines), and each lane then reads its own row from a padded tile.  A lane that loads its own row straight
// from global memory touches 32 different lines per instruction, eight instructions per step; measured, that kept
// the L1 tag stage near 80 % busy with DRAM at 27 %.  The copy of the next step's keys is started as soon as the
// scores of this step are in registers, so it overlaps the value accumulation.  q sits in registers as packed
// bf16 pairs (int8: packed bytes, dp4a — the integer dot is exact either way).
constexpr int R64_PITCH_PAD = 16;

template <typename T>
__device__ __forceinline__ void r64_issue_keys(const T* kh, int64_t k_ts, int idx, unsigned char* tile, int grp, int sub) {
  constexpr int ROWB = 64 * sizeof(T), PITCH = ROWB + R64_PITCH_PAD, CH = ROWB / 8;   // bytes per lane per row
#pragma unroll
  for (int st = 0; st < 8; ++st) {
    const int row = st * 4 + grp;
    const int ic = max(__shfl_sync(0xffffffffu, idx, row), 0);   // a dead slot copies key 0; its score is masked
    const unsigned dst = (unsigned)__cvta_generic_to_shared(tile + row * PITCH + sub * CH);
    const T* src = kh + (int64_t)ic * k_ts + sub * (CH / (int)sizeof(T));
    if (CH == 16) asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(GEN_WARPS * 32, 3) attn_rows64_kernel(const AttnParams p) {
  constexpr int ROWB = 64 * sizeof(T), PITCH = ROWB + R64_PITCH_PAD, WARP_BYTES = 32 * PITCH + ROWB;
  extern __shared__ __align__(16) unsigned char r64_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int start = p.row_offsets[bh];
  const int cnt = p.row_offsets[bh + 1] - start;
  const int r = blockIdx.x * GEN_WARPS + warp;
  if (r >= cnt) return;
  const int64_t grow = (int64_t)start + r;
  const int t = p.token_idx[grow];
  const int Tn = p.T;
  const T* qh = reinterpret_cast<const T*>(p.q) + ((int64_t)bh * Tn + t) * 64;
  const T* kh = reinterpret_cast<const T*>(p.k) + (bh / p.H) * p.kv.k_batch + (bh % p.H) * p.kv.k_head;
  const T* vh = reinterpret_cast<const T*>(p.v) + (bh / p.H) * p.kv.v_batch + (bh % p.H) * p.kv.v_head;
  const int64_t k_ts = p.kv.k_token, v_ts = p.kv.v_token;
  unsigned char* tile = r64_smem + warp * WARP_BYTES;
  const uint4* qrow = reinterpret_cast<const uint4*>(tile + 32 * PITCH);   // the row's q, read as broadcasts
  if (lane < ROWB / 16) reinterpret_cast<uint4*>(tile + 32 * PITCH)[lane] = reinterpret_cast<const uint4*>(qh)[lane];
  __syncwarp();
  float sc = p.scale;
  float vscale = 1.f;
  if (sizeof(T) == 1) {
    sc *= p.q_scale[bh] * p.k_scale[bh];
    vscale = p.v_scale[bh];
  }
  RowCands rc;
  rc.init(p, bh, grow, t, start, cnt);
  const int n_virtual = rc.n_virtual;

  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const int grp = lane >> 3, sub = lane & 7;

  int idx = rc.v_begin + lane < n_virtual ? rc.index_of(rc.v_begin + lane) : -1;
  if (rc.v_begin < n_virtual) r64_issue_keys<T>(kh, k_ts, idx, tile, grp, sub);
  for (int c0 = rc.v_begin; c0 < n_virtual; c0 += 32) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    float s = -INFINITY;
    {
      const uint4* krow = reinterpret_cast<const uint4*>(tile + lane * PITCH);
      if (sizeof(T) == 2) {
        // bf16 -> fp32 is a 16-bit shift; even and odd channels accumulate side by side in one packed fp32 FMA
        float2 a2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 raw = krow[c], qraw = qrow[c];
          const uint32_t kw[4] = {raw.x, raw.y, raw.z, raw.w}, qw[4] = {qraw.x, qraw.y, qraw.z, qraw.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
            a2 = __ffma2_rn(make_float2(__uint_as_float(kw[i] << 16), __uint_as_float(kw[i] & 0xffff0000u)),
                            make_float2(__uint_as_float(qw[i] << 16), __uint_as_float(qw[i] & 0xffff0000u)), a2);
        }
        if (idx >= 0) s = (a2.x + a2.y) * sc;
      } else {
        int a = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 raw = krow[c], qraw = qrow[c];
          a = __dp4a((int)raw.x, (int)qraw.x, a);
          a = __dp4a((int)raw.y, (int)qraw.y, a);
          a = __dp4a((int)raw.z, (int)qraw.z, a);
          a = __dp4a((int)raw.w, (int)qraw.w, a);
        }
        if (idx >= 0) s = (float)a * sc;
      }
    }
    __syncwarp();   // every lane has read its row: the tile may take the next step's keys
    const int idx_cur = idx;
    if (c0 + 32 < n_virtual) {
      idx = c0 + 32 + lane < n_virtual ? rc.index_of(c0 + 32 + lane) : -1;
      r64_issue_keys<T>(kh, k_ts, idx, tile, grp, sub);
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;  // nothing valid yet (warp-uniform)
    const float pr = (s == -INFINITY) ? 0.f : __expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.f : __expf(m - m_new);
    l = l * corr + warp_sum(pr);
    m = m_new;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= corr;
    // eight steps of four candidates, branch-free: eight independent value loads in flight (dead: weight 0, row 0)
#pragma unroll
    for (int st = 0; st < 8; ++st) {
      const float pc = __shfl_sync(0xffffffffu, pr, st * 4 + grp);
      const int ic = max(__shfl_sync(0xffffffffu, idx_cur, st * 4 + grp), 0);
      float vv[8];
      load_vec<T>(vh + (int64_t)ic * v_ts + sub * 8, vv);
      const float2 pc2 = make_float2(pc, pc);
#pragma unroll
      for (int e = 0; e < 8; e += 2) {   // packed fp32 FMA: two channels per instruction, each rounded as before
        const float2 r2 = __ffma2_rn(pc2, make_float2(vv[e], vv[e + 1]), make_float2(acc[e], acc[e + 1]));
        acc[e] = r2.x;
        acc[e + 1] = r2.y;
      }
    }
  }
#pragma unroll
  for (int off = 8; off < 32; off <<= 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], off);
  }
  const int64_t ob = out_row_base(p, bh, t);
  if (p.extras_only) {
    const float m1 = p.ws_m[grow], l1 = p.ws_l[grow];
    const float mm = fmaxf(m, m1);
    const float c1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mm);
    const float c2 = (m == -INFINITY) ? 0.f : __expf(m - mm);
    const float lt = l1 * c1 + l * c2;
    const float inv = lt > 0.f ? 1.f / lt : 0.f;
    if (lane < 8) {   // the window pass stores raw P.V (no value scale); acc here is raw too
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int d = sub * 8 + e;
        store_out(p, ob + d, (p.ws_o[grow * 64 + d] * c1 + acc[e] * c2) * inv * vscale);
      }
    }
    return;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  if (lane < 8) {
#pragma unroll
    for (int e = 0; e < 8; ++e) store_out(p, ob + sub * 8 + e, acc[e] * inv * vscale);
  }
}

// ------------------------------------------------------------------------------------------------
// tensor-core window kernel (D = 64, bf16 or int8 inputs)
// ------------------------------------------------------------------------------------------------
constexpr int WK_ROWS = 64;   // packed rows per CTA
constexpr int WK_KEYS = 64;   // keys per tile
constexpr int WK_D = 64;

// 64x64 bf16 tile, rows of 128 B = 8 chunks of 16 B; chunk c of row r lives at chunk (c ^ (r & 7)).
__device__ __forceinline__ int swz(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// 8 consecutive elements of a row -> one 16-byte bf16 chunk
template <typename T>
__device__ __forceinline__ uint4 load_chunk(const T* row, int chunk);
template <>
__device__ __forceinline__ uint4 load_chunk<__nv_bfloat16>(const __nv_bfloat16* row, int chunk) {
  return reinterpret_cast<const uint4*>(row)[chunk];
}
// Two int8 values (bytes 2*pair and 2*pair+1 of `flipped`, a word whose bytes have had their sign bits flipped) as a
// bf16 pair, without I2F or F2F: each byte goes into the mantissa of 2^23, 8388736 comes off, and the upper half of
// the resulting fp32 IS the bf16 (an integer of magnitude <= 128 needs at most 8 significant bits).
__device__ __forceinline__ uint32_t i8x2_to_bf16x2(uint32_t flipped, int pair) {
  const float a = __uint_as_float(__byte_perm(flipped, 0x4B000000u, 0x7440u + 2 * pair)) - 8388736.0f;
  const float b = __uint_as_float(__byte_perm(flipped, 0x4B000000u, 0x7441u + 2 * pair)) - 8388736.0f;
  return __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x7632u);
}
__device__ __forceinline__ uint4 i8x8_to_bf16x8(uint32_t lo, uint32_t hi) {
  lo ^= 0x80808080u;
  hi ^= 0x80808080u;
  return make_uint4(i8x2_to_bf16x2(lo, 0), i8x2_to_bf16x2(lo, 1), i8x2_to_bf16x2(hi, 0), i8x2_to_bf16x2(hi, 1));
}
template <>
__device__ __forceinline__ uint4 load_chunk<int8_t>(const int8_t* row, int chunk) {
  const uint2 raw = reinterpret_cast<const uint2*>(row)[chunk];
  return i8x8_to_bf16x8(raw.x, raw.y);
}

constexpr int WK_TILE_BYTES = WK_KEYS * 128;  // one 64-key K or V tile in shared memory

// STAGES >= 2: depth of the cp.async ring (bf16 tiles, or raw int8 tiles that are widened in shared memory).
template <typename T, int STAGES>
__global__ void __launch_bounds__(128) attn_window_kernel(const AttnParams p) {
  extern __shared__ __align__(1024) unsigned char wk_smem[];
  unsigned char* q_s = wk_smem;                                   // [64 rows][128 B]
  unsigned char* kv_s = wk_smem + WK_ROWS * 128;                  // STAGES x (K tile | V tile)
  unsigned char* k_s = kv_s;
  unsigned char* v_s = kv_s + WK_TILE_BYTES;
  __shared__ int ts[WK_ROWS];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Ordinary pass: blockIdx.y is a (batch, head) pair, keys are the tokens, a row t sees keys (t - window, t].
  // Anchor pass: blockIdx.y is a (head, residue rho) group, keys are the strided view K[rho + stride * i], and a
  // row of token t = stride * it + rho sees strided keys (it - jmin - an_window, it - jmin]; ts[] then holds
  // it - jmin (possibly negative: a row without anchor keys, which still has to carry its partial state along).
  const bool anchor = p.an_stride > 0;
  const int astr = anchor ? p.an_stride : 1;
  const int bh = anchor ? blockIdx.y / astr : blockIdx.y;
  const int rho = anchor ? blockIdx.y % astr : 0;
  const int32_t* offs = anchor ? p.an_offsets : p.row_offsets;
  const int start = offs[blockIdx.y];
  const int cnt = offs[blockIdx.y + 1] - start;
  // a CTA takes 64-row tiles of its group in turn (the grid's x extent need not cover the largest group)
  for (int r0 = blockIdx.x * WK_ROWS; r0 < cnt; r0 += gridDim.x * WK_ROWS) {
  const int nrows = min(WK_ROWS, cnt - r0);
  const int Tn = anchor ? (p.T - rho + astr - 1) / astr : p.T;   // number of keys in this pass's key space
  const int window = anchor ? p.an_window : (p.has_plan ? (p.plan.window > 0 ? p.plan.window : 1) : (Tn + 1));
  const T* qh = reinterpret_cast<const T*>(p.q) + (int64_t)bh * p.T * WK_D;
  const int64_t k_ts = p.kv.k_token * astr, v_ts = p.kv.v_token * astr;
  const T* kh = reinterpret_cast<const T*>(p.k) + (bh / p.H) * p.kv.k_batch + (bh % p.H) * p.kv.k_head + rho * p.kv.k_token;
  const T* vh = reinterpret_cast<const T*>(p.v) + (bh / p.H) * p.kv.v_batch + (bh % p.H) * p.kv.v_head + rho * p.kv.v_token;
  constexpr int ABSENT = -2147483647;
  __shared__ int grow_s[WK_ROWS];   // workspace / packing row of every tile row

  if (tid < WK_ROWS) {
    int tv = ABSENT, gr = 0;
    if (tid < nrows) {
      if (anchor) {
        tv = p.an_tok[start + r0 + tid];
        if (tv == ANCHOR_NO_KEYS) tv = -1;   // present, sees nothing
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
  // Q rows (gathered) -> swizzled shared tile
  for (int c = tid; c < WK_ROWS * 8; c += 128) {
    const int row = c >> 3, ch = c & 7;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (ts[row] != ABSENT) {
      const int64_t tq = anchor ? (int64_t)p.token_idx[grow_s[row]] : (int64_t)ts[row];
      val = load_chunk<T>(qh + tq * WK_D, ch);
    }
    *reinterpret_cast<uint4*>(q_s + swz(row, ch)) = val;
  }
  // rows ascend inside a group; rows without keys (negative) come first
  const int t_first = ts[0], t_last = ts[nrows - 1];
  const int lo = max(0, t_first - window + 1);
  const int kt_begin = lo / WK_KEYS, kt_end = t_last < 0 ? -1 : t_last / WK_KEYS;  // inclusive

  // this warp's rows
  const int wr0 = warp * 16;
  const int g = lane >> 2, qd = lane & 3;
  const int tg0 = ts[wr0 + g], tg1 = ts[wr0 + g + 8];
  int w_first = -1, w_last = -1;
  for (int i = 0; i < 16; ++i) {
    const int tt = ts[wr0 + i];
    if (tt >= 0) {
      if (w_first < 0) w_first = tt;
      w_last = tt;
    }
  }
  const int w_lo = w_first < 0 ? 0 : max(0, w_first - window + 1);
  const bool has0 = tg0 != ABSENT, has1 = tg1 != ABSENT;

  float sc_log2 = p.scale * 1.4426950408889634f;
  if (sizeof(T) == 1) sc_log2 *= p.q_scale[bh] * p.k_scale[bh];

  __syncthreads();
  uint32_t qa[4][4];
  {
    const int row = wr0 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      ldmatrix_x4(smem_u32(q_s + swz(row, ks * 2 + (lane >> 4))), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
  }

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  if (p.read_partial) {
    // continue from the state an earlier pass left in the workspace (natural-log maximum, denominator, raw P.V);
    // the denominator is kept per quad here and summed over the quad at the end, so only lane qd == 0 takes it
    const float inv_ln2 = 1.4426950408889634f;
    if (has0) {
      const int64_t gr = grow_s[wr0 + g];
      const float mw = p.ws_m[gr];
      m0 = (mw == -INFINITY) ? -INFINITY : mw * inv_ln2;
      l0 = qd == 0 ? p.ws_l[gr] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 pr = *reinterpret_cast<const float2*>(p.ws_o + gr * WK_D + 8 * j + qd * 2);
        o[j][0] = pr.x; o[j][1] = pr.y;
      }
    }
    if (has1) {
      const int64_t gr = grow_s[wr0 + g + 8];
      const float mw = p.ws_m[gr];
      m1 = (mw == -INFINITY) ? -INFINITY : mw * inv_ln2;
      l1 = qd == 0 ? p.ws_l[gr] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 pr = *reinterpret_cast<const float2*>(p.ws_o + gr * WK_D + 8 * j + qd * 2);
        o[j][2] = pr.x; o[j][3] = pr.y;
      }
    }
  }

  // bf16: tiles arrive by cp.async into a ring of STAGES (K | V) buffers, one barrier per tile.
  // int8: raw 64-byte rows arrive by cp.async into a ring of STAGES raw buffers behind two bf16 (K | V) buffers; the
  // raw tile kt+1 is widened into the free bf16 buffer while tile kt is being multiplied, again one barrier per tile.
  constexpr bool kI8 = sizeof(T) == 1;
  constexpr int RAW_TILE = WK_KEYS * WK_D;   // bytes of one raw int8 tile
  unsigned char* raw_s = kv_s + 2 * 2 * WK_TILE_BYTES;
  auto issue = [&](int kt) {  // cp.async tile kt into its ring slot; always commits a group (possibly empty)
    if (kt <= kt_end) {
      if (kI8) {
        unsigned char* rk = raw_s + ((kt - kt_begin) % STAGES) * 2 * RAW_TILE;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int c = tid + 128 * i;
          const int row = c >> 2, rc = c & 3;
          const int key = kt * WK_KEYS + row;
          const int64_t kc = min(key, Tn - 1);
          const int nbytes = key < Tn ? 16 : 0;
          cp_async16(smem_u32(rk + row * 64 + rc * 16), kh + kc * k_ts + rc * 16, nbytes);
          cp_async16(smem_u32(rk + RAW_TILE + row * 64 + rc * 16), vh + kc * v_ts + rc * 16, nbytes);
        }
      } else {
        unsigned char* ks_ = kv_s + ((kt - kt_begin) % STAGES) * 2 * WK_TILE_BYTES;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = tid + 128 * i;
          const int row = c >> 3, ch = c & 7;
          const int key = kt * WK_KEYS + row;
          const int64_t kc = min(key, Tn - 1);
          const int nbytes = key < Tn ? 16 : 0;
          cp_async16(smem_u32(ks_ + swz(row, ch)), kh + kc * k_ts + ch * 8, nbytes);
          cp_async16(smem_u32(ks_ + WK_TILE_BYTES + swz(row, ch)), vh + kc * v_ts + ch * 8, nbytes);
        }
      }
    }
    cp_async_commit();
  };
  auto widen = [&](int kt) {  // int8 only: raw tile kt -> bf16 buffer (kt - kt_begin) % 2, swizzled
    if (!kI8 || kt > kt_end) return;
    const unsigned char* rk = raw_s + ((kt - kt_begin) % STAGES) * 2 * RAW_TILE;
    unsigned char* dk = kv_s + ((kt - kt_begin) % 2) * 2 * WK_TILE_BYTES;
#pragma unroll
    for (int which = 0; which < 2; ++which) {   // K, then V
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int c = tid + 128 * i;
        const int row = c >> 2, rc = c & 3;
        const uint4 raw = *reinterpret_cast<const uint4*>(rk + which * RAW_TILE + row * 64 + rc * 16);
        const uint4 lo = i8x8_to_bf16x8(raw.x, raw.y), hi = i8x8_to_bf16x8(raw.z, raw.w);
        *reinterpret_cast<uint4*>(dk + which * WK_TILE_BYTES + swz(row, 2 * rc)) = lo;
        *reinterpret_cast<uint4*>(dk + which * WK_TILE_BYTES + swz(row, 2 * rc + 1)) = hi;
      }
    }
  };
#pragma unroll
  for (int s_ = 0; s_ < STAGES - 1; ++s_) issue(kt_begin + s_);
  if (kI8) {
    cp_async_wait<(STAGES >= 2 ? STAGES - 2 : 0)>();
    __syncthreads();
    widen(kt_begin);
  }

  // copies that may still be in flight at the top of an iteration: the bf16 path needs tile kt, the int8 path tile kt+1
  constexpr int PEND = kI8 ? (STAGES >= 3 ? STAGES - 3 : 0) : (STAGES >= 2 ? STAGES - 2 : 0);
  for (int kt = kt_begin; kt <= kt_end; ++kt) {
    cp_async_wait<PEND>();           // this thread's copies of tile kt (int8: kt+1) have landed
    __syncthreads();                 // ... everybody's have, and tile kt-1 is no longer being read
    issue(kt + STAGES - 1);          // refill the slot tile kt-1 occupied
    if (kI8) {
      widen(kt + 1);
      k_s = kv_s + ((kt - kt_begin) % 2) * 2 * WK_TILE_BYTES;
    } else {
      k_s = kv_s + ((kt - kt_begin) % STAGES) * 2 * WK_TILE_BYTES;
    }
    v_s = k_s + WK_TILE_BYTES;

    const int kb = kt * WK_KEYS;
    if (w_first < 0 || kb > w_last || kb + WK_KEYS - 1 < w_lo) continue;  // tile outside this warp's rows

    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {  // pairs of 8-key n-tiles
        uint32_t b0, b1, b2, b3;
        const int krow = jp * 16 + (lane & 7) + 8 * (lane >> 4);
        ldmatrix_x4(smem_u32(k_s + swz(krow, ks * 2 + ((lane >> 3) & 1))), b0, b1, b2, b3);
        mma_bf16(s[2 * jp], qa[ks], b0, b1);
        mma_bf16(s[2 * jp + 1], qa[ks], b2, b3);
      }
    }
    // mask + online softmax (base-2 domain)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kb + 8 * j + qd * 2 + (e & 1);
        const int tt = (e < 2) ? tg0 : tg1;
        const bool ok = tt >= 0 && key <= tt && key > tt - window;
        const float val = ok ? s[j][e] * sc_log2 : -INFINITY;
        s[j][e] = val;
        if (e < 2) mx0 = fmaxf(mx0, val); else mx1 = fmaxf(mx1, val);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float cr0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0);
    const float cr1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1);
    const float base0 = (mn0 == -INFINITY) ? 0.f : mn0, base1 = (mn1 == -INFINITY) ? 0.f : mn1;
    m0 = mn0;
    m1 = mn1;
    l0 *= cr0;
    l1 *= cr1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j][0] *= cr0; o[j][1] *= cr0; o[j][2] *= cr1; o[j][3] *= cr1;
      s[j][0] = exp2f(s[j][0] - base0);
      s[j][1] = exp2f(s[j][1] - base0);
      s[j][2] = exp2f(s[j][2] - base1);
      s[j][3] = exp2f(s[j][3] - base1);
      l0 += s[j][0] + s[j][1];
      l1 += s[j][2] + s[j][3];
    }
    // O += P V
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {  // 16 keys per step
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
      pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
      pa[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      pa[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {  // pairs of 8-wide d tiles
        uint32_t b0, b1, b2, b3;
        const int vrow = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        ldmatrix_x4_trans(smem_u32(v_s + swz(vrow, jp * 2 + (lane >> 4))), b0, b1, b2, b3);
        mma_bf16(o[2 * jp], pa, b0, b1);
        mma_bf16(o[2 * jp + 1], pa, b2, b3);
      }
    }
  }

  // finish: quad-reduce the denominators
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float ln2 = 0.6931471805599453f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int tt = half ? tg1 : tg0;
    if (tt == ABSENT) continue;
    const int64_t grow = grow_s[wr0 + g + 8 * half];
    const float mm = half ? m1 : m0, ll = half ? l1 : l0;
    if (p.write_partial) {
      if (qd == 0) {
        p.ws_m[grow] = (mm == -INFINITY) ? -INFINITY : mm * ln2;  // back to the natural-log domain
        p.ws_l[grow] = ll;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float2 pr = make_float2(o[j][2 * half], o[j][2 * half + 1]);
        *reinterpret_cast<float2*>(p.ws_o + grow * WK_D + 8 * j + qd * 2) = pr;
      }
    } else {
      float inv = ll > 0.f ? 1.f / ll : 0.f;
      if (sizeof(T) == 1) inv *= p.v_scale[bh];
      const int64_t ob = out_row_base(p, bh, tt);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d = 8 * j + qd * 2;
        const int64_t oi = ob + d;
        const float a = o[j][2 * half] * inv, b = o[j][2 * half + 1] * inv;
        if (p.out_dtype == ASPA_BF16)
          *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.out) + oi) = __floats2bfloat162_rn(a, b);
        else
          *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + oi) = make_float2(a, b);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // shared tiles and row tables are reused by the next 64-row tile
  }
}

// ------------------------------------------------------------------------------------------------
// Regrouping of the packed rows by (head, token % stride) for the anchor tile pass
// ------------------------------------------------------------------------------------------------
// A stable counting sort of every head's rows by token % stride.  One CTA per head, its rows cut into one segment per
// warp: each warp counts its segment's residues into its own row of a shared-memory table; pass 0 adds the rows up to
// the group sizes (scanned between the passes); pass 1 turns the table into each warp's first position inside every
// group and walks the segment again in order, ranking equal residues inside a step with match_any.  (One warp per
// (head, residue) group walking all rows of the head, as before, visited every row `stride` times: 44 us per pass at
// 16 heads x 6554 rows x 128 residues.)
constexpr int RG_WARPS = 32;

__global__ void __launch_bounds__(RG_WARPS * 32) anchor_regroup_kernel(const int32_t* __restrict__ row_offsets,
                                                                       const int32_t* __restrict__ token_idx, int heads,
                                                                       int stride, int window, int jmin, int fill,
                                                                       int32_t* __restrict__ grp_offsets,
                                                                       int32_t* __restrict__ grp_tok,
                                                                       int32_t* __restrict__ grp_row) {
  extern __shared__ int rg_cnt[];   // [RG_WARPS][stride]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x;
  const int start = row_offsets[bh], cnt = row_offsets[bh + 1] - start;
  const bool pow2 = (stride & (stride - 1)) == 0;
  for (int i = threadIdx.x; i < RG_WARPS * stride; i += blockDim.x) rg_cnt[i] = 0;
  __syncthreads();
  const int seg = ((cnt + RG_WARPS - 1) / RG_WARPS + 31) & ~31;   // rows per warp, whole steps of 32
  const int r_begin = min(cnt, warp * seg), r_end = min(cnt, r_begin + seg);
  int* mine = rg_cnt + warp * stride;
  for (int r0 = r_begin; r0 < r_end; r0 += 128) {   // four loads of the token list in flight per lane
    int tk[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int r = r0 + 32 * u + lane;
      tk[u] = r < r_end ? token_idx[start + r] : -1;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (tk[u] >= 0) atomicAdd(&mine[pow2 ? (tk[u] & (stride - 1)) : (tk[u] % stride)], 1);
  }
  __syncthreads();
  // per residue: group size (pass 0), or each warp's first position inside the group (pass 1)
  for (int rho = threadIdx.x; rho < stride; rho += blockDim.x) {
    int run = fill ? grp_offsets[bh * stride + rho] : 0;
    for (int w = 0; w < RG_WARPS; ++w) {
      const int c = rg_cnt[w * stride + rho];
      if (fill) rg_cnt[w * stride + rho] = run;
      run += c;
    }
    if (!fill) grp_offsets[bh * stride + rho] = run;
  }
  if (!fill) return;
  __syncthreads();
  for (int r0 = r_begin; r0 < r_end; r0 += 32) {
    const int r = r0 + lane;
    const int t = r < r_end ? token_idx[start + r] : -1;
    const int rho = t < 0 ? -1 - lane : (pow2 ? (t & (stride - 1)) : (t % stride));   // absent rows: keys of their own
    const unsigned peers = __match_any_sync(0xffffffffu, rho);
    const int leader = __ffs(peers) - 1;
    int base = 0;
    if (t >= 0 && lane == leader) {
      base = mine[rho];
      mine[rho] = base + __popc(peers);
    }
    base = __shfl_sync(0xffffffffu, base, leader);
    if (t >= 0) {
      const int pos = base + __popc(peers & ((1u << lane) - 1u));
      // rows whose local window already reaches key 0 have no anchor key at all
      grp_tok[pos] = (t + 1 >= window) ? t / stride - jmin : ANCHOR_NO_KEYS;
      grp_row[pos] = start + r;
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(1024) anchor_scan_kernel(int32_t* __restrict__ grp_offsets, int n_groups) {
  __shared__ int tmp[64];
  int running = 0;
  for (int base = 0; base < n_groups; base += 1024) {
    const int i = base + threadIdx.x;
    const int v = i < n_groups ? grp_offsets[i] : 0;
    int tot;
    const int ex = block_exclusive_scan(v, tmp, &tot);
    if (i < n_groups) grp_offsets[i] = running + ex;
    running += tot;
  }
  if (threadIdx.x == 0) grp_offsets[n_groups] = running;
}

}  // namespace aspa

using namespace aspa;

// Does a planned call take the tile (tensor-core) path?  The tile pass streams the union key range of 16 consecutive
// rows (about 16*gap + window keys, gap = mean token distance between the rows of a head); a per-row gather reads
// 16*window.  With very sparse rows the union is mostly keys nobody attends to and the CTA count drops below the SM
// count: gather instead.  total_rows may be a host-side upper bound, which only makes the estimate of the gap
// conservative.
static int g_attn_tc_mode = 1;   // see tc_tiles_wanted
static int g_attn_picks_mode = 1;   // 0: prototype picks always on the row kernel; 1: on warp-MMA tiles where covered
static bool tile_path_ok(int qkv_dtype, int D, bool has_cand, bool has_mask, const aspa_shortlist_plan* plan, int heads,
                         int T, int64_t total_rows) {
  if (!(D == WK_D && (qkv_dtype == ASPA_BF16 || qkv_dtype == ASPA_I8) && !has_cand && !has_mask)) return false;
  if (plan != nullptr) {
    const double gap = (double)T * (double)heads / (double)std::max<int64_t>(total_rows, 1);
    const double window = plan->window > 0 ? plan->window : 1;
    if (16.0 * gap >= 7.0 * window && g_attn_tc_mode != 2) return false;
  }
  return true;
}

// Which tile kernel?  The tcgen05 kernel works on 128-row tiles whose union key range is about 128*gap + window keys,
// of which a row uses `window`; the warp-MMA kernel works on 16-row groups and wastes far less on sparse rows.
// Measured on B200 (16 heads): dense rows 2.3x in favour of tcgen05 (1.18 against 2.74 ms, causal, 32768 tokens), one row
// every 40 tokens with a 2458-key window a draw (0.60 ms each), one row in five with a 362-key window 0.28 against
// 0.19 ms.  So tcgen05 is taken from a third of the tile being useful (window >= 64 * gap).
// Mode 0 = never, 1 = by that rule, 2 = whenever the shape allows.
static bool tc_tiles_wanted(int window, int heads, int T, int64_t total_rows) {
  if (g_attn_tc_mode != 1) return g_attn_tc_mode == 2;
  const double gap = (double)T * (double)heads / (double)std::max<int64_t>(total_rows, 1);
  return (double)window >= 64.0 * gap;
}

// Anchors t - j*stride of the rows of one residue class t % stride are a window over the strided key sequence of that
// class: with enough rows per (head, residue) group they go through the tile kernel too, regrouped.
struct AnchorTiles {
  bool use;      // 64-row tiles over regrouped rows
  bool groups;   // one warp per (head, residue) group (attention_picks.cu): groups too small for 64-row tiles
  int n_loc_full, jmin, an_window;
};
static AnchorTiles anchor_tiles_for(const aspa_shortlist_plan* plan, bool has_ws, int heads, int64_t total_rows) {
  AnchorTiles a = {false, false, 1, 1, 0};
  if (plan == nullptr || !(plan->anchor_slots > 0 && plan->anchor_stride > 0)) return a;
  a.n_loc_full = plan->window > 0 ? plan->window : 1;
  a.jmin = (a.n_loc_full - 1) / plan->anchor_stride + 1;   // first anchor slot outside the window
  a.an_window = plan->anchor_slots - a.jmin + 1;
  a.use = has_ws && plan->anchor_stride <= 1024 && a.an_window >= 64 &&
          total_rows >= (int64_t)8 * heads * plan->anchor_stride;
  a.groups = has_ws && !a.use && plan->anchor_stride <= 1024 && a.an_window >= 1 && g_attn_picks_mode != 0;
  return a;
}
static void launch_regroup(const int32_t* row_offsets, const int32_t* token_idx, int heads, int R, const AnchorTiles& a,
                           int64_t total_rows, void* regroup_ws, cudaStream_t st) {
  const int n_groups = heads * R;
  int32_t* goffs = reinterpret_cast<int32_t*>(regroup_ws);
  int32_t* gtok = goffs + n_groups + 1;
  int32_t* grow_ = gtok + total_rows;
  const size_t smem = (size_t)RG_WARPS * R * sizeof(int);   // at most 128 KB (stride <= 1024)
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaFuncSetAttribute(anchor_regroup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RG_WARPS * 1024 * (int)sizeof(int));
    attr_set[dev] = true;
  }
  anchor_regroup_kernel<<<heads, RG_WARPS * 32, smem, st>>>(row_offsets, token_idx, heads, R, a.n_loc_full, a.jmin, 0, goffs, gtok, grow_);
  anchor_scan_kernel<<<1, 1024, 0, st>>>(goffs, n_groups);
  anchor_regroup_kernel<<<heads, RG_WARPS * 32, smem, st>>>(row_offsets, token_idx, heads, R, a.n_loc_full, a.jmin, 1, goffs, gtok, grow_);
}

extern "C" int aspa_attn_regroup_rows(int qkv_dtype, int heads, int T, int D, const int32_t* row_offsets,
                                      const int32_t* token_idx, int64_t total_rows, const aspa_shortlist_plan* plan,
                                      void* regroup_ws, int32_t* prepared, void* stream) {
  ASPA_CHECK_ARG(row_offsets && token_idx && plan && prepared, "null pointer");
  *prepared = 0;
  if (total_rows <= 0 || regroup_ws == nullptr) return ASPA_OK;
  if (!tile_path_ok(qkv_dtype, D, false, false, plan, heads, T, total_rows)) return ASPA_OK;
  const AnchorTiles a = anchor_tiles_for(plan, true, heads, total_rows);
  if (!a.use && !(a.groups && D == 64 && (qkv_dtype == ASPA_BF16 || qkv_dtype == ASPA_I8))) return ASPA_OK;
  launch_regroup(row_offsets, token_idx, heads, plan->anchor_stride, a, total_rows, regroup_ws, (cudaStream_t)stream);
  ASPA_CHECK_LAUNCH();
  *prepared = 1;
  return ASPA_OK;
}

extern "C" int64_t aspa_attn_regroup_bytes(int64_t total_rows, int heads, int anchor_stride) {
  if (anchor_stride <= 0) return 0;
  return (int64_t)sizeof(int32_t) * ((int64_t)heads * anchor_stride + 1 + 2 * total_rows);
}

extern "C" int aspa_attn_picks_mode(int mode) {
  const int old = g_attn_picks_mode;
  if (mode == 0 || mode == 1) g_attn_picks_mode = mode;
  return old;
}

extern "C" int aspa_attn_tc_mode(int mode) {
  const int old = g_attn_tc_mode;
  if (mode >= 0 && mode <= 2) g_attn_tc_mode = mode;
  return old;
}

extern "C" int64_t aspa_attn_workspace_bytes(int64_t total_rows, int D) {
  return (int64_t)sizeof(float) * total_rows * (D + 2);
}

template <typename T>
static void launch_rows64(const AttnParams& p, dim3 grid, cudaStream_t st) {
  constexpr int ROWB = 64 * (int)sizeof(T);
  constexpr int smem = GEN_WARPS * (32 * (ROWB + R64_PITCH_PAD) + ROWB);
  attn_rows64_kernel<T><<<grid, GEN_WARPS * 32, smem, st>>>(p);
}
template <>
void launch_rows64<float>(const AttnParams&, dim3, cudaStream_t) {}

template <typename T>
static void launch_generic(const AttnParams& p, int max_rows, cudaStream_t st) {
  const dim3 grid((unsigned)ceil_div(max_rows, GEN_WARPS), p.heads);
  if (sizeof(T) <= 2 && p.D == 64 && p.add_mask == nullptr) {
    launch_rows64<T>(p, grid, st);
    return;
  }
  constexpr int VE = VecElems<T>::n;
  const int lpr = p.D % VE == 0 ? p.D / VE : 0;
  const bool vec = lpr >= 1 && lpr <= 32 && (lpr & (lpr - 1)) == 0;
  if (vec) attn_rows_kernel<T, true><<<grid, GEN_WARPS * 32, 0, st>>>(p);
  else attn_rows_kernel<T, false><<<grid, GEN_WARPS * 32, 0, st>>>(p);
}
template <typename T, int STAGES>
static void launch_window(const AttnParams& p, int max_rows, cudaStream_t st, int groups = 0) {
  const dim3 grid((unsigned)ceil_div(max_rows, WK_ROWS), groups > 0 ? groups : p.heads);
  const int smem = sizeof(T) == 1 ? WK_ROWS * 128 + 2 * 2 * WK_TILE_BYTES + STAGES * 2 * WK_KEYS * WK_D
                                  : WK_ROWS * 128 + STAGES * 2 * WK_TILE_BYTES;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(attn_window_kernel<T, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    attr_set = true;
  }
  attn_window_kernel<T, STAGES><<<grid, 128, smem, st>>>(p);
}

extern "C" int aspa_gather_attn_fwd(const void* q, const void* k, const void* v, int qkv_dtype, const float* q_scale,
                                    const float* k_scale, const float* v_scale, int heads, int T, int D, int H,
                                    const int32_t* row_offsets, const int32_t* token_idx, int max_rows,
                                    int64_t total_rows, const int64_t* cand, const int64_t* cand_len, int L,
                                    const aspa_shortlist_plan* plan, const float* add_mask, void* out, int out_dtype,
                                    int out_layout, void* workspace, void* stream) {
  return aspa_gather_attn_fwd_ex(q, k, v, qkv_dtype, q_scale, k_scale, v_scale, heads, T, D, H, row_offsets, token_idx,
                                 max_rows, total_rows, cand, cand_len, L, plan, add_mask, out, out_dtype, out_layout,
                                 nullptr, nullptr, workspace, nullptr, stream);
}

extern "C" int aspa_gather_attn_fwd_ex(const void* q, const void* k, const void* v, int qkv_dtype,
                                       const float* q_scale, const float* k_scale, const float* v_scale, int heads,
                                       int T, int D, int H, const int32_t* row_offsets, const int32_t* token_idx,
                                       int max_rows, int64_t total_rows, const int64_t* cand,
                                       const int64_t* cand_len, int L, const aspa_shortlist_plan* plan,
                                       const float* add_mask, void* out, int out_dtype, int out_layout,
                                       const int32_t* out_row_map, const aspa_kv_layout* kv_layout, void* workspace,
                                       void* regroup_ws, void* stream) {
  return aspa_gather_attn_fwd_prepared(q, k, v, qkv_dtype, q_scale, k_scale, v_scale, heads, T, D, H, row_offsets,
                                       token_idx, max_rows, total_rows, cand, cand_len, L, plan, add_mask, out, out_dtype,
                                       out_layout, out_row_map, kv_layout, workspace, regroup_ws, 0, stream);
}

extern "C" int aspa_gather_attn_fwd_prepared(const void* q, const void* k, const void* v, int qkv_dtype,
                                             const float* q_scale, const float* k_scale, const float* v_scale,
                                             int heads, int T, int D, int H, const int32_t* row_offsets,
                                             const int32_t* token_idx, int max_rows, int64_t total_rows,
                                             const int64_t* cand, const int64_t* cand_len, int L,
                                             const aspa_shortlist_plan* plan, const float* add_mask, void* out,
                                             int out_dtype, int out_layout, const int32_t* out_row_map,
                                             const aspa_kv_layout* kv_layout, void* workspace, void* regroup_ws,
                                             int regroup_prepared, void* stream) {
  ASPA_CHECK_ARG(q && k && v && row_offsets && token_idx && out, "null pointer");
  ASPA_CHECK_ARG(heads > 0 && T > 0 && D > 0 && D <= GEN_MAXD, "head_dim must be in [1, 256]");
  ASPA_CHECK_ARG(qkv_dtype == ASPA_F32 || qkv_dtype == ASPA_BF16 || qkv_dtype == ASPA_I8, "bad qkv dtype");
  ASPA_CHECK_ARG(out_dtype == ASPA_F32 || out_dtype == ASPA_BF16, "bad out dtype");
  ASPA_CHECK_ARG(out_layout == ASPA_OUT_HEAD_MAJOR || (out_layout == ASPA_OUT_TOKEN_MAJOR && H > 0 && heads % H == 0),
                 "token-major output needs H dividing heads");
  ASPA_CHECK_ARG(out_row_map == nullptr || out_layout == ASPA_OUT_TOKEN_MAJOR, "a row map needs the token-major layout");
  if (qkv_dtype == ASPA_I8) ASPA_CHECK_ARG(q_scale && k_scale && v_scale, "int8 inputs need q/k/v scales");
  ASPA_CHECK_ARG((cand == nullptr) == (cand_len == nullptr), "candidates and lengths come together");
  if (cand) ASPA_CHECK_ARG(L > 0, "candidate width must be positive");
  if (max_rows <= 0 || total_rows <= 0) return ASPA_OK;
  cudaStream_t st = (cudaStream_t)stream;

  AttnParams p{};
  p.q = q; p.k = k; p.v = v;
  p.q_scale = q_scale; p.k_scale = k_scale; p.v_scale = v_scale;
  p.heads = heads; p.T = T; p.D = D; p.H = H > 0 ? H : heads;
  p.row_offsets = row_offsets; p.token_idx = token_idx;
  p.cand = cand; p.cand_len = cand_len; p.L = L;
  p.has_plan = (plan != nullptr && cand == nullptr) ? 1 : 0;
  if (p.has_plan) p.plan = *plan;
  p.add_mask = add_mask;
  p.out = out; p.out_dtype = out_dtype; p.out_layout = out_layout; p.out_row_map = out_row_map;
  if (kv_layout) {
    ASPA_CHECK_ARG(H > 0 && heads % H == 0, "a k/v layout needs H dividing heads");
    const int64_t a = 16 / (qkv_dtype == ASPA_F32 ? 4 : (qkv_dtype == ASPA_BF16 ? 2 : 1));  // elements per 16 bytes
    ASPA_CHECK_ARG(kv_layout->k_token % a == 0 && kv_layout->v_token % a == 0 && kv_layout->k_head % a == 0 &&
                       kv_layout->v_head % a == 0 && kv_layout->k_batch % a == 0 && kv_layout->v_batch % a == 0,
                   "k/v strides must keep rows 16-byte aligned");
    p.kv = *kv_layout;
  } else {  // head-major (heads, T, D)
    p.kv.k_token = p.kv.v_token = D;
    p.kv.k_head = p.kv.v_head = (int64_t)T * D;
    p.kv.k_batch = p.kv.v_batch = (int64_t)p.H * T * D;
  }
  p.scale = 1.0f / sqrtf((float)D);
  p.ws_m = p.ws_l = p.ws_o = nullptr;
  p.an_stride = 0;

  const bool tensor_ok = tile_path_ok(qkv_dtype, D, cand != nullptr, add_mask != nullptr, p.has_plan ? plan : nullptr,
                                      heads, T, total_rows);
  if (tensor_ok) {
    const bool extras = p.has_plan && ((plan->anchor_slots > 0 && plan->anchor_stride > 0) ||
                                       (plan->proto_cap > 0 && plan->proto_lists != nullptr));
    if (extras) {
      ASPA_CHECK_ARG(workspace != nullptr, "workspace required when anchors or prototype picks are on");
      float* w = reinterpret_cast<float*>(workspace);
      p.ws_m = w;
      p.ws_l = w + total_rows;
      p.ws_o = w + 2 * total_rows;
      p.write_partial = 1;
    }
    const int win_keys = p.has_plan ? (plan->window > 0 ? plan->window : 1) : T;
    if (!(tc_tiles_wanted(win_keys, heads, T, total_rows) && launch_window_tc(p, qkv_dtype, max_rows, 0, st))) {
      if (qkv_dtype == ASPA_BF16) launch_window<__nv_bfloat16, 3>(p, max_rows, st); else launch_window<int8_t, 4>(p, max_rows, st);
    }
    ASPA_CHECK_LAUNCH();
    const AnchorTiles at = anchor_tiles_for(extras ? plan : nullptr, regroup_ws != nullptr, heads, total_rows);
    if (at.use) {
      const int R = plan->anchor_stride, n_groups = heads * R;
      int32_t* goffs = reinterpret_cast<int32_t*>(regroup_ws);
      int32_t* gtok = goffs + n_groups + 1;
      int32_t* grow_ = gtok + total_rows;
      if (!regroup_prepared) {   // else aspa_attn_regroup_rows has filled regroup_ws for these rows already
        launch_regroup(row_offsets, token_idx, heads, R, at, total_rows, regroup_ws, st);
        ASPA_CHECK_LAUNCH();
      }
      AttnParams pa = p;
      pa.an_stride = R;
      pa.an_window = at.an_window;
      pa.an_jmin = at.jmin;
      pa.an_offsets = goffs;
      pa.an_tok = gtok;
      pa.an_row = grow_;
      pa.read_partial = 1;
      pa.write_partial = 1;
      // rows per group are about total_rows / n_groups: two 64-row tiles per CTA column cover the usual group in
      // one step, and the kernel's tile loop takes care of larger groups
      const int rows_bound = (int)std::min<int64_t>(max_rows, std::max<int64_t>(WK_ROWS, 2 * total_rows / n_groups));
      if (!(tc_tiles_wanted(at.an_window, heads, T, total_rows) && launch_window_tc(pa, qkv_dtype, rows_bound, n_groups, st))) {
        if (qkv_dtype == ASPA_BF16) launch_window<__nv_bfloat16, 3>(pa, rows_bound, st, n_groups);
        else launch_window<int8_t, 4>(pa, rows_bound, st, n_groups);
      }
      ASPA_CHECK_LAUNCH();
      p.anchors_done = 1;
    }
    const bool has_picks = extras && plan->proto_cap > 0 && plan->proto_lists != nullptr;
    if (!at.use && at.groups && anchor_groups_ok(p, qkv_dtype)) {
      const int R = plan->anchor_stride, n_groups = heads * R;
      int32_t* goffs = reinterpret_cast<int32_t*>(regroup_ws);
      int32_t* gtok = goffs + n_groups + 1;
      int32_t* grow_ = gtok + total_rows;
      if (!regroup_prepared) {
        launch_regroup(row_offsets, token_idx, heads, R, at, total_rows, regroup_ws, st);
        ASPA_CHECK_LAUNCH();
      }
      AttnParams pa = p;
      pa.an_stride = R;
      pa.an_window = at.an_window;
      pa.an_jmin = at.jmin;
      pa.an_offsets = goffs;
      pa.an_tok = gtok;
      pa.an_row = grow_;
      pa.read_partial = 1;
      pa.write_partial = has_picks ? 1 : 0;   // without picks this pass writes the final output
      launch_anchor_groups(pa, qkv_dtype, st);
      ASPA_CHECK_LAUNCH();
      if (!has_picks) return ASPA_OK;
      p.anchors_done = 2;
    }
    if (extras) {
      p.write_partial = 0;
      p.extras_only = 1;
      if (g_attn_picks_mode != 0 && !has_picks && p.anchors_done == 1 && p.add_mask == nullptr && p.D == 64)
        launch_finalise_rows(p, qkv_dtype, max_rows, st);   // nothing but the clamping slot and the normalisation is left
      else if (g_attn_picks_mode != 0 && picks_tiles_ok(p, qkv_dtype)) launch_picks_tiles(p, qkv_dtype, st);
      else if (qkv_dtype == ASPA_BF16) launch_generic<__nv_bfloat16>(p, max_rows, st);
      else launch_generic<int8_t>(p, max_rows, st);
      ASPA_CHECK_LAUNCH();
    }
    return ASPA_OK;
  }
  if (qkv_dtype == ASPA_F32) launch_generic<float>(p, max_rows, st);
  else if (qkv_dtype == ASPA_BF16) launch_generic<__nv_bfloat16>(p, max_rows, st);
  else launch_generic<int8_t>(p, max_rows, st);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
