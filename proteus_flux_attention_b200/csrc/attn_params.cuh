// Parameter block shared by the attention kernels (CUDA-core row kernels, warp-MMA window kernel, tcgen05 window kernel).
#pragma once

#include "common.cuh"

namespace aspa {

constexpr int ANCHOR_NO_KEYS = -(1 << 30);  // a row of the anchor pass that has no anchor key

struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  int heads, T, D, H;
  const int32_t* row_offsets;
  const int32_t* token_idx;
  const int64_t* cand;
  const int64_t* cand_len;
  int L;
  int has_plan;
  aspa_shortlist_plan plan;
  const float* add_mask;
  void* out;
  int out_dtype, out_layout;
  const int32_t* out_row_map;  // token-major only: (B*T) row -> compact row, or NULL
  aspa_kv_layout kv;           // element strides of k and v (batch, head, token)
  float scale;
  float* ws_m;  // [total_rows] running max (natural-log domain, already scaled)
  float* ws_l;  // [total_rows] running denominator
  float* ws_o;  // [total_rows][D] unnormalised output
  int extras_only;  // second pass: skip the local window, merge with ws_*
  int anchors_done; // extras pass: 1 = the strided anchor keys were already folded into ws_* by the 64-row tile pass (the
                    // slot that clamps to key 0 is still open), 2 = by the group pass, clamping slot included
  int read_partial; // tile pass: start from the state in ws_* instead of an empty one
  // anchor tile pass: rows regrouped by (head, token % stride); keys are the strided view K[rho + stride * i]
  int an_stride;            // 0 = ordinary window pass
  int an_window, an_jmin;   // strided keys i in (it - jmin - an_window, it - jmin]
  const int32_t* an_offsets;  // (heads * stride + 1) first row of every (head, residue) group
  const int32_t* an_tok;      // per regrouped row: token / stride - jmin, or ANCHOR_NO_KEYS
  const int32_t* an_row;      // per regrouped row: its position in the head-grouped packing (workspace row)
  int write_partial;  // window pass: write ws_* instead of the final output
};

// Element offset of out[bh, t, 0].  With a row map the token-major row b*T + t is replaced by its compact slot.
__device__ __forceinline__ int64_t out_row_base(const AttnParams& p, int bh, int t) {
  if (p.out_layout == ASPA_OUT_HEAD_MAJOR) return ((int64_t)bh * p.T + t) * p.D;
  const int b = bh / p.H, h = bh % p.H;
  int64_t row = (int64_t)b * p.T + t;
  if (p.out_row_map) row = p.out_row_map[row];
  return (row * p.H + h) * p.D;
}

__device__ __forceinline__ void store_out(const AttnParams& p, int64_t idx, float v) {
  if (p.out_dtype == ASPA_BF16)
    reinterpret_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<float*>(p.out)[idx] = v;
}

// tcgen05 / tensor-memory version of the window pass (attention_tc.cu).  Same parameter block and semantics as
// attn_window_kernel; returns false when the shape is not one it covers (head_dim 64, bf16 or int8 only).
bool launch_window_tc(const AttnParams& p, int qkv_dtype, int max_rows, int groups, cudaStream_t st);

// Warp-MMA tile version of the prototype-pick pass of the INT8 shortlist (attention_picks.cu): rows of one (head,
// 128-token block) pair share their pick list.  picks_tiles_ok says whether the call is one it covers.
bool picks_tiles_ok(const AttnParams& p, int qkv_dtype);
void launch_picks_tiles(const AttnParams& p, int qkv_dtype, cudaStream_t st);
// The same kernel over the rows of a (head, token % stride) group and the strided key sequence of that residue class:
// the anchor pass for groups too small for the 64-row tile pass.  `p` carries the regrouped rows (an_*).
// After 64-row tile passes for window and anchors of a plan without picks: the slot that clamps to key 0, and the final
// normalisation of the workspace state (int8 or bf16, head_dim 64).
void launch_finalise_rows(const AttnParams& p, int qkv_dtype, int max_rows, cudaStream_t st);
bool anchor_groups_ok(const AttnParams& p, int qkv_dtype);
void launch_anchor_groups(const AttnParams& p, int qkv_dtype, cudaStream_t st);

}  // namespace aspa
