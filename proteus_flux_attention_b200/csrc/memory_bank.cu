// Key/value memory bank of the layer (reference models/aspa.py:932-1035): per head a ring of `slots` mean keys and mean
// values, pushed once per (batch, head) pair that has active rows in a shortlist call.
//
// What the bank changes in a call.  The reference appends the ring to k and v and hands ids `T + j` to the candidate
// builder as extra candidates; the builder then clamps every candidate to the row's own token (sa.py:570-571), so the
// memory ids collapse onto the row itself and never reach the attention.  What remains observable is (a) the state of
// the four buffers after the call and (b), with INT8 on, the per-head scales of k and v, whose amax is taken over the
// appended rows too.  Both are built here; no attention kernel reads the bank.
#include "common.cuh"

namespace aspa {

constexpr int MB_THREADS = 256;

template <typename T>
__device__ __forceinline__ float round_to(float x);
template <>
__device__ __forceinline__ float round_to<float>(float x) { return x; }
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// One CTA per head; the (batch, head) pairs of that head are taken in batch order, as the reference's loop over the
// ascending active head list does.  Per pair: masked mean of its key and value rows (sum accumulated in fp32 and
// rounded to the activation dtype, divided by the count, rounded again), whole-head decay, write under the pointer,
// advance the pointer.
template <typename T>
__global__ void __launch_bounds__(MB_THREADS) memory_update_kernel(
    const T* __restrict__ k, const T* __restrict__ v, aspa_kv_layout lay, int B, int H, int D,
    const int32_t* __restrict__ row_offsets, const int32_t* __restrict__ token_idx, float decay,
    float* __restrict__ mem_k, float* __restrict__ mem_v, float* __restrict__ mem_c, int64_t* __restrict__ mem_ptr,
    int S) {
  __shared__ float red_k[MB_THREADS], red_v[MB_THREADS];
  const int h = blockIdx.x;
  const int phases = MB_THREADS / D;          // D <= 256 (checked by the host)
  const int d = threadIdx.x % D, ph = threadIdx.x / D;
  const bool live = ph < phases;
  for (int b = 0; b < B; ++b) {
    const int bh = b * H + h;
    const int start = row_offsets[bh], cnt = row_offsets[bh + 1] - start;
    if (cnt <= 0) continue;                   // uniform over the CTA
    const T* kh = k + (int64_t)b * lay.k_batch + (int64_t)h * lay.k_head;
    const T* vh = v + (int64_t)b * lay.v_batch + (int64_t)h * lay.v_head;
    float sk = 0.f, sv = 0.f;
    if (live) {
      for (int r = ph; r < cnt; r += phases) {
        const int64_t t = token_idx[start + r];
        sk += ld_as_float<T>(kh, t * lay.k_token + d);
        sv += ld_as_float<T>(vh, t * lay.v_token + d);
      }
    }
    red_k[threadIdx.x] = sk;
    red_v[threadIdx.x] = sv;
    __syncthreads();
    if (threadIdx.x < D) {
      float ak = 0.f, av = 0.f;
      for (int p = 0; p < phases; ++p) {      // fixed order
        ak += red_k[p * D + d];
        av += red_v[p * D + d];
      }
      const float c = (float)cnt;
      const float mk = round_to<T>(__fdiv_rn(round_to<T>(ak), c));
      const float mv = round_to<T>(__fdiv_rn(round_to<T>(av), c));
      const int slot = (int)mem_ptr[h];
      float* hk = mem_k + (int64_t)h * S * D;
      float* hv = mem_v + (int64_t)h * S * D;
      for (int s = 0; s < S; ++s) {
        hk[s * D + d] = s == slot ? mk : hk[s * D + d] * decay;
        hv[s * D + d] = s == slot ? mv : hv[s * D + d] * decay;
      }
    }
    __syncthreads();                          // everyone has read mem_ptr[h] and the partial sums
    if (threadIdx.x == 0) {
      const int slot = (int)mem_ptr[h];
      for (int s = 0; s < S; ++s) mem_c[h * S + s] = s == slot ? (float)cnt : mem_c[h * S + s] * decay;
      mem_ptr[h] = (slot + 1) % S;
    }
    __syncthreads();
  }
}

// amax_k[bh], amax_v[bh] = max(themselves, amax over the memory rows the reference appends for that pair): the first c
// rows of the ring read from the pointer on, c = number of slots of the head with a positive count, each value rounded
// to the activation dtype first.  Pairs without active rows are left alone.
template <typename T>
__global__ void __launch_bounds__(MB_THREADS) memory_fold_amax_kernel(
    const float* __restrict__ mem_k, const float* __restrict__ mem_v, const float* __restrict__ mem_c,
    const int64_t* __restrict__ mem_ptr, int H, int S, int D, const int32_t* __restrict__ row_offsets,
    float* __restrict__ amax_k, float* __restrict__ amax_v) {
  __shared__ float red_k[MB_THREADS / 32], red_v[MB_THREADS / 32];
  const int bh = blockIdx.x, h = bh % H;
  if (row_offsets[bh + 1] - row_offsets[bh] <= 0) return;
  int c = 0;
  for (int s = 0; s < S; ++s) c += mem_c[h * S + s] > 0.f ? 1 : 0;
  if (c == 0) return;
  const int p0 = (int)mem_ptr[h];
  float mk = 0.f, mv = 0.f;
  for (int i = threadIdx.x; i < c * D; i += blockDim.x) {
    const int slot = (p0 + i / D) % S, d = i % D;
    mk = fmaxf(mk, fabsf(round_to<T>(mem_k[((int64_t)h * S + slot) * D + d])));
    mv = fmaxf(mv, fabsf(round_to<T>(mem_v[((int64_t)h * S + slot) * D + d])));
  }
  mk = warp_max(mk);
  mv = warp_max(mv);
  if ((threadIdx.x & 31) == 0) {
    red_k[threadIdx.x >> 5] = mk;
    red_v[threadIdx.x >> 5] = mv;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 0; w < MB_THREADS / 32; ++w) {
      mk = fmaxf(mk, red_k[w]);
      mv = fmaxf(mv, red_v[w]);
    }
    amax_k[bh] = fmaxf(amax_k[bh], mk);
    amax_v[bh] = fmaxf(amax_v[bh], mv);
  }
}

}  // namespace aspa

using namespace aspa;

extern "C" int aspa_memory_update(const void* k, const void* v, int dtype, const aspa_kv_layout* kv_layout, int B, int H,
                                  int T, int D, const int32_t* row_offsets, const int32_t* token_idx, float decay,
                                  float* mem_keys, float* mem_values, float* mem_counts, int64_t* mem_ptr, int slots,
                                  void* stream) {
  ASPA_CHECK_ARG(k && v && row_offsets && token_idx && mem_keys && mem_values && mem_counts && mem_ptr, "null pointer");
  ASPA_CHECK_ARG(B > 0 && H > 0 && T > 0 && D > 0 && D <= MB_THREADS && slots > 0, "bad sizes (head_dim <= 256)");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  if (!(decay < 1.0f)) return ASPA_OK;   // the reference writes nothing at a decay of 1 (aspa.py:959)
  aspa_kv_layout lay;
  if (kv_layout) {
    lay = *kv_layout;
  } else {
    lay.k_token = lay.v_token = D;
    lay.k_head = lay.v_head = (int64_t)T * D;
    lay.k_batch = lay.v_batch = (int64_t)H * T * D;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == ASPA_BF16)
    memory_update_kernel<__nv_bfloat16><<<H, MB_THREADS, 0, st>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, lay, B, H, D,
                                                                  row_offsets, token_idx, decay, mem_keys, mem_values,
                                                                  mem_counts, mem_ptr, slots);
  else
    memory_update_kernel<float><<<H, MB_THREADS, 0, st>>>((const float*)k, (const float*)v, lay, B, H, D, row_offsets,
                                                          token_idx, decay, mem_keys, mem_values, mem_counts, mem_ptr,
                                                          slots);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_memory_fold_amax(const float* mem_keys, const float* mem_values, const float* mem_counts,
                                     const int64_t* mem_ptr, int B, int H, int slots, int D, int dtype,
                                     const int32_t* row_offsets, float* amax_k, float* amax_v, void* stream) {
  ASPA_CHECK_ARG(mem_keys && mem_values && mem_counts && mem_ptr && row_offsets && amax_k && amax_v, "null pointer");
  ASPA_CHECK_ARG(B > 0 && H > 0 && slots > 0 && D > 0, "bad sizes");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == ASPA_BF16)
    memory_fold_amax_kernel<__nv_bfloat16><<<B * H, MB_THREADS, 0, st>>>(mem_keys, mem_values, mem_counts, mem_ptr, H, slots,
                                                                         D, row_offsets, amax_k, amax_v);
  else
    memory_fold_amax_kernel<float><<<B * H, MB_THREADS, 0, st>>>(mem_keys, mem_values, mem_counts, mem_ptr, H, slots, D,
                                                                 row_offsets, amax_k, amax_v);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
