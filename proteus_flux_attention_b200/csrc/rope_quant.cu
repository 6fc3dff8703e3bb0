// RoPE tables, RoPE + head-major relayout of the fused QKV projection, per-head amax and INT8 quantiser,
// row gather.  All HBM-streaming kernels: 16-byte vector accesses, one pass over the data.
#include "common.cuh"

namespace aspa {

__global__ void rope_table_kernel(const float* __restrict__ inv_freq, int T, int half, int dtype,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)T * half) return;
  const int t = (int)(i / half), j = (int)(i % half);
  const float ang = __fmul_rn((float)t, inv_freq[j]);
  float c = cosf(ang), s = sinf(ang);
  if (dtype == ASPA_BF16) {
    c = bf16_round(c);
    s = bf16_round(s);
  }
  cos_t[i] = c;
  sin_t[i] = s;
}

__device__ __forceinline__ float rope_mix(float a, float c, float rot, float s, bool bf) {
  // (a * cos) + (rot * sin), each op rounded in the activation dtype like the eager reference
  float p = __fmul_rn(a, c), q = __fmul_rn(rot, s);
  if (bf) {
    p = bf16_round(p);
    q = bf16_round(q);
  }
  float r = __fadd_rn(p, q);
  return bf ? bf16_round(r) : r;
}

// One thread moves 8 consecutive channels of one (token, section, head).  E = elements per thread.
template <typename T>
__global__ void __launch_bounds__(256) rope_relayout_kernel(const T* __restrict__ qkv, int B, int Tn, int H, int D,
                                                            const float* __restrict__ cos_t,
                                                            const float* __restrict__ sin_t, T* __restrict__ q,
                                                            T* __restrict__ k, T* __restrict__ v,
                                                            float* __restrict__ amax) {
  constexpr int E = 8;
  const int C = H * D;
  const int vec_per_tok = 3 * C / E;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)B * Tn * vec_per_tok;
  float local_max = 0.f;
  int sec = 0, bh = 0;
  const bool active = gid < total;
  if (active) {
    const int64_t bt = gid / vec_per_tok;
    const int vi = (int)(gid % vec_per_tok);
    const int ch = vi * E;  // channel inside 3C
    sec = ch / C;
    const int c_in = ch % C;
    const int h = c_in / D, d0 = c_in % D;
    const int b = (int)(bt / Tn), t = (int)(bt % Tn);
    bh = b * H + h;
    float val[E];
    const T* src = qkv + bt * (3 * (int64_t)C) + ch;
    if (sizeof(T) == 2) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int i = 0; i < E; ++i) val[i] = __bfloat162float(e[i]);
    } else {
      const float4 a = reinterpret_cast<const float4*>(src)[0], c4 = reinterpret_cast<const float4*>(src)[1];
      val[0] = a.x; val[1] = a.y; val[2] = a.z; val[3] = a.w;
      val[4] = c4.x; val[5] = c4.y; val[6] = c4.z; val[7] = c4.w;
    }
    if (sec < 2 && cos_t != nullptr) {
      const int half = D / 2;
      const float* cr = cos_t + (int64_t)t * half + d0 / 2;
      const float* sr = sin_t + (int64_t)t * half + d0 / 2;
#pragma unroll
      for (int i = 0; i < E; i += 2) {
        const float c = cr[i / 2], s = sr[i / 2];
        const float ev = val[i], od = val[i + 1];
        val[i] = rope_mix(ev, c, -od, s, sizeof(T) == 2);
        val[i + 1] = rope_mix(od, c, ev, s, sizeof(T) == 2);
      }
    }
    T* dst = (sec == 0 ? q : (sec == 1 ? k : v)) + ((int64_t)bh * Tn + t) * D + d0;
    if (sizeof(T) == 2) {
      uint4 raw;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
      for (int i = 0; i < E; ++i) e[i] = __float2bfloat16_rn(val[i]);
      *reinterpret_cast<uint4*>(dst) = raw;
    } else {
      reinterpret_cast<float4*>(dst)[0] = make_float4(val[0], val[1], val[2], val[3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(val[4], val[5], val[6], val[7]);
    }
    if (amax) {
#pragma unroll
      for (int i = 0; i < E; ++i) local_max = fmaxf(local_max, fabsf(val[i]));
    }
  }
  if (amax) {
    // lanes of a warp may belong to different (section, bh) groups: the lowest lane of every group
    // folds in its peers and issues one atomic (non-negative floats order like their bit patterns)
    const int key = active ? (sec * B * H + bh) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    const int leader = __ffs(peers) - 1;
    float gm = local_max;
    for (int l = 0; l < 32; ++l) {
      const float o = __shfl_sync(0xffffffffu, local_max, l);
      if ((peers >> l) & 1u) gm = fmaxf(gm, o);
    }
    if (active && (int)(threadIdx.x & 31) == leader) atomicMax(reinterpret_cast<int*>(amax + key), __float_as_int(gm));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) head_amax_kernel(const T* __restrict__ x, int64_t per_head,
                                                        float* __restrict__ amax) {
  // grid (chunks, heads); non-negative floats order like their int bit patterns
  __shared__ float red[8];
  const T* p = x + (int64_t)blockIdx.y * per_head;
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_head; i += (int64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(ld_as_float<T>(p, i)));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    atomicMax(reinterpret_cast<int*>(amax + blockIdx.y), __float_as_int(m));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) quantize_int8_kernel(const T* __restrict__ x, int64_t per_head,
                                                            const float* __restrict__ amax,
                                                            int8_t* __restrict__ out, float* __restrict__ scales) {
  const int head = blockIdx.y;
  const float scale = fmaxf(__fdiv_rn(amax[head], 127.0f), 1e-6f);
  if (blockIdx.x == 0 && threadIdx.x == 0) scales[head] = scale;
  const T* p = x + (int64_t)head * per_head;
  int8_t* o = out + (int64_t)head * per_head;
  const int64_t nvec = (per_head % 8 == 0) ? per_head / 8 : 0;  // vector path needs 16-byte aligned heads
  for (int64_t vi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += (int64_t)gridDim.x * blockDim.x) {
    float val[8];
    if (sizeof(T) == 2) {
      const uint4 raw = reinterpret_cast<const uint4*>(p)[vi];
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) val[i] = __bfloat162float(e[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) val[i] = ld_as_float<T>(p, vi * 8 + i);
    }
    union { int8_t b[8]; uint2 u; } pk;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float r = rintf(__fdiv_rn(val[i], scale));
      pk.b[i] = (int8_t)fminf(fmaxf(r, -127.f), 127.f);
    }
    reinterpret_cast<uint2*>(o)[vi] = pk.u;
  }
  // tail (per_head not a multiple of 8)
  for (int64_t i = nvec * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < per_head;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float r = rintf(__fdiv_rn(ld_as_float<T>(p, i), scale));
    o[i] = (int8_t)fminf(fmaxf(r, -127.f), 127.f);
  }
}

__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src,
                                                          const int64_t* __restrict__ idx,
                                                          const int32_t* __restrict__ count_dev, int64_t max_rows,
                                                          int64_t vec_per_row, uint4* __restrict__ dst) {
  const int64_t rows = count_dev ? min((int64_t)count_dev[0], max_rows) : max_rows;
  const int64_t total = rows * vec_per_row;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = g / vec_per_row, c = g % vec_per_row;
    dst[g] = src[idx[r] * vec_per_row + c];
  }
}

}  // namespace aspa

using namespace aspa;

extern "C" int aspa_rope_table(const float* inv_freq, int T, int D, int dtype, float* cos_t, float* sin_t,
                               void* stream) {
  ASPA_CHECK_ARG(inv_freq && cos_t && sin_t, "null pointer");
  ASPA_CHECK_ARG(T > 0 && D > 0 && D % 2 == 0, "bad sizes");
  const int64_t n = (int64_t)T * (D / 2);
  rope_table_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, (cudaStream_t)stream>>>(inv_freq, T, D / 2, dtype, cos_t, sin_t);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_rope_relayout(const void* qkv, int dtype, int B, int T, int H, int D, const float* cos_t,
                                  const float* sin_t, void* q, void* k, void* v, float* amax, void* stream) {
  ASPA_CHECK_ARG(qkv && q && k && v, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && H > 0 && D > 0 && D % 8 == 0, "head_dim must be a multiple of 8");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  ASPA_CHECK_ARG((cos_t == nullptr) == (sin_t == nullptr), "cos/sin tables come together");
  const int64_t total = (int64_t)B * T * (3 * H * D / 8);
  const unsigned grid = (unsigned)ceil_div(total, 256);
  if (dtype == ASPA_BF16)
    rope_relayout_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)qkv, B, T, H, D, cos_t, sin_t, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, amax);
  else
    rope_relayout_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)qkv, B, T, H, D, cos_t, sin_t,
                                                                       (float*)q, (float*)k, (float*)v, amax);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_head_amax(const void* x, int dtype, int heads, int64_t per_head, float* amax, void* stream) {
  ASPA_CHECK_ARG(x && amax && heads > 0 && per_head > 0, "bad arguments");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  cudaStream_t st = (cudaStream_t)stream;
  cudaMemsetAsync(amax, 0, sizeof(float) * heads, st);
  const dim3 grid((unsigned)std::min<int64_t>(ceil_div(per_head, 256 * 8), 1024), heads);
  if (dtype == ASPA_BF16)
    head_amax_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, per_head, amax);
  else
    head_amax_kernel<float><<<grid, 256, 0, st>>>((const float*)x, per_head, amax);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_quantize_int8(const void* x, int dtype, int heads, int64_t per_head, const float* amax,
                                  int8_t* out, float* scales, void* stream) {
  ASPA_CHECK_ARG(x && amax && out && scales && heads > 0 && per_head > 0, "bad arguments");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  const dim3 grid((unsigned)std::min<int64_t>(ceil_div(per_head, 256 * 8), 2048), heads);
  if (dtype == ASPA_BF16)
    quantize_int8_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, per_head, amax, out, scales);
  else
    quantize_int8_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)x, per_head, amax, out, scales);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_gather_rows(const void* src, const int64_t* idx, const int32_t* count_dev, int64_t max_rows,
                                int64_t row_bytes, void* dst, void* stream) {
  ASPA_CHECK_ARG(src && idx && dst, "null pointer");
  ASPA_CHECK_ARG(max_rows >= 0 && row_bytes > 0 && row_bytes % 16 == 0, "row_bytes must be a multiple of 16");
  if (max_rows == 0) return ASPA_OK;
  const int64_t total = max_rows * (row_bytes / 16);
  gather_rows_kernel<<<(unsigned)std::min<int64_t>(ceil_div(total, 256), 148 * 16), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, idx, count_dev, max_rows, row_bytes / 16, (uint4*)dst);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
