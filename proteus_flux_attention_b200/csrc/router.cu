// Router: gate probabilities, prototype similarity, blend and token importance.
// fp32 accumulation on CUDA cores over 64-token tiles staged through shared memory.
#include <stdarg.h>

#include "common.cuh"
#include "router_epilogue.cuh"

namespace aspa {

static thread_local char g_err[512] = "ok";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

constexpr int RT_TM = 64;   // tokens per CTA
constexpr int RT_KC = 32;   // reduction chunk
constexpr int RT_NMAX = 128;

template <typename T>
__global__ void __launch_bounds__(256) router_generic_kernel(
    const T* __restrict__ x, int64_t n, int C, const T* __restrict__ w_router, int G,
    const float* __restrict__ proto_hat, const float* __restrict__ conf_eps,
    const float* __restrict__ usage_bias, float proto_temp, float proto_threshold, float proto_span,
    float proto_blend, float usage_boost, float* __restrict__ gate_probs, float* __restrict__ importance,
    float* __restrict__ proto_sim, float* __restrict__ blend, float* __restrict__ stat_partials, int NT) {
  extern __shared__ float smem[];
  float* xs = smem;                             // [RT_TM][RT_KC+1]
  float* ws = xs + RT_TM * (RT_KC + 1);         // [NT][RT_KC+1]
  float* es = ws + RT_NMAX * (RT_KC + 1);       // [RT_TM][NT+1]
  float* ns = es + RT_TM * (RT_NMAX + 1);       // [RT_TM]
  const bool has_proto = proto_hat != nullptr;
  const int N = has_proto ? 2 * G : G;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t tok0 = (int64_t)blockIdx.x * RT_TM;
  const int NJ = NT / 16;
  float acc[4][8];
  float nsq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < C; k0 += RT_KC) {
    {  // x tile: 64 tokens x 32 k, 8 contiguous elements per thread
      const int r = tid >> 2, kk = (tid & 3) * 8;
      const int64_t tok = tok0 + r;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int k = k0 + kk + e;
        xs[r * (RT_KC + 1) + kk + e] = (tok < n && k < C) ? ld_as_float<T>(x, tok * C + k) : 0.f;
      }
    }
    for (int idx = tid; idx < NT * 4; idx += 256) {
      const int r = idx >> 2, kk = (idx & 3) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int k = k0 + kk + e;
        float v = 0.f;
        if (k < C && r < N) v = r < G ? ld_as_float<T>(w_router, (int64_t)r * C + k) : proto_hat[(int64_t)(r - G) * C + k];
        ws[r * (RT_KC + 1) + kk + e] = v;
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < RT_KC; ++k) {
      float xv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        xv[i] = xs[(ty * 4 + i) * (RT_KC + 1) + k];
        nsq[i] = fmaf(xv[i], xv[i], nsq[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j < NJ) {
          const float wv = ws[(tx + 16 * j) * (RT_KC + 1) + k];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i][j] = fmaf(xv[i], wv, acc[i][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < NJ) es[(ty * 4 + i) * (RT_NMAX + 1) + tx + 16 * j] = acc[i][j];
    if (tx == 0) ns[ty * 4 + i] = nsq[i];
  }
  __syncthreads();
  float st_sim = 0.f, st_bs = 0.f;
  if (tid < RT_TM) {
    const int64_t tok = tok0 + tid;
    if (tok < n) {
      float imp;
      router_epilogue(es + tid * (RT_NMAX + 1), 1, G, sizeof(T) == 2, has_proto, ns[tid], conf_eps, usage_bias,
                      proto_temp, proto_threshold, proto_span, proto_blend, usage_boost, gate_probs + tok * G, &imp,
                      proto_sim ? proto_sim + tok : nullptr, blend ? blend + tok : nullptr, &st_sim, &st_bs);
      importance[tok] = imp;
    }
  }
  if (stat_partials) {
    __syncthreads();
    if (tid < RT_TM) {
      xs[tid] = st_sim;
      xs[RT_TM + tid] = st_bs;
    }
    __syncthreads();
    if (tid == 0) {
      float a = 0.f, b = 0.f, c = 0.f;
      for (int i = 0; i < RT_TM; ++i) {
        a += xs[i];
        b += xs[RT_TM + i];
        c += xs[RT_TM + i] > 0.f ? 1.f : 0.f;
      }
      const int64_t nb = gridDim.x;
      stat_partials[blockIdx.x] = a;
      stat_partials[nb + blockIdx.x] = b;
      stat_partials[2 * nb + blockIdx.x] = c;
    }
  }
}

__global__ void normalize_rows_kernel(const float* __restrict__ src, int cols, float eps, float* __restrict__ dst) {
  __shared__ float red[33];
  const float* s = src + (int64_t)blockIdx.x * cols;
  float acc = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) acc = fmaf(s[c], s[c], acc);
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    red[32] = fmaxf(sqrtf(t), eps);
  }
  __syncthreads();
  const float d = red[32];
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[(int64_t)blockIdx.x * cols + c] = __fdiv_rn(s[c], d);
}

__global__ void reduce_partials_kernel(const float* __restrict__ partials, int64_t n_blocks, float* __restrict__ out) {
  // one warp per series, fixed summation order -> run-to-run identical results
  const float* p = partials + (int64_t)blockIdx.x * n_blocks;
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < n_blocks; i += 32) acc += p[i];
  acc = warp_sum(acc);
  if (threadIdx.x == 0) out[blockIdx.x] = acc;
}

// Everything the host may want to know about one layer call, gathered into one fp64 record by a single CTA:
// [row offsets | kept per batch row | k, adaptive k | selected-score sum, entropy sum | prototype sums (3) | status].
// Series sums use the order of reduce_partials_kernel (one warp per series, lane-strided, then a shuffle tree).
__global__ void __launch_bounds__(256) stats_record_kernel(const int32_t* __restrict__ row_offsets, int n_offsets,
                                                           const int32_t* __restrict__ kept, int n_kept,
                                                           double kept_fill, const int32_t* __restrict__ k_dev,
                                                           double k_fill, const float* __restrict__ head_partials,
                                                           int64_t head_blocks,
                                                           const float* __restrict__ proto_partials,
                                                           int64_t proto_blocks, const int32_t* __restrict__ status,
                                                           double* __restrict__ rec) {
  for (int i = threadIdx.x; i < n_offsets; i += blockDim.x) rec[i] = (double)row_offsets[i];
  double* r = rec + n_offsets;
  for (int i = threadIdx.x; i < n_kept; i += blockDim.x) r[i] = kept ? (double)kept[i] : kept_fill;
  r += n_kept;
  if (threadIdx.x < 2) r[threadIdx.x] = k_dev ? (double)k_dev[threadIdx.x] : k_fill;
  r += 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < 5) {
    const bool head = warp < 2;
    const float* p = head ? head_partials : proto_partials;
    const int64_t nb = head ? head_blocks : proto_blocks;
    const int series = head ? warp : warp - 2;
    float acc = 0.f;
    if (p != nullptr)
      for (int64_t i = lane; i < nb; i += 32) acc += p[(int64_t)series * nb + i];
    acc = warp_sum(acc);
    if (lane == 0) r[warp] = (double)acc;
  }
  if (threadIdx.x == 0) r[5] = status ? (double)status[0] : 0.0;
}

}  // namespace aspa

using namespace aspa;

extern "C" const char* aspa_last_error_string(void) { return aspa::last_error(); }
extern "C" int aspa_version(void) { return 1; }

extern "C" int aspa_router_fwd(const void* x, int x_dtype, int64_t n, int C, const void* w_router, int G,
                               const float* proto_hat, const float* conf_eps, const float* usage_bias,
                               float proto_temp, float proto_threshold, float proto_span, float proto_blend,
                               float usage_boost, float* gate_probs, float* importance, float* proto_sim,
                               float* blend, float* stat_partials, void* stream) {
  ASPA_CHECK_ARG(x && w_router && gate_probs && importance, "null pointer");
  ASPA_CHECK_ARG(n >= 0 && C > 0 && G > 0, "bad sizes");
  ASPA_CHECK_ARG(x_dtype == ASPA_F32 || x_dtype == ASPA_BF16, "x must be fp32 or bf16");
  const bool has_proto = proto_hat != nullptr;
  ASPA_CHECK_ARG((has_proto ? 2 * G : G) <= RT_NMAX, "too many gates (2*G must be <= 128)");
  if (n == 0) return ASPA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int N = has_proto ? 2 * G : G;
  const int NT = (int)ceil_div(N, 16) * 16;
  const size_t smem = sizeof(float) * (RT_TM * (RT_KC + 1) + RT_NMAX * (RT_KC + 1) + RT_TM * (RT_NMAX + 1) + RT_TM);
  const dim3 grid((unsigned)ceil_div(n, RT_TM));
  if (x_dtype == ASPA_F32) {
    cudaFuncSetAttribute(router_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    router_generic_kernel<float><<<grid, 256, smem, st>>>((const float*)x, n, C, (const float*)w_router, G, proto_hat,
                                                          conf_eps, usage_bias, proto_temp, proto_threshold, proto_span,
                                                          proto_blend, usage_boost, gate_probs, importance,
                                                          proto_sim, blend, stat_partials, NT);
  } else {
    cudaFuncSetAttribute(router_generic_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    router_generic_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(
        (const __nv_bfloat16*)x, n, C, (const __nv_bfloat16*)w_router, G, proto_hat, conf_eps, usage_bias,
        proto_temp, proto_threshold, proto_span, proto_blend, usage_boost, gate_probs, importance, proto_sim, blend,
        stat_partials, NT);
  }
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_normalize_rows(const float* src, int rows, int cols, float eps, float* dst, void* stream) {
  ASPA_CHECK_ARG(src && dst && rows > 0 && cols > 0, "bad arguments");
  normalize_rows_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(src, cols, eps, dst);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_reduce_partials(const float* partials, int n_series, int64_t n_blocks, float* out, void* stream) {
  ASPA_CHECK_ARG(partials && out && n_series > 0 && n_blocks >= 0, "bad arguments");
  reduce_partials_kernel<<<n_series, 32, 0, (cudaStream_t)stream>>>(partials, n_blocks, out);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_stats_record(const int32_t* row_offsets, int n_offsets, const int32_t* kept, int n_kept,
                                 double kept_fill, const int32_t* k_dev, double k_fill, const float* head_partials,
                                 int64_t head_blocks, const float* proto_partials, int64_t proto_blocks,
                                 const int32_t* status, double* record, void* stream) {
  ASPA_CHECK_ARG(row_offsets && record && n_offsets > 0 && n_kept >= 0 && head_blocks >= 0 && proto_blocks >= 0,
                 "bad arguments");
  stats_record_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(row_offsets, n_offsets, kept, n_kept, kept_fill, k_dev, k_fill,
                                                           head_partials, head_blocks, proto_partials, proto_blocks, status,
                                                           record);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
