// Router on the 5th-generation tensor cores (bf16 activations).
//
// One CTA owns a tile of 128 tokens.  The skinny product  [128 tokens x C] . [C x N]  with
//   N = G router columns + 3*G prototype columns (the fp32 normalised prototypes split into three bf16 terms
//       hi + mid + lo, so that the sum of the three products carries fp32 precision)
// runs as tcgen05.mma (M=128, N, K=16, bf16 x bf16 -> fp32) with the accumulator in tensor memory.
//   warp 4      : TMA producer — 128x64 activation tiles and Nx64 weight tiles, 128-byte swizzle, 3-stage ring
//   warp 5      : allocates tensor memory, issues the MMAs, commits them to the "stage free" and "accumulator
//                 ready" mbarriers, frees tensor memory at the end
//   warps 0..3  : while the ring runs, sum x^2 of their own token row straight from the staged tiles (the L2 norm
//                 the cosine needs); afterwards read the accumulator with tcgen05.ld and run the per-token epilogue
//                 (softmaxes, prototype blend, importance) shared with the CUDA-core kernel.
// x is read from HBM exactly once; the weight tiles (<= 256 KB in total) stay in L2.
// Every mbarrier wait is bounded: on expiry the kernel raises a status word, skips its remaining work, still
// frees tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "router_epilogue.cuh"

namespace aspa {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;       // bf16 per k-block = one 128-byte swizzle row
constexpr int TC_STAGES = 3;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;   // 16 KB
constexpr int TC_B_BYTES_MAX = 128 * TC_BK * 2; // 16 KB
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES_MAX;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait: returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < TC_SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// K-major operand tile, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused by swizzled K-major layouts), 16-byte units
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;            // descriptor version for this architecture
  d |= (uint64_t)2 << 61;            // 128-byte swizzle
  return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__global__ void __launch_bounds__(192, 2)
router_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, int64_t n,
                 int C, int G, int N, int has_proto, const float* __restrict__ conf_eps,
                 const float* __restrict__ usage_bias, float proto_temp, float proto_threshold, float proto_span,
                 float proto_blend, float usage_boost, float* __restrict__ gate_probs,
                 float* __restrict__ importance, float* __restrict__ proto_sim, float* __restrict__ blend,
                 float* __restrict__ stat_partials, int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TC_STAGES * TC_STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 1);
  int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);
  const uint32_t full0 = s_addr(bars), empty0 = s_addr(bars + TC_STAGES), accbar = s_addr(bars + 2 * TC_STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x;
  const int num_k = C / TC_BK;
  const uint32_t tmem_cols = N <= 32 ? 32 : (N <= 64 ? 64 : 128);

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);       // the producer's expect_tx arrival; TMA completes the bytes
      mbar_init(empty0 + 8 * s, 1 + 4);  // one MMA commit + one arrival per norm warp
    }
    mbar_init(accbar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {  // whole warp: allocate tensor memory, publish its base address in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  float nsq = 0.f;
  if (warp == 4) {
    if (lane == 0) {
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % TC_STAGES;
        const uint32_t ph = (kb / TC_STAGES) & 1;
        if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) { atomicExch(abort_flag, 1); atomicExch(status, 1); break; }
        const uint32_t a_dst = s_addr(smem + s * TC_STAGE_BYTES), b_dst = a_dst + TC_A_BYTES;
        mbar_expect_tx(full0 + 8 * s, TC_A_BYTES + N * TC_BK * 2);
        tma_load_2d(a_dst, &tmap_x, kb * TC_BK, tile * TC_BM, full0 + 8 * s);
        tma_load_2d(b_dst, &tmap_w, kb * TC_BK, 0, full0 + 8 * s);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // instruction descriptor: D fp32, A/B bf16, both K-major, N/8 at bit 17, M/16 at bit 24
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < num_k && ok; ++kb) {
        const int s = kb % TC_STAGES;
        const uint32_t ph = (kb / TC_STAGES) & 1;
        if (!mbar_wait(full0 + 8 * s, ph)) { atomicExch(abort_flag, 1); atomicExch(status, 2); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = s_addr(smem + s * TC_STAGE_BYTES), b_addr = a_addr + TC_A_BYTES;
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) {
          umma_bf16(tmem_base, umma_desc_k_sw128(a_addr + k * 32), umma_desc_k_sw128(b_addr + k * 32), idesc,
                    (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(empty0 + 8 * s);  // arrives once the MMAs above have finished reading this stage
      }
      umma_commit(accbar);            // arrives once every MMA has landed in tensor memory
    }
  } else {
    // norm warps: thread r owns token row r of the tile
    const int r = threadIdx.x;
    bool ok = true;
    for (int kb = 0; kb < num_k && ok; ++kb) {
      const int s = kb % TC_STAGES;
      const uint32_t ph = (kb / TC_STAGES) & 1;
      if (!mbar_wait(full0 + 8 * s, ph)) { atomicExch(abort_flag, 1); atomicExch(status, 3); ok = false; break; }
      const unsigned char* row = smem + s * TC_STAGE_BYTES + r * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // the swizzle only permutes 16-byte chunks inside a row; rotate the start so lanes hit different banks
        const uint4 raw = *reinterpret_cast<const uint4*>(row + (((j + r) & 7) << 4));
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          nsq = fmaf(f.x, f.x, nsq);
          nsq = fmaf(f.y, f.y, nsq);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
  }

  // ---- epilogue -----------------------------------------------------------------------------------------
  float st_sim = 0.f, st_bs = 0.f;
  float* es = reinterpret_cast<float*>(smem);  // reuses the ring: every load and MMA has completed by now
  const int stride = 2 * G + 1;
  if (warp < 4) {
    const int r = threadIdx.x;
    bool ok = *reinterpret_cast<volatile int*>(abort_flag) == 0;
    if (ok && !mbar_wait(accbar, 0)) { atomicExch(abort_flag, 1); atomicExch(status, 4); ok = false; }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      float* row = es + r * stride;
      for (int c0 = 0; c0 < N; c0 += 16) {
        float v[16];
        tmem_ld16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int c = c0 + i;
          if (c < G) row[c] = v[i];
          else if (c < 2 * G) row[c] = v[i];          // hi term
          else if (c < 4 * G) row[G + (c - 2 * G) % G] += v[i];  // mid and lo terms fold into the same slot
        }
      }
      const int64_t tok = (int64_t)tile * TC_BM + r;
      if (tok < n) {
        float imp;
        router_epilogue(row, 1, G, true, has_proto != 0, nsq, conf_eps, usage_bias, proto_temp, proto_threshold,
                        proto_span, proto_blend, usage_boost, gate_probs + tok * G, &imp,
                        proto_sim ? proto_sim + tok : nullptr, blend ? blend + tok : nullptr, &st_sim, &st_bs);
        importance[tok] = imp;
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (stat_partials) {  // same layout as the CUDA-core kernel: one entry per 64 tokens
    float* sbuf = es + TC_BM * stride;
    if (warp < 4) {
      sbuf[threadIdx.x] = st_sim;
      sbuf[TC_BM + threadIdx.x] = st_bs;
    }
    __syncthreads();
    if (threadIdx.x < 2) {
      const int64_t nb = (n + 63) / 64, blk = (int64_t)tile * 2 + threadIdx.x;
      if (blk < nb) {
        float a = 0.f, b = 0.f, c = 0.f;
        for (int i = 0; i < 64; ++i) {
          a += sbuf[threadIdx.x * 64 + i];
          b += sbuf[TC_BM + threadIdx.x * 64 + i];
          c += sbuf[TC_BM + threadIdx.x * 64 + i] > 0.f ? 1.f : 0.f;
        }
        stat_partials[blk] = a;
        stat_partials[nb + blk] = b;
        stat_partials[2 * nb + blk] = c;
      }
    }
  }
  if (warp == 5) {
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

extern "C" int aspa_router_fwd_tc(const void* x, int64_t n, int C, const void* w_router, int G,
                                  const float* proto_hat, const float* conf_eps, const float* usage_bias,
                                  float proto_temp, float proto_threshold, float proto_span, float proto_blend,
                                  float usage_boost, float* gate_probs, float* importance, float* proto_sim,
                                  float* blend, float* stat_partials, void* scratch, int32_t* status, void* stream) {
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
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, (uint64_t)n, (uint64_t)C, TC_BM) || !make_map(&mw, wcat, (uint64_t)N, (uint64_t)C, (uint32_t)N)) {
    set_error("aspa_router_fwd_tc: cuTensorMapEncodeTiled failed");
    return ASPA_ERR_CUDA;
  }
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(router_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
    attr_set = true;
  }
  router_tc_kernel<<<(unsigned)ceil_div(n, TC_BM), 192, TC_SMEM_BYTES, st>>>(
      mx, mw, n, C, G, N, has_proto ? 1 : 0, conf_eps, usage_bias, proto_temp, proto_threshold, proto_span,
      proto_blend, usage_boost, gate_probs, importance, proto_sim, blend, stat_partials, status);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
