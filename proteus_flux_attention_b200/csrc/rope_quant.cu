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

// RoPE + relayout.  A CTA owns ROPE_TPB consecutive tokens of one batch element; thread v of the CTA owns the
// 16-byte vector v of every one of those tokens, so section / head / channel are computed once and only the token
// advances in the loop.  bf16 uses packed bf16x2 multiply/add (each rounds to nearest even, like the reference's
// eager bf16 ops); fp32 keeps separate fp32 multiplies and adds.
constexpr int ROPE_TPB = 32;
constexpr int ROPE_MAX_HALF = 64;   // head_dim up to 128 takes the packed (cos, sin) table in shared memory

// rintf(v / scale), the quantiser's rounding, without a division per element: for |v / scale| < 256 the product with
// the rounded reciprocal is within 2^-15 of the correctly rounded quotient, so both round to the same integer unless
// the product lies that close to a tie; only then (about one element in ten thousand) the exact quotient decides.
__device__ __forceinline__ float quant_round(float v, float scale, float inv) {
  const float qp = v * inv;
  float r = rintf(qp);
  if (fabsf(qp - r) > 0.499f || !(fabsf(qp) < 256.f)) r = rintf(__fdiv_rn(v, scale));
  return r;
}

__device__ __forceinline__ uint32_t rope_word_bf16(uint32_t x, float c, float s) {
  // x = (even, odd) packed; out = x * (c, c) + (-odd, even) * (s, s)
  const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(&x);
  const uint32_t swapped = __byte_perm(x, 0, 0x1032) ^ 0x00008000u;  // (odd, even) with the new low half negated
  const __nv_bfloat162 rv = *reinterpret_cast<const __nv_bfloat162*>(&swapped);
  const __nv_bfloat162 cv = __floats2bfloat162_rn(c, c), sv = __floats2bfloat162_rn(s, s);
  // the _rn forms forbid fusing the multiply into the add: each step rounds on its own, as in the reference
  const __nv_bfloat162 o = __hadd2_rn(__hmul2_rn(xv, cv), __hmul2_rn(rv, sv));
  return *reinterpret_cast<const uint32_t*>(&o);
}

// MODE 0: write the rotated / relaid-out values (and optionally their per-head amax); MODE 1: amax only, nothing
// written; MODE 2: write symmetric per-head INT8 of the rotated values using the amax of an earlier MODE 1 pass
// (bf16 only: q8/k8/v8 are passed through the q, k, v pointers).
// The same rotation with the factors of a channel pair ready in two words, (cos, cos) and (-sin, sin) as bf16 pairs:
// out = x * (c, c) + (odd, even) * (-s, s); (-s) * odd rounds to the same bf16 as -(odd * s).
__device__ __forceinline__ uint32_t rope_word_bf16_packed(uint32_t x, uint32_t cc, uint32_t ss) {
  const uint32_t swapped = __byte_perm(x, 0, 0x1032);
  const __nv_bfloat162 xv = *reinterpret_cast<const __nv_bfloat162*>(&x);
  const __nv_bfloat162 rv = *reinterpret_cast<const __nv_bfloat162*>(&swapped);
  const __nv_bfloat162 cv = *reinterpret_cast<const __nv_bfloat162*>(&cc), sv = *reinterpret_cast<const __nv_bfloat162*>(&ss);
  const __nv_bfloat162 o = __hadd2_rn(__hmul2_rn(xv, cv), __hmul2_rn(rv, sv));
  return *reinterpret_cast<const uint32_t*>(&o);
}

// max(a, |b|, |c|) that keeps a NaN
__device__ __forceinline__ float max3_abs_nan(float a, float b, float c) {
  float d;
  asm("{\n\t.reg .f32 t, u;\n\tabs.f32 t, %2;\n\tabs.f32 u, %3;\n\tmax.NaN.f32 %0, %1, t, u;\n\t}" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// The quantiser's bytes for one 16-byte vector of bf16, on the FMA pipe only: adding 1.5 * 2^23 rounds to the nearest
// integer (ties to even, as rintf does) and leaves that integer in the low mantissa bits, whose low byte is the
// two's-complement int8.  Where the product with the reciprocal lies close to a tie (see quant_round) the exact
// quotient decides: that path is a call, so that its division and rounding instructions stay out of the common path
// (inlined and predicated they kept the conversion pipe 86 % busy).
constexpr float QUANT_MAGIC = 12582912.f;

__device__ __noinline__ uint2 quant_vector_exact(uint4 raw, float scale) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float v = __uint_as_float((i & 1) ? (w[i >> 1] & 0xffff0000u) : (w[i >> 1] << 16));
    const float r = fminf(fmaxf(rintf(__fdiv_rn(v, scale)), -127.f), 127.f);
    out[i >> 2] |= (__float_as_uint(__fadd_rn(r, QUANT_MAGIC)) & 0xffu) << (8 * (i & 3));
  }
  return make_uint2(out[0], out[1]);
}

__device__ __forceinline__ uint2 quant_vector(uint4 raw, float scale, float inv) {
  // Two values per packed fp32 instruction: y = v * inv + MAGIC in one rounding (the integer nearest to the exact
  // product), -r = MAGIC - y, d = v * inv - r.  A product within 0.001 of a tie, or an integer outside [-127, 127]
  // (only the percentile bases produce those; the exact path clamps them), sends the vector to the exact path.
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
  const float2 inv2 = make_float2(inv, inv), magic2 = make_float2(QUANT_MAGIC, QUANT_MAGIC), minus2 = make_float2(-1.f, -1.f);
  uint32_t yb[8];
  float dmax = 0.f, rmax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v2 = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
    const float2 y2 = __ffma2_rn(v2, inv2, magic2);
    const float2 nr2 = __ffma2_rn(y2, minus2, magic2);
    const float2 d2 = __ffma2_rn(v2, inv2, nr2);
    dmax = max3_abs_nan(dmax, d2.x, d2.y);
    rmax = max3_abs_nan(rmax, nr2.x, nr2.y);
    yb[2 * i] = __float_as_uint(y2.x);
    yb[2 * i + 1] = __float_as_uint(y2.y);
  }
  if (!(dmax <= 0.499f) || !(rmax <= 127.f)) return quant_vector_exact(raw, scale);
  // the low byte of each y is the two's-complement int8
  const uint32_t lo = __byte_perm(__byte_perm(yb[0], yb[1], 0x0040), __byte_perm(yb[2], yb[3], 0x0040), 0x5410);
  const uint32_t hi = __byte_perm(__byte_perm(yb[4], yb[5], 0x0040), __byte_perm(yb[6], yb[7], 0x0040), 0x5410);
  return make_uint2(lo, hi);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(512) rope_relayout_kernel(const T* __restrict__ qkv, int B, int Tn, int H, int D,
                                                            const float* __restrict__ cos_t,
                                                            const float* __restrict__ sin_t, T* __restrict__ q,
                                                            T* __restrict__ k, T* __restrict__ v,
                                                            float* __restrict__ amax,
                                                            const uint8_t* __restrict__ q_keep, int nsec, int sec0) {
  // the source holds `nsec` sections per token, the first of them being section `sec0` of (q, k, v)
  constexpr int E = 16 / sizeof(T);  // elements per 16-byte vector: 8 bf16 or 4 fp32
  const int C = H * D;
  const int vec_per_tok = nsec * C / E;
  const int b = blockIdx.y;
  const int t0 = blockIdx.x * ROPE_TPB;
  const int t1 = min(Tn, t0 + ROPE_TPB);
  const int half = D / 2;
  // bf16: (cos, sin) of this CTA's tokens once, packed two bf16 to a word, instead of two conversions per word of data
  __shared__ __align__(16) uint32_t cs_s[sizeof(T) == 2 ? 2 * ROPE_TPB * ROPE_MAX_HALF : 1];   // (c, c) words, then (-s, s) words
  const bool packed = sizeof(T) == 2 && cos_t != nullptr && half <= ROPE_MAX_HALF && half % 4 == 0;
  if (packed) {
    for (int i = threadIdx.x; i < (t1 - t0) * half; i += blockDim.x) {
      const float c = cos_t[(int64_t)t0 * half + i], sn = sin_t[(int64_t)t0 * half + i];
      const __nv_bfloat162 wc = __floats2bfloat162_rn(c, c), ws = __floats2bfloat162_rn(-sn, sn);
      cs_s[i] = *reinterpret_cast<const uint32_t*>(&wc);
      cs_s[ROPE_TPB * ROPE_MAX_HALF + i] = *reinterpret_cast<const uint32_t*>(&ws);
    }
    __syncthreads();
  }
  for (int vi = threadIdx.x; vi < vec_per_tok; vi += blockDim.x) {
    const int ch = vi * E;
    const int sec = sec0 + ch / C;
    const int c_in = ch % C;
    const int h = c_in / D, d0 = c_in - h * D;
    const int bh = b * H + h;
    const bool rotate = sec < 2 && cos_t != nullptr;
    const T* src = qkv + ((int64_t)b * Tn + t0) * (nsec * (int64_t)C) + ch;
    T* dst = (sec == 0 ? q : (sec == 1 ? k : v)) + ((int64_t)bh * Tn + t0) * D + d0;
    const float* cr = cos_t ? cos_t + (int64_t)t0 * half + d0 / 2 : nullptr;
    const float* sr = sin_t ? sin_t + (int64_t)t0 * half + d0 / 2 : nullptr;
    float local_max = 0.f;
    __nv_bfloat162 local_max2 = __floats2bfloat162_rn(0.f, 0.f);
    float qscale = 1.f, qinv = 1.f;
    int8_t* dst8 = nullptr;
    if (MODE == 2) {
      qscale = fmaxf(__fdiv_rn(amax[sec * B * H + bh], 127.0f), 1e-6f);
      qinv = __fdiv_rn(1.0f, qscale);
      dst8 = reinterpret_cast<int8_t*>(sec == 0 ? q : (sec == 1 ? k : v)) + ((int64_t)bh * Tn + t0) * D + d0;
    }
    const uint8_t* keep = (sec == 0 && q_keep != nullptr) ? q_keep + (int64_t)b * Tn : nullptr;
    // Tokens in batches of eight: all loads of a batch are issued before the first of them is used, so that eight
    // 16-byte loads per thread are in flight (the plain loop left the stream latency-bound at 2.6 TB/s).
    constexpr int RB = MODE == 2 ? 4 : 8;
    const int64_t src_step = nsec * (int64_t)C;
    for (int tb = t0; tb < t1; tb += RB) {
      uint4 buf[RB];
      bool on[RB];
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        const int t = tb + u;
        // queries of dropped tokens are never read: neither load nor store them
        on[u] = t < t1 && (keep == nullptr || keep[t] != 0);
        if (on[u]) buf[u] = *reinterpret_cast<const uint4*>(src + u * src_step);
      }
#pragma unroll
      for (int u = 0; u < RB; ++u) {
        if (!on[u]) continue;
        const int t = tb + u;
        uint4 raw = buf[u];
        if (sizeof(T) == 2) {
          if (rotate) {
            if (packed) {
              const uint4 wc = *reinterpret_cast<const uint4*>(cs_s + (t - t0) * half + d0 / 2);
              const uint4 ws = *reinterpret_cast<const uint4*>(cs_s + ROPE_TPB * ROPE_MAX_HALF + (t - t0) * half + d0 / 2);
              raw.x = rope_word_bf16_packed(raw.x, wc.x, ws.x);
              raw.y = rope_word_bf16_packed(raw.y, wc.y, ws.y);
              raw.z = rope_word_bf16_packed(raw.z, wc.z, ws.z);
              raw.w = rope_word_bf16_packed(raw.w, wc.w, ws.w);
            } else {
              const float4 c4 = *reinterpret_cast<const float4*>(cr + u * half), s4 = *reinterpret_cast<const float4*>(sr + u * half);
              raw.x = rope_word_bf16(raw.x, c4.x, s4.x);
              raw.y = rope_word_bf16(raw.y, c4.y, s4.y);
              raw.z = rope_word_bf16(raw.z, c4.z, s4.z);
              raw.w = rope_word_bf16(raw.w, c4.w, s4.w);
            }
          }
          if (MODE != 2 && amax) {   // |x| and max on packed bf16 pairs: exact, no conversions
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
            local_max2 = __hmax2(__hmax2(local_max2, __habs2(h2[0])), __hmax2(__habs2(h2[1]), __hmax2(__habs2(h2[2]), __habs2(h2[3]))));
          }
          if (MODE == 2) *reinterpret_cast<uint2*>(dst8 + u * D) = quant_vector(raw, qscale, qinv);
        } else {
          float* f = reinterpret_cast<float*>(&raw);
          if (rotate) {
            const float2 c2 = *reinterpret_cast<const float2*>(cr + u * half), s2 = *reinterpret_cast<const float2*>(sr + u * half);
            const float e0 = f[0], o0 = f[1], e1 = f[2], o1 = f[3];
            f[0] = rope_mix(e0, c2.x, -o0, s2.x, false);
            f[1] = rope_mix(o0, c2.x, e0, s2.x, false);
            f[2] = rope_mix(e1, c2.y, -o1, s2.y, false);
            f[3] = rope_mix(o1, c2.y, e1, s2.y, false);
          }
          if (amax) local_max = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(local_max, fmaxf(fabsf(f[2]), fabsf(f[3]))));
        }
        if (MODE == 0) *reinterpret_cast<uint4*>(dst + u * D) = raw;
      }
      src += RB * src_step;
      dst += RB * D;
      if (MODE == 2) dst8 += RB * D;
      if (cr) { cr += RB * half; sr += RB * half; }
    }
    if (sizeof(T) == 2) {
      const float2 m2 = __bfloat1622float2(local_max2);
      local_max = fmaxf(m2.x, m2.y);
    }
    if (MODE != 2 && amax) {
      // lanes of a warp may belong to different (section, bh) groups: the lowest lane of every group folds in
      // its peers and issues one atomic (non-negative floats order like their bit patterns)
      const int key = sec * B * H + bh;
      const unsigned active = __activemask();
      const unsigned peers = __match_any_sync(active, key);
      const int leader = __ffs(peers) - 1;
      float gm = local_max;
      for (int l = 0; l < 32; ++l) {
        if (!((active >> l) & 1u)) continue;
        const float o = __shfl_sync(active, local_max, l);
        if ((peers >> l) & 1u) gm = fmaxf(gm, o);
      }
      if ((int)(threadIdx.x & 31) == leader) atomicMax(reinterpret_cast<int*>(amax + key), __float_as_int(gm));
    }
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
  const float inv = __fdiv_rn(1.0f, scale);
  if (blockIdx.x == 0 && threadIdx.x == 0) scales[head] = scale;
  const T* p = x + (int64_t)head * per_head;
  int8_t* o = out + (int64_t)head * per_head;
  const int64_t nvec = (per_head % 8 == 0) ? per_head / 8 : 0;  // vector path needs 16-byte aligned heads
  for (int64_t vi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += (int64_t)gridDim.x * blockDim.x) {
    if (sizeof(T) == 2) {
      reinterpret_cast<uint2*>(o)[vi] = quant_vector(reinterpret_cast<const uint4*>(p)[vi], scale, inv);
      continue;
    }
    float val[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) val[i] = ld_as_float<T>(p, vi * 8 + i);
    union { int8_t b[8]; uint2 u; } pk;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float r = quant_round(val[i], scale, inv);
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

// RoPE of compact query rows: row i of q_rows (H*D wide) belongs to token kept_idx[i]; it is rotated at that
// token's position and stored head-major.  One thread per 16-byte vector.
template <typename T>
__global__ void __launch_bounds__(256) rope_rows_q_kernel(const T* __restrict__ q_rows,
                                                          const int64_t* __restrict__ kept_idx,
                                                          const int32_t* __restrict__ count_dev, int64_t max_rows,
                                                          int64_t n_tok, int Tn, int H, int D,
                                                          const float* __restrict__ cos_t,
                                                          const float* __restrict__ sin_t, T* __restrict__ q) {
  constexpr int E = 16 / sizeof(T);
  const int C = H * D, half = D / 2;
  const int vec_per_row = C / E;
  const int64_t rows = count_dev ? min((int64_t)count_dev[0], max_rows) : max_rows;
  const int64_t total = rows * vec_per_row;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = g / vec_per_row;
    const int ch = (int)(g % vec_per_row) * E;
    const int64_t tok = kept_idx[r];
    if (tok < 0 || tok >= n_tok) continue;
    const int b = (int)(tok / Tn), t = (int)(tok % Tn);
    const int h = ch / D, d0 = ch % D;
    uint4 raw = *reinterpret_cast<const uint4*>(q_rows + r * C + ch);
    if (cos_t != nullptr) {
      const float* cr = cos_t + (int64_t)t * half + d0 / 2;
      const float* sr = sin_t + (int64_t)t * half + d0 / 2;
      if (sizeof(T) == 2) {
        const float4 c4 = *reinterpret_cast<const float4*>(cr), s4 = *reinterpret_cast<const float4*>(sr);
        raw.x = rope_word_bf16(raw.x, c4.x, s4.x);
        raw.y = rope_word_bf16(raw.y, c4.y, s4.y);
        raw.z = rope_word_bf16(raw.z, c4.z, s4.z);
        raw.w = rope_word_bf16(raw.w, c4.w, s4.w);
      } else {
        float* f = reinterpret_cast<float*>(&raw);
        const float2 c2 = *reinterpret_cast<const float2*>(cr), s2 = *reinterpret_cast<const float2*>(sr);
        const float e0 = f[0], o0 = f[1], e1 = f[2], o1 = f[3];
        f[0] = rope_mix(e0, c2.x, -o0, s2.x, false);
        f[1] = rope_mix(o0, c2.x, e0, s2.x, false);
        f[2] = rope_mix(e1, c2.y, -o1, s2.y, false);
        f[3] = rope_mix(o1, c2.y, e1, s2.y, false);
      }
    }
    *reinterpret_cast<uint4*>(q + (((int64_t)b * H + h) * Tn + t) * D + d0) = raw;
  }
}

// RoPE in place: row r (H*D wide, rows `row_stride` elements apart) is rotated at position r % Tn.
// With `heads_out` the rotated rows go there instead, head-major ((r / Tn) * H + h, r % Tn, D): the same bytes moved,
// and the keys of one head at consecutive positions become one contiguous run.
template <typename T>
__global__ void __launch_bounds__(256) rope_inplace_kernel(T* __restrict__ x, int64_t n_rows, int Tn,
                                                           int64_t row_stride, int H, int D,
                                                           const float* __restrict__ cos_t,
                                                           const float* __restrict__ sin_t, T* __restrict__ heads_out) {
  // One thread per (row, 16-byte vector of a head): it loads its cos/sin factors once and walks over the heads,
  // HB heads per step so that HB loads are in flight.  Consecutive threads take consecutive vectors of one head
  // (whole 128-byte lines for head_dim 64 in bf16).
  constexpr int E = 16 / sizeof(T);
  constexpr int HB = 8;
  const int half = D / 2, vec_per_head = D / E;
  const int64_t total = n_rows * vec_per_head;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = g / vec_per_head;
    const int d0 = (int)(g % vec_per_head) * E;
    const int t = (int)(r % Tn);
    const float* cr = cos_t + (int64_t)t * half + d0 / 2;
    const float* sr = sin_t + (int64_t)t * half + d0 / 2;
    float c[4], sn[4];
    if (sizeof(T) == 2) {
      const float4 c4 = *reinterpret_cast<const float4*>(cr), s4 = *reinterpret_cast<const float4*>(sr);
      c[0] = c4.x; c[1] = c4.y; c[2] = c4.z; c[3] = c4.w;
      sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
    } else {
      const float2 c2 = *reinterpret_cast<const float2*>(cr), s2 = *reinterpret_cast<const float2*>(sr);
      c[0] = c2.x; c[1] = c2.y; sn[0] = s2.x; sn[1] = s2.y;
      c[2] = c[3] = sn[2] = sn[3] = 0.f;
    }
    T* src = x + r * row_stride + d0;
    T* dst = heads_out ? heads_out + ((r / Tn) * H * (int64_t)Tn + t) * D + d0 : src;
    const int64_t dst_head = heads_out ? (int64_t)Tn * D : (int64_t)D;
    for (int h0 = 0; h0 < H; h0 += HB) {
      uint4 raw[HB];
#pragma unroll
      for (int i = 0; i < HB; ++i)
        if (h0 + i < H) raw[i] = *reinterpret_cast<const uint4*>(src + (int64_t)(h0 + i) * D);
#pragma unroll
      for (int i = 0; i < HB; ++i) {
        if (h0 + i >= H) break;
        if (sizeof(T) == 2) {
          raw[i].x = rope_word_bf16(raw[i].x, c[0], sn[0]);
          raw[i].y = rope_word_bf16(raw[i].y, c[1], sn[1]);
          raw[i].z = rope_word_bf16(raw[i].z, c[2], sn[2]);
          raw[i].w = rope_word_bf16(raw[i].w, c[3], sn[3]);
        } else {
          float* f = reinterpret_cast<float*>(&raw[i]);
          const float e0 = f[0], o0 = f[1], e1 = f[2], o1 = f[3];
          f[0] = rope_mix(e0, c[0], -o0, sn[0], false);
          f[1] = rope_mix(o0, c[0], e0, sn[0], false);
          f[2] = rope_mix(e1, c[1], -o1, sn[1], false);
          f[3] = rope_mix(o1, c[1], e1, sn[1], false);
        }
        *reinterpret_cast<uint4*>(dst + (int64_t)(h0 + i) * dst_head) = raw[i];
      }
    }
  }
}

// dst row i = src[slot_of[i]] for kept rows, `fill` (or zeros) for the others.  One warp per row at a time, lanes over
// the 16-byte vectors of the row: no index arithmetic per vector (a flat index cost two 64-bit divisions per 16 bytes
// stored and kept this store stream at 0.57 of the copy bandwidth).
__global__ void __launch_bounds__(256) scatter_rows_fill_kernel(const uint4* __restrict__ src,
                                                                const int32_t* __restrict__ slot_of,
                                                                const uint8_t* __restrict__ mask,
                                                                const uint4* __restrict__ fill, int64_t n,
                                                                int64_t vec_per_row, uint4* __restrict__ dst) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < n; r += warps) {
    const bool kept = mask[r] != 0;
    const uint4* from = kept ? src + (int64_t)slot_of[r] * vec_per_row : fill;
    uint4* to = dst + r * vec_per_row;
    for (int64_t c = lane; c < vec_per_row; c += 32) to[c] = from != nullptr ? from[c] : make_uint4(0u, 0u, 0u, 0u);
  }
}

__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src,
                                                          const int64_t* __restrict__ idx,
                                                          const int32_t* __restrict__ count_dev, int64_t max_rows,
                                                          int64_t vec_per_row, uint4* __restrict__ dst) {
  const int64_t rows = count_dev ? min((int64_t)count_dev[0], max_rows) : max_rows;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    const int64_t i = idx[r];
    const uint4* from = i >= 0 ? src + i * vec_per_row : nullptr;
    uint4* to = dst + r * vec_per_row;
    for (int64_t c = lane; c < vec_per_row; c += 32) to[c] = from != nullptr ? from[c] : make_uint4(0u, 0u, 0u, 0u);
  }
}

__global__ void scale_from_amax_kernel(const float* __restrict__ amax, int n, float* __restrict__ scales) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) scales[i] = fmaxf(__fdiv_rn(amax[i], 127.0f), 1e-6f);
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
                                  const float* sin_t, void* q, void* k, void* v, float* amax,
                                  const uint8_t* q_keep, void* stream) {
  ASPA_CHECK_ARG(qkv && q && k && v, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && H > 0 && D > 0 && D % 8 == 0, "head_dim must be a multiple of 8");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  ASPA_CHECK_ARG((cos_t == nullptr) == (sin_t == nullptr), "cos/sin tables come together");
  ASPA_CHECK_ARG(!(amax && q_keep), "per-head amax needs every query: do not combine it with q_keep");
  const dim3 grid((unsigned)ceil_div(T, ROPE_TPB), (unsigned)B);
  if (dtype == ASPA_BF16) {
    const int vec = 3 * H * D / 8;
    const int threads = (int)std::min<int64_t>(512, ceil_div(vec, 32) * 32);
    rope_relayout_kernel<__nv_bfloat16, 0><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)qkv, B, T, H, D, cos_t, sin_t, (__nv_bfloat16*)q, (__nv_bfloat16*)k, (__nv_bfloat16*)v, amax, q_keep, 3, 0);
  } else {
    const int vec = 3 * H * D / 4;
    const int threads = (int)std::min<int64_t>(512, ceil_div(vec, 32) * 32);
    rope_relayout_kernel<float, 0><<<grid, threads, 0, (cudaStream_t)stream>>>((const float*)qkv, B, T, H, D, cos_t, sin_t,
                                                                           (float*)q, (float*)k, (float*)v, amax, q_keep, 3, 0);
  }
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
  gather_rows_kernel<<<(unsigned)std::min<int64_t>(ceil_div(max_rows, 8), 148 * 16), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, idx, count_dev, max_rows, row_bytes / 16, (uint4*)dst);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_rope_relayout_kv(const void* kv, int dtype, int B, int T, int H, int D, const float* cos_t,
                                     const float* sin_t, void* k, void* v, void* stream) {
  ASPA_CHECK_ARG(kv && k && v, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && H > 0 && D > 0 && D % 2 == 0, "bad sizes");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  ASPA_CHECK_ARG(D % (dtype == ASPA_BF16 ? 8 : 4) == 0, "head_dim must fill 16-byte vectors");
  ASPA_CHECK_ARG((cos_t == nullptr) == (sin_t == nullptr), "cos/sin tables come together");
  const dim3 grid((unsigned)ceil_div(T, ROPE_TPB), (unsigned)B);
  if (dtype == ASPA_BF16) {
    const int vec = 2 * H * D / 8;
    const int threads = (int)std::min<int64_t>(512, ceil_div(vec, 32) * 32);
    rope_relayout_kernel<__nv_bfloat16, 0><<<grid, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)kv, B, T, H, D, cos_t, sin_t, nullptr, (__nv_bfloat16*)k, (__nv_bfloat16*)v, nullptr, nullptr, 2, 1);
  } else {
    const int vec = 2 * H * D / 4;
    const int threads = (int)std::min<int64_t>(512, ceil_div(vec, 32) * 32);
    rope_relayout_kernel<float, 0><<<grid, threads, 0, (cudaStream_t)stream>>>((const float*)kv, B, T, H, D, cos_t, sin_t, nullptr,
                                                                           (float*)k, (float*)v, nullptr, nullptr, 2, 1);
  }
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_rope_rows_q(const void* q_rows, int dtype, const int64_t* kept_idx, const int32_t* count_dev,
                                int64_t max_rows, int B, int T, int H, int D, const float* cos_t, const float* sin_t,
                                void* q, void* stream) {
  ASPA_CHECK_ARG(q_rows && kept_idx && q, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && H > 0 && D > 0 && D % 2 == 0 && max_rows >= 0, "bad sizes");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  ASPA_CHECK_ARG(D % (dtype == ASPA_BF16 ? 8 : 4) == 0, "head_dim must fill 16-byte vectors");
  ASPA_CHECK_ARG((cos_t == nullptr) == (sin_t == nullptr), "cos/sin tables come together");
  if (max_rows == 0) return ASPA_OK;
  const int64_t total = max_rows * (H * D / (dtype == ASPA_BF16 ? 8 : 4));
  const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(total, 256), 148 * 16);
  if (dtype == ASPA_BF16)
    rope_rows_q_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q_rows, kept_idx, count_dev, max_rows, (int64_t)B * T, T, H, D, cos_t, sin_t, (__nv_bfloat16*)q);
  else
    rope_rows_q_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((const float*)q_rows, kept_idx, count_dev, max_rows,
                                                                        (int64_t)B * T, T, H, D, cos_t, sin_t, (float*)q);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_scatter_rows_fill(const void* src, const int32_t* slot_of, const uint8_t* mask, const void* fill,
                                      int64_t n, int64_t row_bytes, void* dst, void* stream) {
  ASPA_CHECK_ARG(src && slot_of && mask && dst, "null pointer");
  ASPA_CHECK_ARG(n >= 0 && row_bytes > 0 && row_bytes % 16 == 0, "row_bytes must be a multiple of 16");
  if (n == 0) return ASPA_OK;
  scatter_rows_fill_kernel<<<(unsigned)std::min<int64_t>(ceil_div(n, 8), 148 * 32), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, slot_of, mask, (const uint4*)fill, n, row_bytes / 16, (uint4*)dst);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_rope_inplace(void* x, int dtype, int64_t n_rows, int T, int64_t row_stride, int H, int D,
                                 const float* cos_t, const float* sin_t, void* stream) {
  return aspa_rope_rows_to_heads(x, dtype, n_rows, T, row_stride, H, D, cos_t, sin_t, nullptr, stream);
}

extern "C" int aspa_rope_rows_to_heads(void* x, int dtype, int64_t n_rows, int T, int64_t row_stride, int H, int D,
                                       const float* cos_t, const float* sin_t, void* heads_out, void* stream) {
  ASPA_CHECK_ARG(x && cos_t && sin_t, "null pointer");
  ASPA_CHECK_ARG(heads_out == nullptr || n_rows % T == 0, "head-major output needs whole sequences");
  ASPA_CHECK_ARG(n_rows >= 0 && T > 0 && H > 0 && D > 0 && D % 2 == 0 && row_stride >= (int64_t)H * D, "bad sizes");
  ASPA_CHECK_ARG(dtype == ASPA_F32 || dtype == ASPA_BF16, "dtype must be fp32 or bf16");
  const int E = dtype == ASPA_BF16 ? 8 : 4;
  ASPA_CHECK_ARG(D % E == 0 && row_stride % E == 0, "rows must start on 16-byte boundaries");
  if (n_rows == 0) return ASPA_OK;
  const int64_t total = n_rows * (D / E);
  const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(total, 256), 148 * 8);
  if (dtype == ASPA_BF16)
    rope_inplace_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, n_rows, T, row_stride, H, D,
                                                                                 cos_t, sin_t, (__nv_bfloat16*)heads_out);
  else
    rope_inplace_kernel<float><<<blocks, 256, 0, (cudaStream_t)stream>>>((float*)x, n_rows, T, row_stride, H, D, cos_t, sin_t,
                                                                (float*)heads_out);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}

extern "C" int aspa_rope_quantize(const void* qkv, int B, int T, int H, int D, const float* cos_t, const float* sin_t,
                                  int8_t* q8, int8_t* k8, int8_t* v8, float* amax, float* scales, void* stream) {
  ASPA_CHECK_ARG(qkv && q8 && k8 && v8 && amax && scales, "null pointer");
  ASPA_CHECK_ARG(B > 0 && T > 0 && H > 0 && D > 0 && D % 8 == 0, "bad sizes (head_dim must be a multiple of 8)");
  ASPA_CHECK_ARG((cos_t == nullptr) == (sin_t == nullptr), "cos/sin tables come together");
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid((unsigned)ceil_div(T, ROPE_TPB), (unsigned)B);
  const int vec = 3 * H * D / 8;
  const int threads = (int)std::min<int64_t>(512, ceil_div(vec, 32) * 32);
  cudaMemsetAsync(amax, 0, sizeof(float) * 3 * B * H, st);
  const __nv_bfloat16* src = (const __nv_bfloat16*)qkv;
  rope_relayout_kernel<__nv_bfloat16, 1><<<grid, threads, 0, st>>>(src, B, T, H, D, cos_t, sin_t, nullptr, nullptr, nullptr,
                                                                   amax, nullptr, 3, 0);
  ASPA_CHECK_LAUNCH();
  rope_relayout_kernel<__nv_bfloat16, 2><<<grid, threads, 0, st>>>(
      src, B, T, H, D, cos_t, sin_t, reinterpret_cast<__nv_bfloat16*>(q8), reinterpret_cast<__nv_bfloat16*>(k8),
      reinterpret_cast<__nv_bfloat16*>(v8), amax, nullptr, 3, 0);
  ASPA_CHECK_LAUNCH();
  // scales = max(amax / 127, 1e-6), the formula of the quantiser
  scale_from_amax_kernel<<<(unsigned)ceil_div(3 * B * H, 256), 256, 0, st>>>(amax, 3 * B * H, scales);
  ASPA_CHECK_LAUNCH();
  return ASPA_OK;
}
