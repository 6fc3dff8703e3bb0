// Per-token router epilogue shared by the CUDA-core and the tensor-core router kernels.
#pragma once

#include "common.cuh"

namespace aspa {

// Per-token epilogue shared by both router kernels.  `row` points at 2G floats in shared memory:
// [0,G) router logits (fp32 accumulators), [G,2G) raw dot products with the normalised prototypes.
// Each arithmetic step is rounded separately (no fused multiply-add) because the reference
// evaluates it as a chain of separate tensor ops.
__device__ __forceinline__ void router_epilogue(float* row, int stride, int G, bool bf16_act, bool has_proto,
                                                float nsq, const float* conf_eps, const float* usage_bias,
                                                float proto_temp, float proto_threshold, float proto_span,
                                                float proto_blend, float usage_boost, float* gate_out, float* imp_out,
                                                float* sim_out, float* blend_out, float* st_sim, float* st_bs) {
  float m = -INFINITY;
  for (int g = 0; g < G; ++g) {
    float l = row[g * stride];
    if (bf16_act) l = bf16_round(l);
    row[g * stride] = l;
    m = fmaxf(m, l);
  }
  float s = 0.f;
  for (int g = 0; g < G; ++g) {
    float e = expf(row[g * stride] - m);
    row[g * stride] = e;
    s += e;
  }
  for (int g = 0; g < G; ++g) {
    float p = __fdiv_rn(row[g * stride], s);
    row[g * stride] = bf16_act ? bf16_round(p) : p;
  }
  float sim = 0.f, bs = 0.f;
  if (has_proto) {
    const float denom = fmaxf(sqrtf(nsq), 1e-6f);
    float zmax = -INFINITY;
    sim = -INFINITY;
    for (int g = 0; g < G; ++g) {
      float sg = __fdiv_rn(row[(G + g) * stride], denom);
      sim = fmaxf(sim, sg);
      float z = __fdiv_rn(sg, proto_temp);
      row[(G + g) * stride] = z;
      zmax = fmaxf(zmax, z);
    }
    float zs = 0.f;
    for (int g = 0; g < G; ++g) {
      float e = expf(row[(G + g) * stride] - zmax);
      row[(G + g) * stride] = e;
      zs += e;
    }
    float tot = 0.f;
    for (int g = 0; g < G; ++g) {
      float pp = __fdiv_rn(row[(G + g) * stride], zs);
      if (conf_eps) pp = __fmul_rn(pp, conf_eps[g]);
      row[(G + g) * stride] = pp;
      tot += pp;
    }
    if (conf_eps) {
      tot = fmaxf(tot, 1e-6f);
      for (int g = 0; g < G; ++g) row[(G + g) * stride] = __fdiv_rn(row[(G + g) * stride], tot);
    }
    bs = __fdiv_rn(__fsub_rn(sim, proto_threshold), proto_span);
    bs = fminf(fmaxf(bs, 0.f), 1.f);
    const float blend = __fmul_rn(proto_blend, bs);
    const float keep = __fsub_rn(1.0f, blend);
    float gs = 0.f;
    for (int g = 0; g < G; ++g) {
      float v = __fadd_rn(__fmul_rn(row[g * stride], keep), __fmul_rn(row[(G + g) * stride], blend));
      if (usage_bias) v = __fadd_rn(v, __fmul_rn(usage_bias[g], __fmul_rn(__fsub_rn(1.0f, bs), usage_boost)));
      v = fmaxf(v, 0.f);
      row[g * stride] = v;
      gs += v;
    }
    gs = fmaxf(gs, 1e-6f);
    for (int g = 0; g < G; ++g) row[g * stride] = __fdiv_rn(row[g * stride], gs);
  }
  float gmax = -INFINITY;
  for (int g = 0; g < G; ++g) {
    float v = row[g * stride];
    gate_out[g] = v;
    gmax = fmaxf(gmax, v);
  }
  float imp = gmax;
  if (has_proto) {
    imp = __fadd_rn(__fmul_rn(gmax, __fsub_rn(1.0f, bs)), __fmul_rn(sim, bs));
    if (sim_out) *sim_out = sim;
    if (blend_out) *blend_out = bs;
  }
  *imp_out = imp;
  *st_sim = sim;
  *st_bs = bs;
}

// The same epilogue with the row held in registers (G known at compile time, every loop unrolled): the independent
// exponentials and divisions of a row overlap instead of queueing behind shared-memory round trips.  Operation order
// and rounding are those of router_epilogue, so both produce the same bits.
//   lg[g]: router logits (fp32 accumulators); pd[g]: raw dot products with the normalised prototypes.
template <int GT>
__device__ __forceinline__ void router_epilogue_regs(float (&lg)[GT], float (&pd)[GT], bool bf16_act, bool has_proto,
                                                     float nsq, const float* conf_eps, const float* usage_bias,
                                                     float proto_temp, float proto_threshold, float proto_span,
                                                     float proto_blend, float usage_boost, float* gate_out,
                                                     float* imp_out, float* sim_out, float* blend_out, float* st_sim,
                                                     float* st_bs) {
  float m = -INFINITY;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (bf16_act) lg[g] = bf16_round(lg[g]);
    m = fmaxf(m, lg[g]);
  }
  float s = 0.f;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    lg[g] = expf(lg[g] - m);
    s += lg[g];
  }
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const float p = __fdiv_rn(lg[g], s);
    lg[g] = bf16_act ? bf16_round(p) : p;
  }
  float sim = 0.f, bs = 0.f;
  if (has_proto) {
    const float denom = fmaxf(sqrtf(nsq), 1e-6f);
    float zmax = -INFINITY;
    sim = -INFINITY;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      const float sg = __fdiv_rn(pd[g], denom);
      sim = fmaxf(sim, sg);
      pd[g] = __fdiv_rn(sg, proto_temp);
      zmax = fmaxf(zmax, pd[g]);
    }
    float zs = 0.f;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      pd[g] = expf(pd[g] - zmax);
      zs += pd[g];
    }
    float tot = 0.f;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float pp = __fdiv_rn(pd[g], zs);
      if (conf_eps) pp = __fmul_rn(pp, conf_eps[g]);
      pd[g] = pp;
      tot += pp;
    }
    if (conf_eps) {
      tot = fmaxf(tot, 1e-6f);
#pragma unroll
      for (int g = 0; g < GT; ++g) pd[g] = __fdiv_rn(pd[g], tot);
    }
    bs = __fdiv_rn(__fsub_rn(sim, proto_threshold), proto_span);
    bs = fminf(fmaxf(bs, 0.f), 1.f);
    const float blend = __fmul_rn(proto_blend, bs);
    const float keep = __fsub_rn(1.0f, blend);
    float gs = 0.f;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float v = __fadd_rn(__fmul_rn(lg[g], keep), __fmul_rn(pd[g], blend));
      if (usage_bias) v = __fadd_rn(v, __fmul_rn(usage_bias[g], __fmul_rn(__fsub_rn(1.0f, bs), usage_boost)));
      v = fmaxf(v, 0.f);
      lg[g] = v;
      gs += v;
    }
    gs = fmaxf(gs, 1e-6f);
#pragma unroll
    for (int g = 0; g < GT; ++g) lg[g] = __fdiv_rn(lg[g], gs);
  }
  float gmax = -INFINITY;
#pragma unroll
  for (int g = 0; g < GT; g += 4) {
    *reinterpret_cast<float4*>(gate_out + g) = make_float4(lg[g], lg[g + 1], lg[g + 2], lg[g + 3]);
    gmax = fmaxf(fmaxf(gmax, fmaxf(lg[g], lg[g + 1])), fmaxf(lg[g + 2], lg[g + 3]));
  }
  float imp = gmax;
  if (has_proto) {
    imp = __fadd_rn(__fmul_rn(gmax, __fsub_rn(1.0f, bs)), __fmul_rn(sim, bs));
    if (sim_out) *sim_out = sim;
    if (blend_out) *blend_out = bs;
  }
  *imp_out = imp;
  *st_sim = sim;
  *st_bs = bs;
}

}  // namespace aspa
