// 16-bit activation planes: how GEMM inputs are stored between kernels.
//
// The tensor-core GEMM multiplies fp16 operands.  To keep f32-class accuracy an
// activation x is held as two fp16 planes, hi = fp16(x) and
// lo = fp16((x - hi) * 2^11), so x ~= hi + lo * 2^-11 with about 22 significant
// bits; the GEMM runs both planes through one MMA and recombines in f32.
// Scaling the residual by 2^11 keeps it in fp16's normal range.  A
// configuration that asks for rounded activations stores one plane only.
#pragma once
#include "common.cuh"

namespace logos {

constexpr int LOGOS_ACT_PLANES = 100;  // c_dtype value: write through an ActOut

struct ActOut {
  __half* hi = nullptr;
  __half* lo = nullptr;   // written only in LOGOS_F32 mode
  int     mode = LOGOS_F32;  // LOGOS_F32: two planes; LOGOS_F16 / LOGOS_BF16: rounded, one plane
};

__device__ __forceinline__ float act_clamp(float x) { return fminf(fmaxf(x, -65504.f), 65504.f); }

__device__ __forceinline__ void act_store(const ActOut& o, int64_t i, float x) {
  if (o.mode == LOGOS_BF16) x = __bfloat162float(__float2bfloat16_rn(x));
  x = act_clamp(x);
  __half h = __float2half_rn(x);
  o.hi[i] = h;
  if (o.mode == LOGOS_F32) o.lo[i] = __float2half_rn((x - __half2float(h)) * 2048.f);
}

__device__ __forceinline__ float act_load(const __half* hi, const __half* lo, int64_t i) {
  float v = __half2float(hi[i]);
  if (lo) v = fmaf(__half2float(lo[i]), 4.8828125e-4f, v);
  return v;
}

}  // namespace logos
