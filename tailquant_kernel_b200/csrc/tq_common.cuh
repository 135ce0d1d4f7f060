// Shared device helpers for the split W4A4 + tail kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tailquant.h"

namespace tq {

// ---------------------------------------------------------------------------- host side
void set_last_cuda_error(cudaError_t e);
void set_last_error_text(const char* s);  // message for failures that have no cudaError_t (driver entry points)
int check_launch();  // cudaGetLastError -> TQ_OK / TQ_ERR_CUDA

int run_prologue(const void* x, int M, int K, int had_kind, int R, int dr, float eps, int scale_mode,
                 uint8_t* a_pack, int8_t* a_q8, float* body_scale, float* top_scale, uint16_t* tail_idx16,
                 void* tail_val, int tail_ld, uint16_t* tail_ptr, int ptr_ld, uint32_t* tail_rec, uint16_t* tail_cnt,
                 int32_t* idx32, int8_t* top_q, void* x_rot, const void* gamma, float rms_eps, cudaStream_t st,
                 int dtype = TQ_BF16, void* tail_dense = nullptr);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------- bf16 bits
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits) { return __uint_as_float(bits << 16); }

__device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
}

// SwiGLU of one (gate, up) pair the way a bf16 framework evaluates it on the two linears' bf16 outputs
// (the reference computes act(gate) * up in PyTorch: tools/bench_prefill_bf16_romeoquarotdense_split_total_v61_sharedprepare.py:214):
// both inputs rounded to bf16, silu(g) = g / (1 + exp(-g)) in fp32 rounded to bf16, product rounded to bf16.
__device__ __forceinline__ uint32_t swiglu_bf16_bits(float g, float u) {
  g = bf16_bits_to_f32(f32_to_bf16_bits(g));
  u = bf16_bits_to_f32(f32_to_bf16_bits(u));
  const float s = bf16_bits_to_f32(f32_to_bf16_bits(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g)))));
  return f32_to_bf16_bits(__fmul_rn(s, u));
}

// clamp(rint(x / scale), -8, 7) with true fp32 division semantics.  t = x * fl(1 / scale) differs from the
// correctly rounded quotient by less than 3 ulp, i.e. by less than 2e-6 for |t| < 16 (and beyond 8.5 both
// evaluations clamp to the same side), so it decides every case that is not within 1e-5 of a rounding boundary;
// those cases (4 in 100000) take the IEEE division.
__device__ __forceinline__ int quant_s4(float x, float scale, float rinv) {
  float t = x * rinv;
  float r = rintf(t);
  if (fabsf(fabsf(t - r) - 0.5f) < 1e-5f) r = rintf(__fdiv_rn(x, scale));
  r = fminf(fmaxf(r, -8.0f), 7.0f);
  return (int)r;
}

// ---------------------------------------------------------------------------- vector loads
__device__ __forceinline__ uint4 ldg_nc_128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

}  // namespace tq
