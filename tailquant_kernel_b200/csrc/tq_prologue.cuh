// Types and small helpers shared by the two prologue kernels (tq_prologue.cu, tq_prologue_fast.cu).
#pragma once

#include "tq_common.cuh"

namespace tq {
namespace {

// 12x12 Paley-I Hadamard over GF(11): bit j of row a2 set <=> H[a2][j] = -1.
__device__ constexpr unsigned short H12_NEG[12] = {0x000, 0x475, 0x8e9, 0x1d3, 0x3a5, 0x749,
                                                   0xe91, 0xd23, 0xa47, 0x48f, 0x91d, 0x23b};

struct PrologueParams {
  const __nv_bfloat16* x;
  int M, R, dr, tail_ld, ptr_ld;
  float eps, hscale;
  int scale_mode;  // 0: max(t, eps) / 7 (activations); 1: max(t / 7, eps) (weights)
  uint8_t* a_pack;
  int8_t* a_q8;
  float* body_scale;
  float* top_scale;
  uint16_t* tail_idx16;
  uint16_t* tail_val;
  uint16_t* tail_ptr;  // [M, ptr_ld]: entries with index < 128 * j, j = 0 .. K/128
  uint32_t* tail_rec;  // [2 ceil(M/256)][K/64][128][TQ_TAIL_REC_CAP]: tile position | bf16 << 16
  uint16_t* tail_cnt;  // [2 ceil(M/256)][K/64][128]: entries per 64-wide half slice
  int32_t* idx32;
  int8_t* top_q;
  uint16_t* x_rot;
  uint16_t* tail_dense;   // [M, K] bf16: the rotated row with every element outside the tail set to zero (R > 0), or NULL
  const uint16_t* gamma;  // [K] bf16 RMSNorm weight, or NULL: x is used as it is
  float rms_eps;
};

__device__ __forceinline__ float make_scale(float t, float eps, int mode) {
  return mode == 0 ? __fdiv_rn(fmaxf(t, eps), 7.0f) : fmaxf(__fdiv_rn(t, 7.0f), eps);
}

}  // namespace

// Kernel of tq_prologue_fast.cu for the (rotation, K, dtype) combinations it is built for; TQ_ERR_UNSUPPORTED
// otherwise (the caller then runs the general kernel).
int run_prologue_fast(int kind, int K, int dtype, const PrologueParams& p, cudaStream_t st);

}  // namespace tq
