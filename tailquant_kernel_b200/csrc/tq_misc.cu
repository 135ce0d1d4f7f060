// Small kernels around the hot path: weight re-layouts (offline), the split-K finisher and the
// reference-compatible INT4-tail ("T4") epilogues.
#include "tq_common.cuh"

namespace tq {
namespace {

// ------------------------------------------------------------------ [N,K] bf16 -> [K,N] bf16
__global__ void transpose_bf16_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int N, int K) {
  __shared__ uint16_t tile[64][66];
  const int k0 = blockIdx.x * 64, n0 = blockIdx.y * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int n = n0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const int k = k0 + j;
      tile[i][j] = (n < N && k < K) ? in[(size_t)n * K + k] : (uint16_t)0;
    }
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int k = k0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const int n = n0 + j;
      if (n < N && k < K) out[(size_t)k * N + n] = tile[j][i];
    }
  }
}

// ------------------------------------------------------------------ b_col [N,K/2] -> b_row [K,N/2]
// low nibble of b_row[k][n/2] = code (n even), high nibble = code (n odd)
// (layout read by tools/fused_sparse_epilogue_ext_v58.py:63-71).
__global__ void col_to_row_s4_kernel(const uint8_t* __restrict__ b_col, uint8_t* __restrict__ b_row, int N, int K) {
  const int n2 = blockIdx.x * blockDim.x + threadIdx.x;  // pair of output channels
  const int k2 = blockIdx.y;                             // pair of input channels
  if (n2 >= N / 2) return;
  const uint8_t a = b_col[(size_t)(2 * n2) * (K / 2) + k2];      // codes (n, 2k2), (n, 2k2+1)
  const uint8_t b = b_col[(size_t)(2 * n2 + 1) * (K / 2) + k2];  // codes (n+1, ..)
  b_row[(size_t)(2 * k2) * (N / 2) + n2] = (uint8_t)((a & 0x0f) | ((b & 0x0f) << 4));
  b_row[(size_t)(2 * k2 + 1) * (N / 2) + n2] = (uint8_t)((a >> 4) | (b & 0xf0));
}

// ------------------------------------------------------------------ split-K finisher
__global__ void dequant_finish_kernel(const int32_t* __restrict__ C, const float* __restrict__ sx,
                                      const float* __restrict__ sw, const float* __restrict__ tail,
                                      const float* __restrict__ bias, uint16_t* __restrict__ out, int M, int N) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  float d = __fmul_rn(__fmul_rn((float)C[i], sx[m]), sw[n]);
  if (tail) d = __fadd_rn(d, tail[i]);
  if (bias) d = __fadd_rn(d, bias[n]);
  out[i] = (uint16_t)f32_to_bf16_bits(d);
}

// the same with the accumulators still split over `splits` K ranges ([splits, M, N]): summed here, exactly.
// act = 1: SwiGLU over interleaved (gate, up) channel pairs, out [M, N/2]; one thread per output either way.
__global__ void dequant_finish_partials_kernel(const int32_t* __restrict__ P, int splits, const float* __restrict__ sx,
                                               const float* __restrict__ sw, const float* __restrict__ tail,
                                               const float* __restrict__ bias, uint16_t* __restrict__ out, int M, int N,
                                               int act) {
  const size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)M * N;
  const int per = act ? 2 : 1;  // accumulators per output
  if (o * per >= total) return;
  float d[2];
  for (int e = 0; e < per; ++e) {
    const size_t i = o * per + e;
    const int m = (int)(i / N), n = (int)(i % N);
    int acc = 0;
    for (int s = 0; s < splits; ++s) acc += P[(size_t)s * total + i];
    float v = __fmul_rn(__fmul_rn((float)acc, sx[m]), sw[n]);
    if (tail) v = __fadd_rn(v, tail[i]);
    if (bias) v = __fadd_rn(v, bias[n]);
    d[e] = v;
  }
  out[o] = (uint16_t)(act ? swiglu_bf16_bits(d[0], d[1]) : f32_to_bf16_bits(d[0]));
}

// ------------------------------------------------------------------ T4 sparse term
__device__ __forceinline__ int s4(uint32_t nib) { return (int)((nib & 0xfu) ^ 8u) - 8; }

template <typename IdxT>
__device__ __forceinline__ void sparse_sum8(const int8_t* __restrict__ tq_row, const IdxT* __restrict__ idx_row,
                                            const uint8_t* __restrict__ b_row, int R, int N, int n0, int (&acc)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0;
  for (int r = 0; r < R; ++r) {
    const int k = (int)idx_row[r];
    const int a = (int)tq_row[r];
    const uint32_t w = *reinterpret_cast<const uint32_t*>(b_row + ((size_t)k * N + n0) / 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += a * s4(w >> (4 * i));
  }
}

__device__ __forceinline__ void store16(void* out, size_t i, float v, int dtype) {
  if (dtype == TQ_BF16)
    reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
}
__device__ __forceinline__ float load16(const void* p, size_t i, int dtype) {
  return dtype == TQ_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                          : __half2float(reinterpret_cast<const __half*>(p)[i]);
}

// mode 0: out = f16(float(C)*bs*ws + float(sum)*ts*ws)      (tools/fused_sparse_epilogue_ext_v58.py:76-86)
// mode 1: out = f16(float(out) + float(sum)*ts*ws)          (tools/sparse_correction_add_ext_v1.py:64-123)
// mode 2: out = f16(float(sum)*ts*ws)                       (tools/split_sparse_idx16_ext_v1.py:50-109)
template <typename IdxT>
__global__ void t4_epilogue_kernel(int mode, const int32_t* __restrict__ C, const float* __restrict__ bs,
                                   const int8_t* __restrict__ top_q, const IdxT* __restrict__ idx,
                                   const uint8_t* __restrict__ b_row, const float* __restrict__ ts,
                                   const void* __restrict__ ws, int ws_bf16, void* out, int out_dtype, int M, int N,
                                   int R) {
  const int m = blockIdx.y;
  const int n0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (m >= M || n0 >= N) return;
  int acc[8];
  sparse_sum8<IdxT>(top_q + (size_t)m * R, idx + (size_t)m * R, b_row, R, N, n0, acc);
  const float tsm = ts[m];
  const float bsm = (mode == 0) ? bs[m] : 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const size_t o = (size_t)m * N + n0 + i;
    const float w = ws_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ws)[n0 + i])
                            : reinterpret_cast<const float*>(ws)[n0 + i];
    const float sparse = __fmul_rn(__fmul_rn((float)acc[i], tsm), w);
    float v = sparse;
    if (mode == 0) v = __fadd_rn(__fmul_rn(__fmul_rn((float)C[o], bsm), w), sparse);
    if (mode == 1) v = __fadd_rn(load16(out, o, out_dtype), sparse);
    store16(out, o, v, out_dtype);
  }
}

__global__ void idx_i32_to_u16_kernel(const int32_t* __restrict__ in, uint16_t* __restrict__ out, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = (uint16_t)in[i];
}

int t4_launch(int mode, const int32_t* C, const float* bs, const int8_t* top_q, const void* idx, int idx_u16,
              const uint8_t* b_row, const float* ts, const void* ws, int ws_bf16, void* out, int out_dtype, int M,
              int N, int K, int R, cudaStream_t st) {
  if (!top_q || !idx || !b_row || !ts || !ws || !out || M < 0 || N <= 0 || K <= 0 || R <= 0) return TQ_ERR_BAD_ARG;
  if (mode == 0 && (!C || !bs)) return TQ_ERR_BAD_ARG;
  if (N % 8 != 0) return TQ_ERR_UNSUPPORTED;
  if (out_dtype != TQ_BF16 && out_dtype != TQ_FP16) return TQ_ERR_BAD_ARG;
  if (M == 0) return TQ_OK;
  dim3 block(128), grid((N / 8 + 127) / 128, M);
  if (idx_u16)
    t4_epilogue_kernel<uint16_t><<<grid, block, 0, st>>>(mode, C, bs, top_q, reinterpret_cast<const uint16_t*>(idx),
                                                         b_row, ts, ws, ws_bf16, out, out_dtype, M, N, R);
  else
    t4_epilogue_kernel<int32_t><<<grid, block, 0, st>>>(mode, C, bs, top_q, reinterpret_cast<const int32_t*>(idx),
                                                        b_row, ts, ws, ws_bf16, out, out_dtype, M, N, R);
  return check_launch();
}

}  // namespace

int run_transpose_bf16(const void* in, void* out, int N, int K, cudaStream_t st) {
  dim3 block(32, 8), grid((K + 63) / 64, (N + 63) / 64);
  transpose_bf16_kernel<<<grid, block, 0, st>>>(reinterpret_cast<const uint16_t*>(in),
                                                reinterpret_cast<uint16_t*>(out), N, K);
  return check_launch();
}

int run_col_to_row_s4(const uint8_t* b_col, uint8_t* b_row, int N, int K, cudaStream_t st) {
  dim3 block(128), grid((N / 2 + 127) / 128, K / 2);
  col_to_row_s4_kernel<<<grid, block, 0, st>>>(b_col, b_row, N, K);
  return check_launch();
}

}  // namespace tq

extern "C" int tq_dequant_finish(const int32_t* C, const float* body_scale, const float* w_scale, const float* tail,
                                 const float* bias, void* out_bf16, int M, int N, void* stream) {
  if (!C || !body_scale || !w_scale || !out_bf16 || M < 0 || N <= 0) return TQ_ERR_BAD_ARG;
  if (M == 0) return TQ_OK;
  const size_t total = (size_t)M * N;
  tq::dequant_finish_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      C, body_scale, w_scale, tail, bias, reinterpret_cast<uint16_t*>(out_bf16), M, N);
  return tq::check_launch();
}

extern "C" int tq_dequant_finish_partials(const int32_t* partials, int splits, const float* body_scale,
                                          const float* w_scale, const float* tail, const float* bias, void* out_bf16,
                                          int M, int N, int act, void* stream) {
  if (!partials || splits < 1 || !body_scale || !w_scale || !out_bf16 || M < 0 || N <= 0 || act < 0 || act > 1)
    return TQ_ERR_BAD_ARG;
  if (act && (N & 1)) return TQ_ERR_UNSUPPORTED;
  if (M == 0) return TQ_OK;
  const size_t outputs = (size_t)M * N / (act ? 2 : 1);
  tq::dequant_finish_partials_kernel<<<(unsigned)((outputs + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      partials, splits, body_scale, w_scale, tail, bias, reinterpret_cast<uint16_t*>(out_bf16), M, N, act);
  return tq::check_launch();
}

extern "C" int tq_scale_sparse_epilogue(const int32_t* C, const float* body_scale, const int8_t* top_q,
                                        const int32_t* idx, const uint8_t* b_row, const float* top_scale,
                                        const float* w_scale, void* out, int out_dtype, int M, int N, int K, int R,
                                        void* stream) {
  return tq::t4_launch(0, C, body_scale, top_q, idx, 0, b_row, top_scale, w_scale, 0, out, out_dtype, M, N, K, R,
                       (cudaStream_t)stream);
}

extern "C" int tq_sparse_correction_add(void* out, int out_dtype, const int8_t* top_q, const int32_t* idx,
                                        const uint8_t* b_row, const float* top_scale, const void* w_scale,
                                        int w_scale_bf16, int M, int N, int K, int R, void* stream) {
  return tq::t4_launch(1, nullptr, nullptr, top_q, idx, 0, b_row, top_scale, w_scale, w_scale_bf16, out, out_dtype, M,
                       N, K, R, (cudaStream_t)stream);
}

extern "C" int tq_sparse_top_write(void* out, int out_dtype, const int8_t* top_q, const void* idx, int idx_u16,
                                   const uint8_t* b_row, const float* top_scale, const float* w_scale, int M, int N,
                                   int K, int R, void* stream) {
  return tq::t4_launch(2, nullptr, nullptr, top_q, idx, idx_u16, b_row, top_scale, w_scale, 0, out, out_dtype, M, N, K,
                       R, (cudaStream_t)stream);
}

extern "C" int tq_idx_i32_to_u16(const int32_t* idx, uint16_t* out, long long n, void* stream) {
  if (!idx || !out || n < 0) return TQ_ERR_BAD_ARG;
  if (n == 0) return TQ_OK;
  tq::idx_i32_to_u16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(idx, out, n);
  return tq::check_launch();
}
