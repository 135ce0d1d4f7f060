// Host-side glue of the C ABI: error reporting and offline weight preparation.
#include "tq_common.cuh"

namespace tq {

static thread_local char g_cuda_error[256] = "";

void set_last_cuda_error(cudaError_t e) {
  const char* s = cudaGetErrorString(e);
  int i = 0;
  for (; s && s[i] && i < 255; ++i) g_cuda_error[i] = s[i];
  g_cuda_error[i] = 0;
}

void set_last_error_text(const char* s) {
  int i = 0;
  for (; s && s[i] && i < 255; ++i) g_cuda_error[i] = s[i];
  g_cuda_error[i] = 0;
}

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return TQ_OK;
  set_last_cuda_error(e);
  return TQ_ERR_CUDA;
}

int run_transpose_bf16(const void* in, void* out, int N, int K, cudaStream_t st);
int run_col_to_row_s4(const uint8_t* b_col, uint8_t* b_row, int N, int K, cudaStream_t st);

}  // namespace tq

extern "C" int tq_version(void) { return 100; }

extern "C" const char* tq_error_string(int code) {
  switch (code) {
    case TQ_OK: return "ok";
    case TQ_ERR_BAD_ARG: return "bad argument (null pointer, size, R >= K, rank out of range)";
    case TQ_ERR_UNSUPPORTED: return "unsupported K / rotation kind / dtype / N for this build";
    case TQ_ERR_MISALIGNED: return "pointer is not 16-byte aligned";
    case TQ_ERR_CUDA: return "CUDA call failed (see tq_last_cuda_error)";
    case TQ_ERR_DEVICE_STATUS: return "a bounded device-side wait ran out (see tq_gemm_status)";
    case TQ_ERR_TOO_LARGE: return "size beyond the stated maximum of this entry point";
    default: return "unknown error code";
  }
}

extern "C" const char* tq_last_cuda_error(void) { return tq::g_cuda_error; }

// Rotation + RTN quantisation of a weight matrix is the pure (R = 0) prologue applied to the
// rows of W with the weight flavour of the scale clamp; the two tail layouts are re-layouts
// of its outputs.
extern "C" int tq_prepare_weight(const void* w, int N, int K, int had_kind, float eps, uint8_t* b_col,
                                 float* w_scale, void* w_rot, uint8_t* b_row, void* w_t, void* stream) {
  if (!w || !b_col || !w_scale || N <= 0 || K <= 0) return TQ_ERR_BAD_ARG;
  if (w_t && !w_rot) return TQ_ERR_BAD_ARG;
  if ((b_row || w_t) && (N % 2 != 0)) return TQ_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = tq::run_prologue(w, N, K, had_kind, 0, 1, eps, 1, b_col, nullptr, w_scale, nullptr, nullptr, nullptr, 0, nullptr, 0, nullptr, nullptr,
                            nullptr, nullptr, w_rot, nullptr, 0.0f, st);
  if (rc != TQ_OK) return rc;
  if (w_t) {
    rc = tq::run_transpose_bf16(w_rot, w_t, N, K, st);
    if (rc != TQ_OK) return rc;
  }
  if (b_row) rc = tq::run_col_to_row_s4(b_col, b_row, N, K, st);
  return rc;
}
