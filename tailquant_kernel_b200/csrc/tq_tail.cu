// Sparse tail correction, tail mode T16 (sm_100a):
//   tail[m,n] = sum_r  x_tail[m,r] * W_t[idx[m,r], n]        (W_t = rotated weight, [K,N] bf16)
// as one fp32 fma chain per output in ascending index order.
//
// The rotation scatters the tail positions uniformly over K, so rows share nothing: the work is
// M*R*N multiply-adds that each need one bf16 weight.  A CTA therefore owns a unit of 256 rows
// x 64 columns, streams the 64-column strip of W_t through shared memory in 512-row chunks
// (plain 2-D TMA loads into a two-slot ring), and lets eight lanes read one gathered weight row
// segment (8 x 16 B = 128 contiguous bytes: bank-conflict free) while each of them carries 8
// accumulators for 4 rows.  Index lists are ascending, so the entries of a row that fall into a
// chunk are a contiguous run: every quarter warp walks its cursor through the resident window
// of two chunks, which evens out the different run lengths of the rows sharing a warp.
//
// Reference behaviour covered (for the bf16-tail mode): `sparse_top_add_rowmajor_quad_shared`
// (call site tools/bench_hadamard_three_schemes_quarot_dense_sharedqkv_inplace_fusedtopr_v43.py:287-295)
// and tools/sparse_correction_add_ext_v1.py:64-123.
#include "tq_common.cuh"
#include "tq_ptx.cuh"

namespace tq {
namespace {

constexpr int T_THREADS = 512;
constexpr int T_RQ = 4;                       // rows per quarter warp
constexpr int T_ROWS = (T_THREADS / 8) * T_RQ;  // 256 rows per unit
constexpr int T_COLS = 64;                    // columns per unit (128 bytes of bf16)
constexpr int T_KC = 512;                     // weight rows per chunk
constexpr int T_KC_LOG = 9;
constexpr int T_BUF = T_KC * T_COLS * 2;      // 64 KB per ring slot
constexpr int T_SMEM = 2 * T_BUF + 64 + 1024;
constexpr int T_SENT = 0x7fffffff;

struct TailParams {
  const uint16_t* idx;
  const uint16_t* val;
  float* out;
  int M, N, K, R, ld;
  int units_m, units_n;
};

__global__ void __launch_bounds__(T_THREADS, 1)
tail_kernel(const __grid_constant__ CUtensorMap tmap_w, const TailParams p) {
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_dyn + (base - raw);
  const uint32_t bar0 = base + 2 * T_BUF;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + 2 * T_BUF + 32);

  const int tid = threadIdx.x;
  const int l8 = tid & 7, qw = tid >> 3;
  const int nch = (p.K + T_KC - 1) / T_KC;
  const int total_units = p.units_m * p.units_n;

  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](int g, int chunk, int n0) {  // thread 0 only: chunk -> ring slot g & 1
    const uint32_t bar = bar0 + 8u * (g & 1);
    const uint32_t dst = base + (uint32_t)(g & 1) * T_BUF;
    mbar_arrive_expect_tx(bar, T_BUF);
    tma_load_2d(dst, &tmap_w, n0, chunk * T_KC, bar);
    tma_load_2d(dst + T_BUF / 2, &tmap_w, n0, chunk * T_KC + T_KC / 2, bar);
  };

  int g = 0;  // running chunk number of this CTA: ring slot g & 1, barrier parity (g >> 1) & 1
  bool ok = true;
  for (int u = blockIdx.x; ok && u < total_units; u += gridDim.x) {
    const int n0 = (u % p.units_n) * T_COLS;  // neighbouring CTAs share the rows' index lists
    const int m0 = (u / p.units_n) * T_ROWS;
    if (tid == 0) {
      issue(g, 0, n0);
      if (nch > 1) issue(g + 1, 1, n0);
    }
    float acc[T_RQ][8];
    int cur[T_RQ], kk[T_RQ];
    uint32_t xx[T_RQ];
    const uint16_t* irow[T_RQ];
    const uint16_t* vrow[T_RQ];
#pragma unroll
    for (int j = 0; j < T_RQ; ++j) {
      const int row = m0 + qw * T_RQ + j;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = 0.0f;
      irow[j] = p.idx + (size_t)row * p.ld;
      vrow[j] = p.val + (size_t)row * p.ld;
      cur[j] = 0;
      if (row < p.M && p.R > 0) {
        kk[j] = (int)__ldg(irow[j]);
        xx[j] = (uint32_t)__ldg(vrow[j]);
      } else {
        kk[j] = T_SENT;
        xx[j] = 0;
      }
    }
    if (!(ok = mbar_wait(bar0 + 8u * (g & 1), (uint32_t)((g >> 1) & 1), abort_flag, 0x100u))) break;

    for (int c = 0; c < nch; ++c) {
      if (c + 1 < nch) {
        const int g1 = g + c + 1;
        if (!(ok = mbar_wait(bar0 + 8u * (g1 & 1), (uint32_t)((g1 >> 1) & 1), abort_flag, 0x200u))) break;
      }
      const int chunk_end = (c + 1) * T_KC;      // entries below this must be done in this phase
      const int win_end = (c + 2) * T_KC;        // entries below this have their weights resident
      const int slot_xor = (g + c) & 1;          // ring slot of chunk c; chunk c+1 sits in the other
      bool need;
      do {
        need = false;
#pragma unroll
        for (int j = 0; j < T_RQ; ++j) {
          const int k = kk[j];
          if (k < win_end) {
            const int slot = ((k >> T_KC_LOG) - c) ^ slot_xor;  // (k>>9) is c or c+1
            const uint4 w = *reinterpret_cast<const uint4*>(sm + (slot & 1) * T_BUF + (k & (T_KC - 1)) * (T_COLS * 2) + l8 * 16);
            const float x = bf16_bits_to_f32(xx[j]);
            acc[j][0] = fmaf(x, __uint_as_float(w.x << 16), acc[j][0]);
            acc[j][1] = fmaf(x, __uint_as_float(w.x & 0xffff0000u), acc[j][1]);
            acc[j][2] = fmaf(x, __uint_as_float(w.y << 16), acc[j][2]);
            acc[j][3] = fmaf(x, __uint_as_float(w.y & 0xffff0000u), acc[j][3]);
            acc[j][4] = fmaf(x, __uint_as_float(w.z << 16), acc[j][4]);
            acc[j][5] = fmaf(x, __uint_as_float(w.z & 0xffff0000u), acc[j][5]);
            acc[j][6] = fmaf(x, __uint_as_float(w.w << 16), acc[j][6]);
            acc[j][7] = fmaf(x, __uint_as_float(w.w & 0xffff0000u), acc[j][7]);
            const int nx = ++cur[j];
            if (nx < p.R) {
              kk[j] = (int)__ldg(irow[j] + nx);
              xx[j] = (uint32_t)__ldg(vrow[j] + nx);
            } else {
              kk[j] = T_SENT;
            }
          }
          need |= kk[j] < chunk_end;
        }
      } while (__any_sync(0xffffffffu, need));
      __syncthreads();  // every thread is past chunk c: its ring slot may be refilled
      if (tid == 0 && c + 2 < nch) issue(g + c + 2, c + 2, n0);
    }
    if (!ok) break;
    g += nch;

#pragma unroll
    for (int j = 0; j < T_RQ; ++j) {
      const int row = m0 + qw * T_RQ + j;
      const int n = n0 + l8 * 8;
      if (row < p.M && n < p.N) {
        float* o = p.out + (size_t)row * p.N + n;
        *reinterpret_cast<float4*>(o) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
      }
    }
    // the first chunk of the next unit goes to slot g & 1, last read by chunk nch-2 or nch-1 of
    // this unit; both were fenced by the __syncthreads that ended their phases
  }
}

}  // namespace
}  // namespace tq

extern "C" int tq_tail_gather(const uint16_t* tail_idx16, const void* tail_val, const void* w_t, float* tail,
                              int M, int N, int K, int R, int tail_ld, void* stream) {
  using namespace tq;
  if (!tail_idx16 || !tail_val || !w_t || !tail || M < 0 || N <= 0 || K <= 0 || R <= 0 || R >= K || tail_ld < R)
    return TQ_ERR_BAD_ARG;
  if (N % 8 != 0 || K > 65536) return TQ_ERR_UNSUPPORTED;
  if (!aligned16(w_t) || !aligned16(tail)) return TQ_ERR_MISALIGNED;
  if (M == 0) return TQ_OK;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(dev < 64 && configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return TQ_ERR_CUDA;
    }
    if (dev < 64) configured[dev] = true;
  }
  CUtensorMap map;
  if (!make_tensor_map_2d(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, w_t, (uint64_t)N, (uint64_t)K,
                          (uint64_t)N * 2, T_COLS, T_KC / 2))
    return TQ_ERR_CUDA;
  TailParams p;
  p.idx = tail_idx16;
  p.val = reinterpret_cast<const uint16_t*>(tail_val);
  p.out = tail;
  p.M = M;
  p.N = N;
  p.K = K;
  p.R = R;
  p.ld = tail_ld;
  p.units_m = (M + T_ROWS - 1) / T_ROWS;
  p.units_n = (N + T_COLS - 1) / T_COLS;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = p.units_m * p.units_n;
  const int grid = total < sms ? total : sms;
  tail_kernel<<<grid, T_THREADS, T_SMEM, (cudaStream_t)stream>>>(map, p);
  return check_launch();
}
