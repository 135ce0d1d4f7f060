// Dense INT4 x INT4 GEMM on the Blackwell tensor cores (sm_100a): tcgen05.mma kind::i8 with
// int32 accumulators in tensor memory, operands staged by TMA as packed INT4 and widened to
// INT8 in shared memory, dequant (+ tail + bias) fused into the epilogue.
//
// One persistent CTA per SM, 14 warps with fixed roles:
//   warp 0        TMA producer: packed A [128 x 64 B] and B [BN x 64 B] tiles of one 128-wide
//                 k-block into a ring of staging buffers (plain 2-D tiled loads, one CTA each)
//   warps 6..13   unpackers: read 16 packed bytes, widen the 32 nibbles to INT8 (value x 16,
//                 sign kept in the top nibble, so no sign extension is needed) and store them
//                 into the canonical K-major 128-byte-swizzled UMMA operand layout
//   warp 1        MMA issuer: 4 x tcgen05.mma (M128 x BN x K32) per k-block into one of two
//                 TMEM accumulators; tcgen05.commit releases operand stages / hands the
//                 accumulator to the epilogue
//   warps 2..5    epilogue: tcgen05.ld the accumulator (one TMEM lane quadrant per warp),
//                 >> 8 (both operands carry the factor 16), then int32 store / int32 atomic
//                 add (split-K) / fused dequant to bf16
// Both operands are widened with the same nibble permutation inside each 32-element group,
// which leaves the dot product unchanged.
//
// Every mbarrier wait is bounded: when a wait runs out, the CTA records a code in a status
// word, raises a block-wide abort flag, drains and frees its tensor memory.
//
// Reference behaviour covered: `qext.matmul(A_pack[M,K/2], B_col[N,K/2]) -> int32 [M,N]`
// (call site tools/bench_hadamard_three_schemes_quarot_dense_sharedqkv_inplace_fusedtopr_v43.py:235-239)
// and the dequant `scale_i32_to_fp16` that follows it (same file :262,283).
#include <cuda.h>

#include <mutex>

#include "tq_common.cuh"
#include "tq_ptx.cuh"

namespace tq {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;            // int8 elements per k-block = one 128-byte swizzle row
constexpr int BKP = BK / 2;        // packed bytes per row per k-block
constexpr int NUM_UNPACK_WARPS = 8;
constexpr int NUT = NUM_UNPACK_WARPS * 32;
constexpr int NUM_THREADS = (6 + NUM_UNPACK_WARPS) * 32;
constexpr int NUM_EPI_THREADS = 128;

enum : int { MODE_I32 = 0, MODE_I32_ATOMIC = 1, MODE_FUSED = 2 };

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, split_k, kb_per_split, kb_total;
  int mode;
  int32_t* C;
  const float* sx;
  const float* sw;
  const float* tail;
  const float* bias;
  __nv_bfloat16* out;
};

template <int BN>
struct Smem {
  static constexpr int SP = (BN == 256) ? 3 : 4;  // packed staging ring
  static constexpr int SU = (BN == 256) ? 3 : 4;  // int8 operand ring
  static constexpr int PACKED_STAGE = (BM + BN) * BKP;
  static constexpr int OPER_STAGE = (BM + BN) * BK;
  static constexpr int OPER_OFF = 0;  // operand ring first: 1024-byte aligned stages
  static constexpr int PACKED_OFF = SU * OPER_STAGE;
  static constexpr int BAR_OFF = PACKED_OFF + SP * PACKED_STAGE;
  static constexpr int NUM_BARS = 2 * SP + 2 * SU + 4;
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int DYN = TOTAL + 1024;  // slack to align the base to 1024 bytes
};

struct TileCoord {
  int mt, nt, kb0, nkb;
};
__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, int t) {
  TileCoord c;
  c.mt = t % p.tiles_m;
  const int r = t / p.tiles_m;
  c.nt = r % p.tiles_n;
  const int ks = r / p.tiles_n;
  c.kb0 = ks * p.kb_per_split;
  c.nkb = min(p.kb_per_split, p.kb_total - c.kb0);
  return c;
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using S = Smem<BN>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_dyn + (base - raw);

  const uint32_t bars = base + S::BAR_OFF;
  auto full_p = [&](int s) { return bars + 8u * s; };
  auto empty_p = [&](int s) { return bars + 8u * (S::SP + s); };
  auto full_u = [&](int s) { return bars + 8u * (2 * S::SP + s); };
  auto empty_u = [&](int s) { return bars + 8u * (2 * S::SP + S::SU + s); };
  auto acc_full = [&](int s) { return bars + 8u * (2 * S::SP + 2 * S::SU + s); };
  auto acc_empty = [&](int s) { return bars + 8u * (2 * S::SP + 2 * S::SU + 2 + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + S::BAR_OFF + S::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + S::BAR_OFF + S::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n * p.split_k;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_a)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_b)) : "memory");
    for (int s = 0; s < S::SP; ++s) {
      mbar_init(full_p(s), 1);
      mbar_init(empty_p(s), NUM_UNPACK_WARPS);
    }
    for (int s = 0; s < S::SU; ++s) {
      mbar_init(full_u(s), NUM_UNPACK_WARPS);
      mbar_init(empty_u(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), NUM_EPI_THREADS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const TileCoord c = tile_coord(p, t);
        for (int kb = c.kb0; kb < c.kb0 + c.nkb; ++kb) {
          if (!(ok = mbar_wait(empty_p(s), ph ^ 1u, abort_flag, 0x1u))) break;
          mbar_arrive_expect_tx(full_p(s), S::PACKED_STAGE);
          const uint32_t dst = base + S::PACKED_OFF + s * S::PACKED_STAGE;
          tma_load_2d(dst, &tmap_a, kb * BKP, c.mt * BM, full_p(s));
          tma_load_2d(dst + BM * BKP, &tmap_b, kb * BKP, c.nt * BN, full_p(s));
          if (++s == S::SP) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_i8<BN>();
      int su = 0, as = 0;
      uint32_t phu = 0, pha = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const TileCoord c = tile_coord(p, t);
        if (!(ok = mbar_wait(acc_empty(as), pha ^ 1u, abort_flag, 0x2u))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
        for (int kb = 0; kb < c.nkb; ++kb) {
          if (!(ok = mbar_wait(full_u(su), phu, abort_flag, 0x4u))) break;
          tc_fence_after();
          const uint32_t a_addr = base + S::OPER_OFF + su * S::OPER_STAGE;
          const uint32_t b_addr = a_addr + BM * BK;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_i8(d_tmem, make_smem_desc(a_addr + k * 32), make_smem_desc(b_addr + k * 32), idesc,
                    (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty_u(su));
          if (++su == S::SU) {
            su = 0;
            phu ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(acc_full(as));
        if (++as == 2) {
          as = 0;
          pha ^= 1u;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    int as = 0;
    uint32_t pha = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const TileCoord c = tile_coord(p, t);
      if (!(ok = mbar_wait(acc_full(as), pha, abort_flag, 0x8u))) break;
      tc_fence_after();
      const int row = c.mt * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const float sx = (p.mode == MODE_FUSED && row_ok) ? p.sx[row] : 0.0f;
      const size_t rowoff = (size_t)row * p.N;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(as * BN + c0), r);
        const int n0 = c.nt * BN + c0;
        if (!row_ok || n0 >= p.N) continue;
        if (p.mode == MODE_I32) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (n0 + 4 * j < p.N) {
              int4 v = make_int4((int)r[4 * j] >> 8, (int)r[4 * j + 1] >> 8, (int)r[4 * j + 2] >> 8, (int)r[4 * j + 3] >> 8);
              *reinterpret_cast<int4*>(p.C + rowoff + n0 + 4 * j) = v;
            }
          }
        } else if (p.mode == MODE_I32_ATOMIC) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (n0 + j < p.N) atomicAdd(p.C + rowoff + n0 + j, (int)r[j] >> 8);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = n0 + 8 * j;
            if (n < p.N) {
              float d[8];
              const float4 w0 = *reinterpret_cast<const float4*>(p.sw + n);
              const float4 w1 = *reinterpret_cast<const float4*>(p.sw + n + 4);
              const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
              for (int i = 0; i < 8; ++i)
                d[i] = __fmul_rn(__fmul_rn((float)((int)r[8 * j + i] >> 8), sx), ws[i]);
              if (p.tail) {
                const float4 t0 = *reinterpret_cast<const float4*>(p.tail + rowoff + n);
                const float4 t1 = *reinterpret_cast<const float4*>(p.tail + rowoff + n + 4);
                const float ts[8] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) d[i] = __fadd_rn(d[i], ts[i]);
              }
              if (p.bias) {
                const float4 b0 = *reinterpret_cast<const float4*>(p.bias + n);
                const float4 b1 = *reinterpret_cast<const float4*>(p.bias + n + 4);
                const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) d[i] = __fadd_rn(d[i], bs[i]);
              }
              uint4 o;
              o.x = f32_to_bf16_bits(d[0]) | (f32_to_bf16_bits(d[1]) << 16);
              o.y = f32_to_bf16_bits(d[2]) | (f32_to_bf16_bits(d[3]) << 16);
              o.z = f32_to_bf16_bits(d[4]) | (f32_to_bf16_bits(d[5]) << 16);
              o.w = f32_to_bf16_bits(d[6]) | (f32_to_bf16_bits(d[7]) << 16);
              *reinterpret_cast<uint4*>(p.out + rowoff + n) = o;
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty(as));
      if (++as == 2) {
        as = 0;
        pha ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ unpackers
    const int utid = threadIdx.x - 6 * 32;
    int sp = 0, su = 0;
    uint32_t php = 0, phu = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const TileCoord c = tile_coord(p, t);
      for (int kb = 0; kb < c.nkb; ++kb) {
        if (!(ok = mbar_wait(full_p(sp), php, abort_flag, 0x10u))) break;
        if (!(ok = mbar_wait(empty_u(su), phu ^ 1u, abort_flag, 0x20u))) break;
        tc_fence_after();
        const unsigned char* src = sm + S::PACKED_OFF + sp * S::PACKED_STAGE;
        unsigned char* dst = sm + S::OPER_OFF + su * S::OPER_STAGE;
#pragma unroll
        for (int task = utid; task < (BM + BN) * 4; task += NUT) {
          const int row = task >> 2, piece = task & 3;
          const uint4 w = *reinterpret_cast<const uint4*>(src + row * BKP + piece * 16);
          unsigned char* drow = dst + (row >> 3) * 1024 + (row & 7) * 128;
          uint4 lo, hi;
          lo.x = (w.x << 4) & 0xf0f0f0f0u;
          lo.y = w.x & 0xf0f0f0f0u;
          lo.z = (w.y << 4) & 0xf0f0f0f0u;
          lo.w = w.y & 0xf0f0f0f0u;
          hi.x = (w.z << 4) & 0xf0f0f0f0u;
          hi.y = w.z & 0xf0f0f0f0u;
          hi.z = (w.w << 4) & 0xf0f0f0f0u;
          hi.w = w.w & 0xf0f0f0f0u;
          *reinterpret_cast<uint4*>(drow + (((2 * piece) ^ (row & 7)) << 4)) = lo;
          *reinterpret_cast<uint4*>(drow + (((2 * piece + 1) ^ (row & 7)) << 4)) = hi;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(full_u(su));
          mbar_arrive(empty_p(sp));
        }
        if (++sp == S::SP) {
          sp = 0;
          php ^= 1u;
        }
        if (++su == S::SU) {
          su = 0;
          phu ^= 1u;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------ host side
// [rows, K/2] bytes, box = [64 bytes, box_rows]; rows past the end read as zero.
bool make_packed_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
  return make_tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, ptr, (uint64_t)(K / 2), (uint64_t)rows,
                            (uint64_t)(K / 2), BKP, box_rows);
}

template <int BN>
int launch_gemm(const uint8_t* a_pack, const uint8_t* b_col, GemmParams p, cudaStream_t st) {
  using S = Smem<BN>;
  auto kern = gemm_kernel<BN>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(dev < 64 && configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::DYN);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return TQ_ERR_CUDA;
    }
    if (dev < 64) configured[dev] = true;
  }
  CUtensorMap ma, mb;
  if (!make_packed_map(&ma, a_pack, p.M, p.K, BM) || !make_packed_map(&mb, b_col, p.N, p.K, BN)) return TQ_ERR_CUDA;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.kb_total = p.K / BK;
  if (p.split_k < 1) p.split_k = 1;
  if (p.split_k > p.kb_total) p.split_k = p.kb_total;
  p.kb_per_split = (p.kb_total + p.split_k - 1) / p.split_k;
  p.split_k = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = p.tiles_m * p.tiles_n * p.split_k;
  const int grid = total < sms ? total : sms;
  kern<<<grid, NUM_THREADS, S::DYN, st>>>(ma, mb, p);
  return check_launch();
}

int run_gemm(const uint8_t* a_pack, const uint8_t* b_col, GemmParams p, cudaStream_t st) {
  if (!a_pack || !b_col || p.M < 0 || p.N <= 0 || p.K <= 0) return TQ_ERR_BAD_ARG;
  if (p.K % BK != 0 || p.N % 8 != 0) return TQ_ERR_UNSUPPORTED;
  if (!aligned16(a_pack) || !aligned16(b_col)) return TQ_ERR_MISALIGNED;
  if (p.M == 0) return TQ_OK;
  // wide tiles when they still fill the machine, narrow ones for small problems / split-K
  const long tiles256 = (long)((p.M + BM - 1) / BM) * ((p.N + 255) / 256) * (p.split_k > 0 ? p.split_k : 1);
  if (tiles256 >= 148) return launch_gemm<256>(a_pack, b_col, p, st);
  return launch_gemm<128>(a_pack, b_col, p, st);
}

}  // namespace
}  // namespace tq

extern "C" int tq_int4_matmul(const uint8_t* a_pack, const uint8_t* b_col, int32_t* C, int M, int N, int K,
                              int split_k, void* stream) {
  if (!C) return TQ_ERR_BAD_ARG;
  if (!tq::aligned16(C)) return TQ_ERR_MISALIGNED;
  tq::GemmParams p = {};
  p.M = M;
  p.N = N;
  p.K = K;
  p.split_k = split_k < 1 ? 1 : split_k;
  p.mode = p.split_k > 1 ? tq::MODE_I32_ATOMIC : tq::MODE_I32;
  p.C = C;
  return tq::run_gemm(a_pack, b_col, p, (cudaStream_t)stream);
}

extern "C" int tq_split_gemm_fused(const uint8_t* a_pack, const float* body_scale, const uint8_t* b_col,
                                   const float* w_scale, const float* tail, const float* bias, void* out_bf16,
                                   int M, int N, int K, void* stream) {
  if (!body_scale || !w_scale || !out_bf16) return TQ_ERR_BAD_ARG;
  if (!tq::aligned16(out_bf16) || !tq::aligned16(w_scale) || (tail && !tq::aligned16(tail)) ||
      (bias && !tq::aligned16(bias)))
    return TQ_ERR_MISALIGNED;
  tq::GemmParams p = {};
  p.M = M;
  p.N = N;
  p.K = K;
  p.split_k = 1;
  p.mode = tq::MODE_FUSED;
  p.sx = body_scale;
  p.sw = w_scale;
  p.tail = tail;
  p.bias = bias;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  return tq::run_gemm(a_pack, b_col, p, (cudaStream_t)stream);
}

extern "C" int tq_gemm_status(unsigned int* status) {
  if (!status) return TQ_ERR_BAD_ARG;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(status, tq::g_status, sizeof(unsigned int));
  if (e == cudaSuccess && *status) {  // read-and-clear: a code reports the launches since the previous call
    const unsigned int zero = 0;
    e = cudaMemcpyToSymbol(tq::g_status, &zero, sizeof(unsigned int));
  }
  if (e != cudaSuccess) {
    tq::set_last_cuda_error(e);
    return TQ_ERR_CUDA;
  }
  return *status ? TQ_ERR_DEVICE_STATUS : TQ_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Split-K linear without any allocation by anybody: the int32 accumulators that the split-K GEMM needs
// between its atomic adds and the finishing pass live in a fixed array inside the library image instead of
// in a buffer handed in by the caller.
//
// Who needs this: a host that may not, or cannot, obtain device memory at the time it runs a small-M linear.
// Typical cases are a serving process that gave the whole device to its own memory pool at start-up (a later
// cudaMalloc then fails or eats into the pool's headroom), a decode loop in a plain C/C++ host that has no
// caching allocator and must not call cudaMalloc/cudaFree per token because both synchronise the device, and
// plug-in style code whose execute callback is forbidden to allocate.  Such a caller still owns its inputs
// and its output; only the intermediate accumulators come from here.
//
// Limits and rules:
//  * M * N <= TQ_NOALLOC_MAX_ELEMS (1 Mi accumulators = 4 MiB).  Every GPU that loads the library carries the
//    array in its module image until the process exits, which is why it is kept this small.
//  * The array is shared by all calls on a device and keeps whatever the last call left: this entry point
//    zeroes the M * N accumulators it is about to use at the start of every call.  Two calls whose GPU work
//    overlaps (different streams, or different host threads on different streams) race on it; serialise them.
//  * The device address of the array is looked up with cudaGetSymbolAddress on the first call on each device
//    (with that device current) and cached.  Make that first call once during start-up, before any stream
//    capture is begun on the device.
//  * No cudaMalloc, cudaFree or allocating library routine is called here.
namespace tq {
namespace {

static __device__ __align__(256) int32_t g_noalloc_acc[TQ_NOALLOC_MAX_ELEMS];

// In host code the array's name only stands in for the symbol; the kernels need its device address.
int32_t* noalloc_acc_ptr(int* rc) {
  static std::mutex mu;
  static int32_t* ptrs[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && (dev < 0 || dev >= 64)) e = cudaErrorInvalidDevice;
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    *rc = TQ_ERR_CUDA;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_acc);
    if (e != cudaSuccess || !ptr) {
      set_last_cuda_error(e == cudaSuccess ? cudaErrorInvalidSymbol : e);
      *rc = TQ_ERR_CUDA;
      return nullptr;
    }
    ptrs[dev] = reinterpret_cast<int32_t*>(ptr);
  }
  *rc = TQ_OK;
  return ptrs[dev];
}

__global__ void noalloc_finish_kernel(const int32_t* __restrict__ acc, const float* __restrict__ sx,
                                      const float* __restrict__ sw, const float* __restrict__ tail,
                                      const float* __restrict__ bias, uint16_t* __restrict__ out, int M, int N) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  float d = __fmul_rn(__fmul_rn((float)acc[i], sx[m]), sw[n]);
  if (tail) d = __fadd_rn(d, tail[i]);
  if (bias) d = __fadd_rn(d, bias[n]);
  out[i] = (uint16_t)f32_to_bf16_bits(d);
}

}  // namespace
}  // namespace tq

extern "C" int tq_int4_linear_splitk_noalloc(const uint8_t* a_pack, const float* body_scale, const uint8_t* b_col,
                                             const float* w_scale, const float* tail, const float* bias,
                                             void* out_bf16, int M, int N, int K, int split_k, void* stream) {
  using namespace tq;
  if (!a_pack || !body_scale || !b_col || !w_scale || !out_bf16 || M < 0 || N <= 0 || K <= 0) return TQ_ERR_BAD_ARG;
  if ((unsigned long long)M * (unsigned long long)N > (unsigned long long)TQ_NOALLOC_MAX_ELEMS) return TQ_ERR_TOO_LARGE;
  if (K % BK != 0 || N % 8 != 0) return TQ_ERR_UNSUPPORTED;
  if (!aligned16(a_pack) || !aligned16(b_col)) return TQ_ERR_MISALIGNED;
  if (M == 0) return TQ_OK;
  int rc = TQ_OK;
  int32_t* acc = noalloc_acc_ptr(&rc);
  if (!acc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t total = (size_t)M * N;
  cudaError_t e = cudaMemsetAsync(acc, 0, total * sizeof(int32_t), st);  // the atomic adds need zeros
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return TQ_ERR_CUDA;
  }
  GemmParams p = {};
  p.M = M;
  p.N = N;
  p.K = K;
  p.split_k = split_k < 1 ? 1 : split_k;
  p.mode = MODE_I32_ATOMIC;
  p.C = acc;
  rc = run_gemm(a_pack, b_col, p, st);
  if (rc != TQ_OK) return rc;
  noalloc_finish_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      acc, body_scale, w_scale, tail, bias, reinterpret_cast<uint16_t*>(out_bf16), M, N);
  return check_launch();
}
