// Small-M (decode) path, M <= 64 token rows: HBM-bound streaming of the INT4 weights.
//
//  * gemv_s4_kernel: C[m,n] += sum_k qa[m,k] qw[n,k] over one K range (split-K over blockIdx.y), exact int32.
//    A CTA owns 64 output channels: its eight warps take eight channels each and stream their packed weight
//    rows with one 128-bit load per lane and 128-wide K slice; the (few) activation rows of the K range are
//    staged once in shared memory.  Both operands are widened with the same nibble order (value x 16 in the
//    top nibble, exact >> 8 afterwards) and multiplied with mma.sync m16n8k32 s8: with at most 64 rows the
//    tensor-core rate is irrelevant, the weight stream is what takes time.  Partial sums are added with int32
//    atomics into C, which the entry point zeroes first (integer addition: any order gives the same bits); with a
//    single K range the results are stored directly.
//  * tail_small_kernel: the tail correction for few rows reads only the weight rows it needs (M*R rows of the
//    [K,N] bf16 matrix) instead of streaming whole strips.  The sum over the R entries is split into eight
//    interleaved fp32 fma chains (entry r goes to chain r mod 8) that are combined pairwise in a fixed order,
//    which is what the CPU oracle states for this path.
//
// Reference behaviour covered: the reference has no small-M path of its own (its decode bench runs the same
// kernels at M = 16/64/256: tools/bench_qwen3_decode_split_romeo_quarot_v33.py:36,97-108).
#include "tq_common.cuh"

namespace tq {
namespace {

constexpr int DV_THREADS = 256;
constexpr int DV_CH = 64;     // channels per CTA
constexpr int DV_KS = 128;    // K slice per step

__device__ __forceinline__ void widen16(const uint4& w, uint32_t (&o)[8]) {
  o[0] = (w.x << 4) & 0xf0f0f0f0u;
  o[1] = w.x & 0xf0f0f0f0u;
  o[2] = (w.y << 4) & 0xf0f0f0f0u;
  o[3] = w.y & 0xf0f0f0f0u;
  o[4] = (w.z << 4) & 0xf0f0f0f0u;
  o[5] = w.z & 0xf0f0f0f0u;
  o[6] = (w.w << 4) & 0xf0f0f0f0u;
  o[7] = w.w & 0xf0f0f0f0u;
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT = number of 16-row tiles of the activations (M <= 16 * MT).  A8: shared memory holds the activations as
// bytes in the order widen16 produces, so their fragments are plain loads.  SRC8: they also arrive that way, as
// true INT8 codes -- the prologue's a_q8 output; otherwise they arrive packed and are widened (value x 16) either
// while staging (A8; measured slower than per-fragment widening, kept as an instantiation option) or per fragment.
// NB = 8-channel tiles per warp (a CTA owns 64 NB channels).  With more than one 16-row tile of activations the
// fragment loads from shared memory, not the weight stream, are what a warp spends its time on (64 rows x 128 bytes
// per K slice against 512 bytes of weights for 8 channels): NB = 4 uses every activation fragment for four channel
// tiles, a lane then streams the weights of four channels.
template <int MT, bool A8, bool SRC8, int NB>
__global__ void __launch_bounds__(DV_THREADS)
gemv_s4_kernel(const uint8_t* __restrict__ a_pack, const uint8_t* __restrict__ b_col, int32_t* __restrict__ C, int M,
               int N, int K, int k_per_split, int direct, int cgroups, long long pstride) {
  extern __shared__ __align__(16) unsigned char sm_a[];  // [16*MT rows][pitch] packed activations of this K range
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, j = lane & 3;
  const int k0 = blockIdx.y * k_per_split;
  const int k1 = min(K, k0 + k_per_split);
  if (k0 >= k1) return;
  C += (size_t)blockIdx.y * (size_t)pstride;  // partial-sum mode: one [M, N] slab per K range (pstride = M * N)
  static_assert(A8 || !SRC8, "INT8 input is staged as bytes");
  constexpr int AB = A8 ? 1 : 2;           // K elements per staged activation byte
  constexpr int SB = SRC8 ? 1 : 2;         // K elements per input byte
  const int kbytes = (k1 - k0) / AB;       // staged bytes per row in this range
  // row pitch chosen so that the fragment loads of a quarter warp fall into distinct 16-byte bank groups
  const int pitch = kbytes + (A8 ? 16 : 64);

  const int nslices = (k1 - k0) / DV_KS;
  constexpr int PF = (MT <= 2 ? 8 : 4) / NB > 2 ? (MT <= 2 ? 8 : 4) / NB : 2;  // K slices of weight loads in flight per lane
  constexpr int CH = DV_CH * NB;       // channels per CTA
  const bool hi_rows = M > 8;  // rows 8..15 of the (only) tile exist

  // A CTA goes through `cgroups` groups of 64 channels with the same staged activations.
  for (int cg = 0; cg < cgroups; ++cg) {
    const int nbase = (blockIdx.x * cgroups + cg) * CH;
    if (nbase >= N) break;
    // the weight stream starts first: it does not depend on the activations
    const uint8_t* wrow[NB];  // rows of the channels whose weights this lane streams: tile b, row g of the tile
    bool wok[NB];
    uint4 wq[PF][NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const int n = nbase + (warp * NB + b) * 8 + g;
      wok[b] = n < N;
      wrow[b] = b_col + (size_t)min(n, N - 1) * (K / 2) + k0 / 2 + j * 16;
    }
#pragma unroll
    for (int s = 0; s < PF; ++s)
#pragma unroll
      for (int b = 0; b < NB; ++b)
        wq[s][b] = (s < nslices && wok[b]) ? ldg_nc_128(wrow[b] + (size_t)s * (DV_KS / 2)) : make_uint4(0u, 0u, 0u, 0u);

    if (cg == 0) {
      const int in_bytes = (k1 - k0) / SB;  // input bytes per row in this range
      for (int i = tid; i < 16 * MT * (in_bytes / 16); i += DV_THREADS) {
        const int row = i / (in_bytes / 16), piece = i % (in_bytes / 16);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < M) v = *reinterpret_cast<const uint4*>(a_pack + (size_t)row * (K / SB) + k0 / SB + piece * 16);
        if (A8 && !SRC8) {
          uint32_t o[8];
          widen16(v, o);
          *reinterpret_cast<uint4*>(sm_a + row * pitch + piece * 32) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(sm_a + row * pitch + piece * 32 + 16) = make_uint4(o[4], o[5], o[6], o[7]);
        } else {
          *reinterpret_cast<uint4*>(sm_a + row * pitch + piece * 16) = v;
        }
      }
      __syncthreads();
    }

    int acc[MT][NB][4];
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[t][b][i] = 0;
    for (int s0 = 0; s0 < nslices; s0 += PF) {
#pragma unroll
      for (int u = 0; u < PF; ++u) {
        const int s = s0 + u;
        if (s < nslices) {
          uint32_t bw[NB][8];
          const int sn = s + PF;
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            widen16(wq[u][b], bw[b]);
            wq[u][b] = (sn < nslices && wok[b]) ? ldg_nc_128(wrow[b] + (size_t)sn * (DV_KS / 2)) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int t = 0; t < MT; ++t) {
            uint32_t a[8], c[8];
            if (A8) {
              const unsigned char* plo = sm_a + (16 * t + g) * pitch + s * DV_KS + j * 32;
              const unsigned char* phi = sm_a + (16 * t + g + 8) * pitch + s * DV_KS + j * 32;
              const uint4 l0 = *reinterpret_cast<const uint4*>(plo), l1 = *reinterpret_cast<const uint4*>(plo + 16);
              a[0] = l0.x, a[1] = l0.y, a[2] = l0.z, a[3] = l0.w, a[4] = l1.x, a[5] = l1.y, a[6] = l1.z, a[7] = l1.w;
              if (MT > 1 || hi_rows) {
                const uint4 h0 = *reinterpret_cast<const uint4*>(phi), h1 = *reinterpret_cast<const uint4*>(phi + 16);
                c[0] = h0.x, c[1] = h0.y, c[2] = h0.z, c[3] = h0.w, c[4] = h1.x, c[5] = h1.y, c[6] = h1.z, c[7] = h1.w;
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) c[i] = 0u;
              }
            } else {
              const uint4 alo = *reinterpret_cast<const uint4*>(sm_a + (16 * t + g) * pitch + s * (DV_KS / 2) + j * 16);
              widen16(alo, a);
              if (MT > 1 || hi_rows) {
                const uint4 ahi = *reinterpret_cast<const uint4*>(sm_a + (16 * t + g + 8) * pitch + s * (DV_KS / 2) + j * 16);
                widen16(ahi, c);
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) c[i] = 0u;
              }
            }
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
              for (int qd = 0; qd < 4; ++qd)
                mma_s8(acc[t][b], a[2 * qd], c[2 * qd], a[2 * qd + 1], c[2 * qd + 1], bw[b][2 * qd], bw[b][2 * qd + 1]);
          }
        }
      }
    }

    // accumulator fragment: rows g and g + 8 of the tile, channels 2j and 2j + 1 of the eight of channel tile b
#pragma unroll
    for (int t = 0; t < MT; ++t) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int nc = nbase + (warp * NB + b) * 8 + 2 * j;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = 16 * t + g + ((i >> 1) << 3), col = nc + (i & 1);
          if (row < M && col < N) {
            const int v = acc[t][b][i] >> (SRC8 ? 4 : 8);  // one or both operands carry a factor 16
            if (direct)
              C[(size_t)row * N + col] = v;  // the only K range: no accumulation across CTAs
            else
              atomicAdd(C + (size_t)row * N + col, v);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- tail, few rows
constexpr int TS_THREADS = 256;   // 8 warps = 8 interleaved chains, 32 lanes x 8 columns = 256 columns per CTA

__global__ void __launch_bounds__(TS_THREADS)
tail_small_kernel(const uint16_t* __restrict__ idx, const uint16_t* __restrict__ val, const uint16_t* __restrict__ w_t,
                  float* __restrict__ out, int N, int R, int ld) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  uint16_t* s_idx = reinterpret_cast<uint16_t*>(sm_raw);
  uint16_t* s_val = s_idx + ((R + 7) & ~7);
  float* s_part = reinterpret_cast<float*>(s_val + ((R + 7) & ~7));  // [8][256]
  const int tid = threadIdx.x, chain = tid >> 5, lane = tid & 31;
  const int m = blockIdx.y;
  const int n = blockIdx.x * 256 + lane * 8;
  for (int r = tid; r < R; r += TS_THREADS) {
    s_idx[r] = idx[(size_t)m * ld + r];
    s_val[r] = val[(size_t)m * ld + r];
  }
  __syncthreads();
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  if (n < N) {
    constexpr int U = 4;
    for (int r0 = chain; r0 < R; r0 += 8 * U) {
      uint4 w[U];
      float x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = r0 + 8 * u;
        const bool in = r < R;
        x[u] = in ? bf16_bits_to_f32(s_val[r]) : 0.0f;
        w[u] = in ? ldg_nc_128(w_t + (size_t)s_idx[r] * N + n) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (r0 + 8 * u < R) {
          acc[0] = fmaf(x[u], __uint_as_float(w[u].x << 16), acc[0]);
          acc[1] = fmaf(x[u], __uint_as_float(w[u].x & 0xffff0000u), acc[1]);
          acc[2] = fmaf(x[u], __uint_as_float(w[u].y << 16), acc[2]);
          acc[3] = fmaf(x[u], __uint_as_float(w[u].y & 0xffff0000u), acc[3]);
          acc[4] = fmaf(x[u], __uint_as_float(w[u].z << 16), acc[4]);
          acc[5] = fmaf(x[u], __uint_as_float(w[u].z & 0xffff0000u), acc[5]);
          acc[6] = fmaf(x[u], __uint_as_float(w[u].w << 16), acc[6]);
          acc[7] = fmaf(x[u], __uint_as_float(w[u].w & 0xffff0000u), acc[7]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) s_part[chain * 256 + lane * 8 + i] = acc[i];
  __syncthreads();
  const int col = blockIdx.x * 256 + tid;
  if (col < N) {
    float p[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) p[c] = s_part[c * 256 + tid];
    const float s = __fadd_rn(__fadd_rn(__fadd_rn(p[0], p[1]), __fadd_rn(p[2], p[3])),
                              __fadd_rn(__fadd_rn(p[4], p[5]), __fadd_rn(p[6], p[7])));
    out[(size_t)m * N + col] = s;
  }
}

template <int MT, bool A8, bool SRC8, int NB>
int launch_gemv(const uint8_t* a_pack, const uint8_t* b_col, int32_t* C, int M, int N, int K, int kps, int splits,
                int cgroups, bool partials, cudaStream_t st) {
  const size_t smem = (size_t)16 * MT * (A8 ? kps + 16 : kps / 2 + 64);
  auto kern = gemv_s4_kernel<MT, A8, SRC8, NB>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && !(dev < 64 && configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return TQ_ERR_CUDA;
    }
    if (dev < 64) configured[dev] = true;
  }
  dim3 grid((N + DV_CH * NB * cgroups - 1) / (DV_CH * NB * cgroups), splits);
  if (splits > 1 && !partials) {  // partial sums of the K ranges meet in C through atomics
    cudaError_t e = cudaMemsetAsync(C, 0, (size_t)M * N * sizeof(int32_t), st);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return TQ_ERR_CUDA;
    }
  }
  kern<<<grid, DV_THREADS, smem, st>>>(a_pack, b_col, C, M, N, K, kps, (splits == 1 || partials) ? 1 : 0, cgroups,
                                             partials ? (long long)M * N : 0ll);
  return check_launch();
}

}  // namespace
}  // namespace tq

namespace tq {
namespace {

struct GemvPlan {
  int sps, splits, mt, cgroups, nb;
};

int g_gemv_tiles = -1;  // tq_set_gemv_channel_tiles: -1 = by row count, 1 / 2 / 4 = 8-channel tiles per warp

// K ranges of a call: `split_k` < 1 lets the library choose
GemvPlan plan_gemv(int M, int N, int K, int split_k, bool a8) {
  GemvPlan g;
  const int slices = K / DV_KS;
  g.mt = (M + 15) / 16;
  // More than 16 rows (packed activations): four channel tiles per warp share every activation fragment.  Timed on
  // the Qwen3-8B layer shapes with the weights coming from HBM: 17..32 rows -- four tiles ahead everywhere (gate_up
  // 21 against 26 us, down 11 against 16 us); 33..64 rows -- ahead only where K or N is large, one tile otherwise.
  g.nb = (a8 || g.mt < 2) ? 1 : (g_gemv_tiles > 0 ? g_gemv_tiles : ((g.mt == 2 || K >= 8192 || N >= 16384) ? 4 : 1));
  // groups of 64 channels per CTA (sharing the staged activations): more than one measured slower at every M
  // on the Qwen3-8B layer shapes -- the smaller grid costs more than the repeated staging
  g.cgroups = 1;
  if (split_k < 1) {
    const int ctas_n = (N + DV_CH * g.nb * g.cgroups - 1) / (DV_CH * g.nb * g.cgroups);
    if (g.nb == 1 && g.mt == 1) {
      // Up to 16 rows: a K range of eight slices -- exactly the eight weight loads a lane keeps in flight, requested
      // in one go before anything else happens in the CTA -- was the fastest split on every Qwen3-8B layer shape
      // (weights from HBM: qkv 6.1 us with 4 ranges against 6.9 with 7, o 4.9 against 5.8 with 8, down 9.8 with 12
      // against 11.0 with 10, gate_up 15.2 with 4); shorter ranges only where that leaves SMs without a CTA
      int sps = slices < 8 ? slices : 8;
      while (sps > 1 && (long)ctas_n * ((slices + sps - 1) / sps) < 148) --sps;
      split_k = (slices + sps - 1) / sps;
    } else {  // (timed likewise) four CTAs per SM with one channel tile per warp, two with four tiles
      const int per_sm = g.nb == 1 ? (ctas_n >= 256 ? 8 : 4) : 2;
      split_k = (per_sm * 148 + ctas_n - 1) / ctas_n;
    }
  }
  if (split_k > slices) split_k = slices;
  g.sps = (slices + split_k - 1) / split_k;  // slices per split
  // staged activation rows: at most 56 KB, four CTAs per SM
  const int max_sps = (56 * 1024 / (16 * g.mt) - 64) / (a8 ? DV_KS : DV_KS / 2);
  if (g.sps > max_sps) g.sps = max_sps;
  g.splits = (slices + g.sps - 1) / g.sps;
  return g;
}

int run_gemv(const uint8_t* a_pack, const int8_t* a_q8, const uint8_t* b_col, int32_t* C, int M, int N, int K,
             int split_k, bool partials, cudaStream_t st) {
  if ((a_pack == nullptr) == (a_q8 == nullptr) || !b_col || !C || M < 0 || N <= 0 || K <= 0) return TQ_ERR_BAD_ARG;
  if (M > 64 || K % DV_KS != 0) return TQ_ERR_UNSUPPORTED;
  const bool a8 = a_q8 != nullptr;
  const uint8_t* a = a8 ? reinterpret_cast<const uint8_t*>(a_q8) : a_pack;
  if (!aligned16(a) || !aligned16(b_col)) return TQ_ERR_MISALIGNED;
  if (M == 0) return TQ_OK;
  const GemvPlan g = plan_gemv(M, N, K, split_k, a8);
  if (partials && split_k >= 1 && g.splits != split_k) return TQ_ERR_BAD_ARG;  // the slab count must be the caller's
  const int kps = g.sps * DV_KS, splits = g.splits, cgroups = g.cgroups, mt = g.mt;
  if (a8) {
    if (mt == 1) return launch_gemv<1, true, true, 1>(a, b_col, C, M, N, K, kps, splits, cgroups, partials, st);
    if (mt == 2) return launch_gemv<2, true, true, 1>(a, b_col, C, M, N, K, kps, splits, cgroups, partials, st);
    if (mt == 3) return launch_gemv<3, true, true, 1>(a, b_col, C, M, N, K, kps, splits, cgroups, partials, st);
    return launch_gemv<4, true, true, 1>(a, b_col, C, M, N, K, kps, splits, cgroups, partials, st);
  }
#define TQ_GEMV(MT_, NB_) \
  if (mt == MT_ && g.nb == NB_) \
    return launch_gemv<MT_, false, false, NB_>(a, b_col, C, M, N, K, kps, splits, cgroups, partials, st);
  TQ_GEMV(1, 1)
  TQ_GEMV(2, 1) TQ_GEMV(2, 2) TQ_GEMV(2, 4)
  TQ_GEMV(3, 1) TQ_GEMV(3, 2) TQ_GEMV(3, 4)
  TQ_GEMV(4, 1) TQ_GEMV(4, 2) TQ_GEMV(4, 4)
#undef TQ_GEMV
  return TQ_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace tq

extern "C" int tq_int4_gemv_splitk(const uint8_t* a_pack, const int8_t* a_q8, const uint8_t* b_col, int32_t* C, int M,
                                   int N, int K, int split_k, void* stream) {
  return tq::run_gemv(a_pack, a_q8, b_col, C, M, N, K, split_k, false, (cudaStream_t)stream);
}

extern "C" int tq_set_gemv_channel_tiles(int tiles) {
  if (tiles != -1 && tiles != 1 && tiles != 2 && tiles != 4) return TQ_ERR_BAD_ARG;
  tq::g_gemv_tiles = tiles;
  return TQ_OK;
}

extern "C" int tq_int4_gemv_plan(int M, int N, int K, int a_is_int8) {
  if (M < 1 || M > 64 || N <= 0 || K <= 0 || K % tq::DV_KS != 0) return TQ_ERR_BAD_ARG;
  return tq::plan_gemv(M, N, K, 0, a_is_int8 != 0).splits;
}

extern "C" int tq_int4_gemv_partials(const uint8_t* a_pack, const int8_t* a_q8, const uint8_t* b_col, int32_t* partials,
                                     int M, int N, int K, int splits, void* stream) {
  if (splits < 1) return TQ_ERR_BAD_ARG;
  return tq::run_gemv(a_pack, a_q8, b_col, partials, M, N, K, splits, true, (cudaStream_t)stream);
}

extern "C" int tq_tail_gather_small(const uint16_t* tail_idx16, const void* tail_val, const void* w_t, float* tail,
                                    int M, int N, int K, int R, int tail_ld, void* stream) {
  using namespace tq;
  if (!tail_idx16 || !tail_val || !w_t || !tail || M < 0 || N <= 0 || K <= 0 || R <= 0 || R >= K || tail_ld < R)
    return TQ_ERR_BAD_ARG;
  if (N % 8 != 0 || R > 8192) return TQ_ERR_UNSUPPORTED;
  if (!aligned16(w_t)) return TQ_ERR_MISALIGNED;
  if (M == 0) return TQ_OK;
  const size_t smem = (size_t)((R + 7) & ~7) * 4 + 8 * 256 * sizeof(float);
  dim3 grid((N + 255) / 256, M);
  tail_small_kernel<<<grid, TS_THREADS, smem, (cudaStream_t)stream>>>(
      tail_idx16, reinterpret_cast<const uint16_t*>(tail_val), reinterpret_cast<const uint16_t*>(w_t), tail, N, R,
      tail_ld);
  return check_launch();
}
