// Split GEMM with the tail on the tensor cores (sm_100a): one kernel computes
//   out[m,n] = bf16( (float(sum_k qx[m,k] qw[n,k]) * s_x[m]) * s_w[n]  +  sum_r x_tail[m,r] W_rot[n, idx[m,r]]  + bias[n] )
// with the dense part on tcgen05 kind::i8 (int32 accumulator in tensor memory) and the tail on tcgen05
// kind::f16 (bf16 x bf16, fp32 accumulator in tensor memory) over the zero-filled tail matrix.
//
// Why not gather: after the rotation the tail positions are spread uniformly over K, so the gathered
// form is M*R*N scalar multiply-adds with no operand reuse; on this GPU the dense bf16 MMA over a K-wide,
// 95 %-zero A operand is several times faster than that at ratio 0.05.  The exact-order gather kernel
// (tq_tail.cu) stays available as the bit-exact mode.
//
// One persistent CTA per SM.  For every 128-wide slice of K a tile consumes three operand slots:
//   slot kind        A operand [128 rows]                         B operand [BN rows]
//   int8  (128 k)    INT8 codes of the activations, TMA           INT4 weights: TMA to staging, widened to
//                    (128-byte swizzle) straight into the slot    INT8 (x16) by warps 2..5
//   bf16  (64 k) x2  tail values scattered by the builder warps   rotated bf16 weight rows [N,K], TMA
//                    from the rows' (index, value) lists into a    (128-byte swizzle) straight into the slot
//                    zero-filled tile
// Warp roles: 0 = TMA producer of the INT8 path, 14 = TMA producer of the bf16 weight rows, 1 = MMA issuer
// (+ tensor-memory allocation), 2..5 = weight wideners during the main loop and epilogue at the end of the
// tile, 6..13 = tail-tile builders.  All loads are plain 2-D tiled TMA loads of this GPU's own memory, issued per CTA.
// Every mbarrier wait is bounded (see mbar_wait).
//
// The activation codes arrive as INT8 with the two nibble planes of each 8-element group de-interleaved
// ([0,2,4,6,1,3,5,7]), which is the order the builders' widening of the weights produces, so both
// operands see the same permutation of K and the dot product is unchanged.  Weights carry a factor 16
// (the nibble is kept in the top half of the byte, which makes it sign-correct without an extension),
// removed by an exact >> 4 of the accumulator.
//
// Reference behaviour covered: GEMM + dequant + sparse correction in one kernel, i.e. what the reference
// prototypes in tools/quarot_split_fused_epilogue_ext_v1.py:283-432 and
// tools/qfactory_split_fused_epilogue_v1.py:153-233 (there with an INT4 tail and R fixed at compile time).
#include "tq_common.cuh"
#include "tq_ptx.cuh"

namespace tq {
namespace {

// Diagnostic build (-DTQ_GEMM_PROFILE): cycles each role spends in its barrier waits, summed over CTAs, in
// g_wait_cycles[code]; read back with tq_gemm_wait_cycles().  Compiled out otherwise.
#ifdef TQ_GEMM_PROFILE
__device__ unsigned long long g_wait_cycles[16];
#define TQ_WAIT(slot, call)                                                        \
  [&]() -> bool {                                                                  \
    const long long t0_ = clock64();                                               \
    const bool r_ = (call);                                                        \
    atomicAdd(&g_wait_cycles[slot], (unsigned long long)(clock64() - t0_));        \
    return r_;                                                                     \
  }()
#else
#define TQ_WAIT(slot, call) (call)
#endif

// Diagnostic build (-DTQ_GEMM_TRACE): clock64 stamps of CTA 0's roles for slot uses [TQ_TRACE_Q0, +128), in
// g_trace[role][use][event]; read back with tq_gemm_trace().  Compiled out otherwise.
#ifdef TQ_GEMM_TRACE
#ifndef TQ_TRACE_Q0
#define TQ_TRACE_Q0 30
#endif
__device__ unsigned long long g_trace[8][128][4];
#define TQ_TRACE(role, q, ev)                                                              \
  do {                                                                                     \
    if (blockIdx.x == 0 && (q) >= TQ_TRACE_Q0 && (q) < TQ_TRACE_Q0 + 128)                  \
      g_trace[role][(q) - TQ_TRACE_Q0][ev] = (unsigned long long)clock64();                \
  } while (0)
#else
#define TQ_TRACE(role, q, ev) do { } while (0)
#endif

constexpr int G_BM = 128;
constexpr int G_BK = 128;
constexpr int G_BUILD_WARPS = 8;
constexpr int G_NBT = G_BUILD_WARPS * 32;  // builder threads
constexpr int G_THREADS = (6 + G_BUILD_WARPS + 1) * 32;  // + the warp of the second TMA producer
constexpr int G_SENT = 0x7fffffff;

struct SplitGemmParams {
  int M, N, K, R, ld, ptr_ld;
  int tiles_m, tiles_n, kb_total, has_tail;
  int act;               // 0: out [M, N]; 1: SwiGLU over interleaved (gate, up) channel pairs, out [M, N/2]
  const uint16_t* idx;   // [M, ld] ascending tail indices (only read for runs longer than the record capacity)
  const uint16_t* val;   // [M, ld] tail values
  const uint16_t* ptr;   // [M, ptr_ld] ptr[m][j] = entries of row m with index < 128 j
  const uint32_t* rec;   // [tiles_m][K/64][128][TQ_TAIL_REC_CAP]: tile position | bf16 << 16 (see tq_split_prologue)
  const uint16_t* cnt;   // [tiles_m][K/64][128]: entries of the row in the 64-wide half slice
  const float* sx;
  const float* sw;
  const float* bias;
  __nv_bfloat16* out;
  int32_t* dbg_acc;   // optional [M,N]: the int32 accumulators
  float* dbg_tail;    // optional [M,N]: the fp32 tail sums
};

template <int BN>
struct GS {
  static constexpr int SU = 4;                            // operand slots
  static constexpr int SP = 2;                            // packed-weight staging buffers
  static constexpr int SLOT = (G_BM + BN) * 128;          // A region (16 KB) then B region
  static constexpr int B_OFF = G_BM * 128;
  static constexpr int STAGE = BN * (G_BK / 2);
  static constexpr int STAGE_OFF = SU * SLOT;
  static constexpr int BAR_OFF = STAGE_OFF + SP * STAGE;
  static constexpr int NUM_BARS = 2 * SP + 2 * SU + 2;
  static constexpr int DYN = BAR_OFF + NUM_BARS * 8 + 16 + 1024;
};

template <int BN, int ACT>  // ACT 1: SwiGLU over interleaved (gate, up) channel pairs, out [M, N/2]
__global__ void __launch_bounds__(G_THREADS, 1)
split_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a8, const __grid_constant__ CUtensorMap tmap_b4,
                  const __grid_constant__ CUtensorMap tmap_w, const SplitGemmParams p) {
  using S = GS<BN>;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_dyn + (base - raw);

  const uint32_t bars = base + S::BAR_OFF;
  auto full_p = [&](int s) { return bars + 8u * s; };
  auto empty_p = [&](int s) { return bars + 8u * (S::SP + s); };
  auto full_u = [&](int s) { return bars + 8u * (2 * S::SP + s); };
  auto empty_u = [&](int s) { return bars + 8u * (2 * S::SP + S::SU + s); };
  const uint32_t acc_full = bars + 8u * (2 * S::SP + 2 * S::SU);
  const uint32_t acc_empty = acc_full + 8u;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + S::BAR_OFF + S::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + S::BAR_OFF + S::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;
  const bool has_tail = p.has_tail != 0;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // int32 accumulator, then fp32 tail accumulator

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_a8)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_b4)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    for (int s = 0; s < S::SP; ++s) {
      mbar_init(full_p(s), 1);
      mbar_init(empty_p(s), 4);
    }
    for (int s = 0; s < S::SU; ++s) {
      mbar_init(full_u(s), 4 + 1);  // four warps (wideners, or the tail builders of one half) + the producer's expect_tx
      mbar_init(empty_u(s), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 128);
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

  // slot use number q -> (slot, parity)
  auto slot_of = [](int q) { return q % S::SU; };
  auto par_of = [](int q) { return (uint32_t)((q / S::SU) & 1); };

  // INT4 -> INT8 (x16) of one weight tile by four warps (wtid = 0..127): staging buffer (kbg mod SP) -> B region
  // of slot use q
  auto widen = [&](int q, int kbg_, int wtid) -> bool {
    const int s = slot_of(q), sp = kbg_ % S::SP;
    const uint32_t php = (uint32_t)((kbg_ / S::SP) & 1);
    if (!TQ_WAIT(7, mbar_wait(full_p(sp), php, abort_flag, 0x80000u))) return false;
    if (!TQ_WAIT(8, mbar_wait(empty_u(s), par_of(q) ^ 1u, abort_flag, 0x100000u))) return false;
    tc_fence_after();
    const unsigned char* src = sm + S::STAGE_OFF + sp * S::STAGE;
    unsigned char* dst = sm + s * S::SLOT + S::B_OFF;
#pragma unroll
    for (int task = wtid; task < BN * 4; task += 128) {
      const int row = task >> 2, piece = task & 3;
      const uint4 w = *reinterpret_cast<const uint4*>(src + row * (G_BK / 2) + piece * 16);
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
      mbar_arrive(full_u(s));
      mbar_arrive(empty_p(sp));
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer, INT8 path
    // (packed INT4 weights -> staging, INT8 activations -> slot).  The bf16 weight rows have their own producer
    // (last warp): a producer blocks on the slot it is about to fill, and with a single one a busy bf16 slot
    // held back the next packed-weight load although its staging buffer was free.
    if (lane == 0) {
      int q = 0, sp = 0;
      uint32_t php = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const int mt = t % p.tiles_m, nt = t / p.tiles_m;
        for (int kb = 0; kb < p.kb_total; ++kb) {
          if (!(ok = TQ_WAIT(0, mbar_wait(empty_p(sp), php ^ 1u, abort_flag, 0x1000u)))) break;
          mbar_arrive_expect_tx(full_p(sp), S::STAGE);
          tma_load_2d(base + S::STAGE_OFF + sp * S::STAGE, &tmap_b4, kb * (G_BK / 2), nt * BN, full_p(sp));
          if (++sp == S::SP) {
            sp = 0;
            php ^= 1u;
          }
          const int s = slot_of(q);
          if (!(ok = TQ_WAIT(1, mbar_wait(empty_u(s), par_of(q) ^ 1u, abort_flag, 0x2000u)))) break;
          mbar_arrive_expect_tx(full_u(s), G_BM * 128);
          tma_load_2d(base + s * S::SLOT, &tmap_a8, kb * G_BK, mt * G_BM, full_u(s));
          q += has_tail ? 3 : 1;
        }
      }
    }
  } else if (warp == 6 + G_BUILD_WARPS) {
    // ------------------------------------------------------------------ TMA producer, bf16 weight rows
    if (lane == 0 && has_tail) {
      int q = 1;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const int nt = t / p.tiles_m;
        for (int kb = 0; kb < p.kb_total && ok; ++kb) {
          for (int h = 0; h < 2; ++h) {
            const int s = slot_of(q + h);
            if (!(ok = TQ_WAIT(2, mbar_wait(empty_u(s), par_of(q + h) ^ 1u, abort_flag, 0x4000u)))) break;
            mbar_arrive_expect_tx(full_u(s), BN * 128);
            tma_load_2d(base + s * S::SLOT + S::B_OFF, &tmap_w, kb * G_BK + h * 64, nt * BN, full_u(s));
          }
          q += 3;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_i8 = make_idesc_i8<BN>();
      constexpr uint32_t idesc_bf = make_idesc_bf16<BN>();
      int q = 0;
      uint32_t pha = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        if (!(ok = TQ_WAIT(3, mbar_wait(acc_empty, pha ^ 1u, abort_flag, 0x8000u)))) break;
        tc_fence_after();
        for (int kb = 0; kb < p.kb_total && ok; ++kb) {
          {
            const int s = slot_of(q);
            if (!(ok = TQ_WAIT(4, mbar_wait(full_u(s), par_of(q), abort_flag, 0x10000u)))) break;
            tc_fence_after();
            const uint32_t a_addr = base + s * S::SLOT, b_addr = a_addr + S::B_OFF;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_i8(tmem_base, make_smem_desc(a_addr + k * 32), make_smem_desc(b_addr + k * 32), idesc_i8,
                      (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit(empty_u(s));
            ++q;
          }
          if (has_tail) {
            for (int h = 0; h < 2; ++h) {
              const int s = slot_of(q);
              if (!(ok = TQ_WAIT(5, mbar_wait(full_u(s), par_of(q), abort_flag, 0x20000u)))) break;
              tc_fence_after();
              const uint32_t a_addr = base + s * S::SLOT, b_addr = a_addr + S::B_OFF;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_bf16(tmem_base + BN, make_smem_desc(a_addr + k * 32), make_smem_desc(b_addr + k * 32), idesc_bf,
                          (kb > 0 || h > 0 || k > 0) ? 1u : 0u);
              umma_commit(empty_u(s));
              ++q;
            }
          }
        }
        if (!ok) break;
        umma_commit(acc_full);
        pha ^= 1u;
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ wideners + epilogue
    // These four warps widen the INT4 weight tiles of a tile's K slices, then drain its accumulators.
    // (The tensor memory holds one accumulator set, so the next tile's MMAs wait for the epilogue anyway.)
    const int quad = warp & 3;
    const int etid = threadIdx.x - 2 * 32;  // 0..127
    uint32_t pha = 0;
    bool ok = true;
    int wq = 0, kbg = 0;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      const int mt = t % p.tiles_m, nt = t / p.tiles_m;
      for (int kb = 0; kb < p.kb_total && ok; ++kb, ++kbg) {
        ok = widen(wq, kbg, etid);
        wq += has_tail ? 3 : 1;
      }
      if (!ok) break;
      if (!(ok = TQ_WAIT(6, mbar_wait(acc_full, pha, abort_flag, 0x40000u)))) break;
      tc_fence_after();
      const int row = mt * G_BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const float sx = row_ok ? p.sx[row] : 0.0f;
      const size_t rowoff = (size_t)row * p.N;
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t ri[32], rf[32];
        __syncwarp();
        tmem_ld32(lane_addr + (uint32_t)c0, ri);
        if (has_tail) {
          tmem_ld32(lane_addr + (uint32_t)(BN + c0), rf);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) rf[i] = 0u;
        }
        const int n0 = nt * BN + c0;
        if (!row_ok || n0 >= p.N) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + 8 * j;
          if (n < p.N) {
            float d[8];
            const float4 w0 = *reinterpret_cast<const float4*>(p.sw + n);
            const float4 w1 = *reinterpret_cast<const float4*>(p.sw + n + 4);
            const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float dense = __fmul_rn(__fmul_rn((float)((int)ri[8 * j + i] >> 4), sx), ws[i]);
              d[i] = has_tail ? __fadd_rn(dense, __uint_as_float(rf[8 * j + i])) : dense;
            }
            if (p.bias) {
              const float4 b0 = *reinterpret_cast<const float4*>(p.bias + n);
              const float4 b1 = *reinterpret_cast<const float4*>(p.bias + n + 4);
              const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) d[i] = __fadd_rn(d[i], bs[i]);
            }
            if (ACT) {
              uint2 o;
              o.x = swiglu_bf16_bits(d[0], d[1]) | (swiglu_bf16_bits(d[2], d[3]) << 16);
              o.y = swiglu_bf16_bits(d[4], d[5]) | (swiglu_bf16_bits(d[6], d[7]) << 16);
              *reinterpret_cast<uint2*>(p.out + ((size_t)row * p.N + n) / 2) = o;
            } else {
              uint4 o;
              o.x = f32_to_bf16_bits(d[0]) | (f32_to_bf16_bits(d[1]) << 16);
              o.y = f32_to_bf16_bits(d[2]) | (f32_to_bf16_bits(d[3]) << 16);
              o.z = f32_to_bf16_bits(d[4]) | (f32_to_bf16_bits(d[5]) << 16);
              o.w = f32_to_bf16_bits(d[6]) | (f32_to_bf16_bits(d[7]) << 16);
              *reinterpret_cast<uint4*>(p.out + rowoff + n) = o;
            }
            if (p.dbg_acc) {
              *reinterpret_cast<int4*>(p.dbg_acc + rowoff + n) =
                  make_int4((int)ri[8 * j] >> 4, (int)ri[8 * j + 1] >> 4, (int)ri[8 * j + 2] >> 4, (int)ri[8 * j + 3] >> 4);
              *reinterpret_cast<int4*>(p.dbg_acc + rowoff + n + 4) =
                  make_int4((int)ri[8 * j + 4] >> 4, (int)ri[8 * j + 5] >> 4, (int)ri[8 * j + 6] >> 4, (int)ri[8 * j + 7] >> 4);
            }
            if (p.dbg_tail) {
              *reinterpret_cast<uint4*>(p.dbg_tail + rowoff + n) = make_uint4(rf[8 * j], rf[8 * j + 1], rf[8 * j + 2], rf[8 * j + 3]);
              *reinterpret_cast<uint4*>(p.dbg_tail + rowoff + n + 4) = make_uint4(rf[8 * j + 4], rf[8 * j + 5], rf[8 * j + 6], rf[8 * j + 7]);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(acc_empty);
      pha ^= 1u;
    }
  } else if (warp < 6 + G_BUILD_WARPS) {
    // ------------------------------------------------------------------ tail builders
    // 256 threads = 128 rows x the two 64-wide halves of a K slice: each builds its row of the zero-filled
    // bf16 tail tile of that half.  The row's entries of a half slice come as one record of TQ_TAIL_REC_CAP words
    // ([half slice][row][j]: 128-bit loads), fetched two slices ahead; a word already holds the swizzled
    // position of the value inside the 128-byte tile row.
    if (has_tail) {
      constexpr int C = TQ_TAIL_REC_CAP;
      const int btid = threadIdx.x - 6 * 32;
      const int brow = btid & 127, half = btid >> 7;
      const uint32_t roff = (uint32_t)((brow >> 3) * 1024 + (brow & 7) * 128);
      bool ok = true;
      int q = 1 + half;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const int mt = t % p.tiles_m;
        const int grow = mt * G_BM + brow;
        // records / counts of this thread's 64-wide half of every K slice of the tile
        const uint32_t* recb = p.rec + (((size_t)mt * 2 * p.kb_total + half) * 128 + brow) * C;
        const uint16_t* cntb = p.cnt + ((size_t)mt * 2 * p.kb_total + half) * 128 + brow;
        auto load_cnt = [&](int kb) -> int {  // (rows at or beyond M of a partial last tile have zero counts)
          uint32_t n16 = 0u;
          if (kb < p.kb_total) asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(n16) : "l"(cntb + (size_t)kb * 256));
          return (int)n16;
        };
        // `npre` holds the count of slice kb (loaded two fetches ago): only existing records are loaded; the
        // count of slice kb + 2 is requested for the next fetch into this register set
        auto fetch = [&](uint32_t(&r)[C], int& n, int& npre, int kb) {
          n = npre;
          const uint4* rv = reinterpret_cast<const uint4*>(recb + (size_t)kb * 2 * 128 * C);
#pragma unroll
          for (int j = 0; j < C / 4; ++j)
            if (4 * j < n)
              asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(r[4 * j]), "=r"(r[4 * j + 1]), "=r"(r[4 * j + 2]), "=r"(r[4 * j + 3])
                           : "l"(rv + j));
          npre = load_cnt(kb + 2);
        };
        auto fill = [&](int kb, const uint32_t(&r)[C], int n) -> bool {
          const int s = slot_of(q);
          if (!TQ_WAIT(9, mbar_wait(empty_u(s), par_of(q) ^ 1u, abort_flag, 0x200000u))) return false;
          tc_fence_after();
          unsigned char* arow = sm + s * S::SLOT + roff;
          const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(arow + ((c ^ (brow & 7)) << 4)) = z;
          const int nmax = __reduce_max_sync(0xffffffffu, min(n, C));  // warp-uniform trip count
#pragma unroll
          for (int j = 0; j < C; ++j) {
            if (j < nmax) {
              if (j < n) *reinterpret_cast<uint16_t*>(arow + ((r[j] & 63u) << 1)) = (uint16_t)(r[j] >> 16);
            }
          }
          if (n > C) {  // a run longer than the record: the rest comes from the row's sorted list, 8 entries a load
            const size_t lrow = (size_t)grow;
            int e0 = (int)__ldg(p.ptr + lrow * p.ptr_ld + kb);
            if (half) e0 += (int)__ldg(cntb - 128 + (size_t)kb * 256);  // entries of the slice's first half
            const int lo = e0 + C, hi = e0 + n;  // list positions [lo, hi)
            const int kb0 = kb * G_BK + 64 * half;
            if ((p.ld & 7) == 0 && ((reinterpret_cast<uintptr_t>(p.idx) | reinterpret_cast<uintptr_t>(p.val)) & 15) == 0) {
              const uint4* irow = reinterpret_cast<const uint4*>(p.idx + lrow * p.ld);
              const uint4* vrow = reinterpret_cast<const uint4*>(p.val + lrow * p.ld);
              for (int g8 = lo >> 3; g8 <= (hi - 1) >> 3; ++g8) {
                const uint4 gi = __ldg(irow + g8), gv = __ldg(vrow + g8);
                const uint32_t wi[4] = {gi.x, gi.y, gi.z, gi.w}, wv[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                  const int e = g8 * 8 + u;
                  const int c = (int)((wi[u >> 1] >> ((u & 1) * 16)) & 0xffffu) - kb0;
                  if (e >= lo && e < hi && c >= 0 && c < 64)
                    *reinterpret_cast<uint16_t*>(arow + (((c >> 3) ^ (brow & 7)) << 4) + (c & 7) * 2) =
                        (uint16_t)(wv[u >> 1] >> ((u & 1) * 16));
                }
              }
            } else {
              for (int e = lo; e < hi; ++e) {
                const int c = (int)__ldg(p.idx + lrow * p.ld + e) - kb0;
                if (c >= 0 && c < 64)
                  *reinterpret_cast<uint16_t*>(arow + (((c >> 3) ^ (brow & 7)) << 4) + (c & 7) * 2) =
                      __ldg(p.val + lrow * p.ld + e);
              }
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(full_u(s));
          q += 3;
          return true;
        };
        uint32_t ra[C], rb[C];
        int na = 0, nb = 0, npa = load_cnt(0), npb = load_cnt(1);
        fetch(ra, na, npa, 0);
        fetch(rb, nb, npb, 1);
        for (int kb = 0; kb < p.kb_total && ok; kb += 2) {
          ok = fill(kb, ra, na);
          if (!ok) break;
          fetch(ra, na, npa, kb + 2);
          if (kb + 1 < p.kb_total) {
            ok = fill(kb + 1, rb, nb);
            if (!ok) break;
            fetch(rb, nb, npb, kb + 3);
          }
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

template <int BN, int ACT>
int launch_split_gemm(const int8_t* a_q8, const uint8_t* b_col, const void* w_rot, SplitGemmParams p, cudaStream_t st) {
  using S = GS<BN>;
  auto kern = split_gemm_kernel<BN, ACT>;
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
  CUtensorMap ma, mb, mw;
  if (!make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_q8, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)p.K, 128,
                          G_BM, true))
    return TQ_ERR_CUDA;
  if (!make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_col, (uint64_t)(p.K / 2), (uint64_t)p.N,
                          (uint64_t)(p.K / 2), G_BK / 2, BN))
    return TQ_ERR_CUDA;
  // without a tail the bf16 map is never used; point it at the packed weights to keep it valid
  const void* wsrc = p.has_tail ? w_rot : (const void*)b_col;
  if (!make_tensor_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, wsrc, (uint64_t)(p.has_tail ? p.K : p.K / 4),
                          (uint64_t)p.N, (uint64_t)(p.has_tail ? p.K * 2 : p.K / 2), 64, BN, true))
    return TQ_ERR_CUDA;
  p.tiles_m = (p.M + G_BM - 1) / G_BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.kb_total = p.K / G_BK;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = p.tiles_m * p.tiles_n;
  const int grid = total < sms ? total : sms;
  kern<<<grid, G_THREADS, S::DYN, st>>>(ma, mb, mw, p);
  return check_launch();
}

}  // namespace
}  // namespace tq

namespace tq {
// -1 = choose by shape, 0 = one-CTA kernel, 1 = CTA-pair kernel (set by tq_set_gemm_pair_mode only)
static int g_gemm_pair_mode = -1;
int run_pair_gemm(const int8_t* a_q8, const float* body_scale, const uint8_t* b_col, const float* w_scale,
                  const void* w_rot, const uint16_t* tail_idx16, const void* tail_val, int tail_ld,
                  const uint16_t* tail_ptr, int ptr_ld, const uint32_t* tail_rec, const uint16_t* tail_cnt,
                  const void* tail_dense, int R, const float* bias, void* out_bf16, int32_t* dbg_acc, float* dbg_tail,
                  int M, int N, int K, int act, cudaStream_t st);
}

#ifdef TQ_GEMM_PROFILE
extern "C" int tq_gemm_wait_cycles(unsigned long long* out16, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out16, tq::g_wait_cycles, sizeof(unsigned long long) * 16);
  if (reset) {
    unsigned long long z[16] = {};
    cudaMemcpyToSymbol(tq::g_wait_cycles, z, sizeof(z));
  }
  return 0;
}
#endif

#ifdef TQ_GEMM_TRACE
extern "C" int tq_gemm_trace(unsigned long long* out, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, tq::g_trace, sizeof(unsigned long long) * 8 * 128 * 4);
  if (reset) {
    static unsigned long long z[8 * 128 * 4] = {};
    cudaMemcpyToSymbol(tq::g_trace, z, sizeof(z));
  }
  return 0;
}
#endif

extern "C" int tq_set_gemm_pair_mode(int mode) {
  if (mode < -1 || mode > 1) return TQ_ERR_BAD_ARG;
  tq::g_gemm_pair_mode = mode;
  return TQ_OK;
}

namespace tq {
static int run_split_gemm_mma(const int8_t* a_q8, const float* body_scale, const uint8_t* b_col,
                              const float* w_scale, const void* w_rot, const uint16_t* tail_idx16,
                              const void* tail_val, int tail_ld, const uint16_t* tail_ptr, int ptr_ld,
                              const uint32_t* tail_rec, const uint16_t* tail_cnt, const void* tail_dense, int R,
                              const float* bias, void* out_bf16, int32_t* dbg_acc, float* dbg_tail, int M, int N, int K,
                              int act, void* stream) {
  if (!a_q8 || !body_scale || !b_col || !w_scale || !out_bf16 || M < 0 || N <= 0 || K <= 0 || R < 0 || R >= K)
    return TQ_ERR_BAD_ARG;
  if (R > 0 && (!w_rot || !tail_idx16 || !tail_val || tail_ld < R || !tail_ptr || ptr_ld < K / G_BK + 1 || !tail_rec ||
                !tail_cnt))
    return TQ_ERR_BAD_ARG;
  if (K % G_BK != 0 || N % 8 != 0 || K > 65536) return TQ_ERR_UNSUPPORTED;
  if (!aligned16(a_q8) || !aligned16(b_col) || !aligned16(out_bf16) || !aligned16(w_scale) ||
      (R > 0 && !aligned16(w_rot)) || (bias && !aligned16(bias)) || (dbg_acc && !aligned16(dbg_acc)) ||
      (dbg_tail && !aligned16(dbg_tail)))
    return TQ_ERR_MISALIGNED;
  if (M == 0) return TQ_OK;
  {
    // Choice between the one-CTA kernel (128 x 256 tiles) and the CTA-pair kernel (256 x 256 tiles, half the B
    // traffic per CTA), from timings over M = 256..8192 on the Qwen3-8B and Llama-3-8B layer shapes: the pair
    // kernel is 1.7-2x faster without a tail and 10-40 % faster with one, except for problems of at most 74
    // one-CTA tiles (half a wave), where a tile's latency decides and the one-CTA kernel is 7-12 % ahead.
    // tq_set_gemm_pair_mode(0 / 1) forces one of them.
    const long tiles_single = (long)((M + 127) / 128) * ((N + 255) / 256);
    const bool pair = g_gemm_pair_mode == 1 || (g_gemm_pair_mode < 0 && (R == 0 || tiles_single > 74));
    if (pair)
      return run_pair_gemm(a_q8, body_scale, b_col, w_scale, w_rot, tail_idx16, tail_val, tail_ld, tail_ptr, ptr_ld,
                           tail_rec, tail_cnt, tail_dense, R, bias, out_bf16, dbg_acc, dbg_tail, M, N, K, act,
                           (cudaStream_t)stream);
  }
  // (the one-CTA kernel serves small problems and always walks the row's list for runs longer than a record)
  SplitGemmParams p = {};
  p.act = act;
  p.M = M;
  p.N = N;
  p.K = K;
  p.R = R;
  p.ld = tail_ld;
  p.ptr_ld = ptr_ld;
  p.ptr = tail_ptr;
  p.rec = tail_rec;
  p.cnt = tail_cnt;
  p.has_tail = R > 0 ? 1 : 0;
  p.idx = tail_idx16;
  p.val = reinterpret_cast<const uint16_t*>(tail_val);
  p.sx = body_scale;
  p.sw = w_scale;
  p.bias = bias;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.dbg_acc = dbg_acc;
  p.dbg_tail = dbg_tail;
  const long tiles256 = (long)((M + G_BM - 1) / G_BM) * ((N + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (tiles256 >= 148)
    return act ? launch_split_gemm<256, 1>(a_q8, b_col, w_rot, p, st) : launch_split_gemm<256, 0>(a_q8, b_col, w_rot, p, st);
  return act ? launch_split_gemm<128, 1>(a_q8, b_col, w_rot, p, st) : launch_split_gemm<128, 0>(a_q8, b_col, w_rot, p, st);
}
}  // namespace tq

extern "C" int tq_split_gemm_mma(const int8_t* a_q8, const float* body_scale, const uint8_t* b_col,
                                 const float* w_scale, const void* w_rot, const uint16_t* tail_idx16,
                                 const void* tail_val, int tail_ld, const uint16_t* tail_ptr, int ptr_ld,
                                 const uint32_t* tail_rec, const uint16_t* tail_cnt, const void* tail_dense, int R,
                                 const float* bias, void* out_bf16,
                                 int32_t* dbg_acc, float* dbg_tail, int M, int N, int K, void* stream) {
  return tq::run_split_gemm_mma(a_q8, body_scale, b_col, w_scale, w_rot, tail_idx16, tail_val, tail_ld, tail_ptr,
                                ptr_ld, tail_rec, tail_cnt, tail_dense, R, bias, out_bf16, dbg_acc, dbg_tail, M, N, K, 0,
                                stream);
}

extern "C" int tq_split_gemm_mma_swiglu(const int8_t* a_q8, const float* body_scale, const uint8_t* b_col,
                                        const float* w_scale, const void* w_rot, const uint16_t* tail_idx16,
                                        const void* tail_val, int tail_ld, const uint16_t* tail_ptr, int ptr_ld,
                                        const uint32_t* tail_rec, const uint16_t* tail_cnt, const void* tail_dense,
                                        int R, const float* bias, void* out_bf16, int M, int N, int K, void* stream) {
  return tq::run_split_gemm_mma(a_q8, body_scale, b_col, w_scale, w_rot, tail_idx16, tail_val, tail_ld, tail_ptr,
                                ptr_ld, tail_rec, tail_cnt, tail_dense, R, bias, out_bf16, nullptr, nullptr, M, N, K, 1,
                                stream);
}
