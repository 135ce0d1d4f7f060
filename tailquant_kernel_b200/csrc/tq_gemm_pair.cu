// Split GEMM on CTA pairs (sm_100a): the same computation as tq_gemm_tail.cu -- dense INT4 x INT4 part on tcgen05
// kind::i8, tail as a bf16 tcgen05 product over the zero-filled tail tile, one fused epilogue -- but two CTAs of a
// cluster share one 256 x 256 output tile: tcgen05.mma.cta_group::2 with M = 256.
//
// Why pairs: at M = 2048 these GEMMs are bound by the L2 -> SM bandwidth (see the profile summaries), and the B
// operands dominate the traffic (INT4 weights + bf16 weight rows).  In a pair each CTA loads only ITS half of the
// B tile (128 of the 256 output channels) and its own 128 rows of A; the tensor cores of both SMs read both
// halves.  Per 128-wide K slice a CTA then loads 16 KB + 8 KB + 32 KB (+ 8 KB records) instead of
// 16 KB + 16 KB + 64 KB (+ 8 KB).  Smaller slots also leave room for six of them.
//
// Protocol (rank 0 = leader issues every MMA):
//   * every "slot full" barrier that the MMA issuer waits on lives in the LEADER; the other CTA's wideners and
//     tail builders arrive on it through its shared::cluster address, and both CTAs' TMA loads count their bytes
//     on it (cta_group::2 form of the tiled load; each CTA loads its own tiles, nothing is broadcast);
//   * "slot empty" and "accumulator full" are signalled to both CTAs by one tcgen05.commit;
//   * "accumulator empty" collects the epilogue threads of both CTAs in the leader;
//   * tensor memory is allocated / freed by warp 1 of both CTAs with the cta_group::2 forms; the kernel starts
//     and ends with a cluster-wide barrier so that no CTA touches a peer that has not started or has left.
// Every mbarrier wait is bounded as in the one-CTA kernel.
#include "tq_common.cuh"
#include "tq_ptx.cuh"

namespace tq {
namespace {

constexpr int P_BM = 128;  // rows of A per CTA (256 per pair)
constexpr int P_BK = 128;
constexpr int P_BUILD_WARPS = 8;
// warp 0: packed-weight producer, 1: MMA issuer, 2..5: wideners, 6..13: tail builders, 14: INT8 activation
// producer, 15: bf16 weight-row producer.  Warps 2..13 share the epilogue.
constexpr int P_THREADS = (6 + P_BUILD_WARPS + 2) * 32;
constexpr int P_LOOK = 2;  // K slices of the next tile prepared before a tile's epilogue

struct PairGemmParams {
  int M, N, K, R, ld, ptr_ld;
  int tiles_m, tiles_n, kb_total, has_tail;
  int dense;             // the zero-filled tail matrix is available (tmap_d): half slices with long runs load it
  const uint16_t* idx;   // [M, ld] ascending tail indices (only read for runs longer than the record capacity)
  const uint16_t* val;   // [M, ld] tail values
  const uint16_t* ptr;   // [M, ptr_ld] ptr[m][j] = entries of row m with index < 128 j
  const uint32_t* rec;   // [2 tiles_m][K/64][128][TQ_TAIL_REC_CAP]: tile position | bf16 << 16 (see tq_split_prologue)
  const uint16_t* cnt;   // [2 tiles_m][K/64][128]: entries of the row in the 64-wide half slice (0 for rows >= M)
  const float* sx;
  const float* sw;
  const float* bias;
  __nv_bfloat16* out;
  int32_t* dbg_acc;   // optional [M,N]: the int32 accumulators
  float* dbg_tail;    // optional [M,N]: the fp32 tail sums
};

constexpr int P_BN = 256;         // output channels per pair tile
constexpr int P_BH = P_BN / 2;    // B rows (output channels) loaded by each CTA

struct PS {
  static constexpr int SU = 6;                            // operand slots
  static constexpr int SP = 4;                            // packed-weight staging buffers
  static constexpr int SLOT = (P_BM + P_BH) * 128;        // A region (16 KB) then this CTA's half of B (16 KB)
  static constexpr int B_OFF = P_BM * 128;
  static constexpr int STAGE = P_BH * (P_BK / 2);
  static constexpr int STAGE_OFF = SU * SLOT;
  static constexpr int BAR_OFF = STAGE_OFF + SP * STAGE;
  static constexpr int NUM_BARS = 2 * SP + 2 * SU + 4;  // + accumulator full / empty, two buffers each
  static constexpr int DYN = BAR_OFF + NUM_BARS * 8 + 16 + 1024;
};
static_assert(PS::DYN <= 232448, "shared memory of the pair kernel");

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int ACT>  // 0: out [M, N]; 1: SwiGLU over interleaved (gate, up) channel pairs, out [M, N/2]
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
pair_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a8, const __grid_constant__ CUtensorMap tmap_b4,
                  const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_d,
                  const PairGemmParams p) {
  using S = PS;
  constexpr int BN = P_BN;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_dyn + (base - raw);

  const uint32_t bars = base + S::BAR_OFF;
  auto full_p = [&](int s) { return bars + 8u * s; };
  auto empty_p = [&](int s) { return bars + 8u * (S::SP + s); };
  auto full_u = [&](int s) { return bars + 8u * (2 * S::SP + s); };
  auto empty_u = [&](int s) { return bars + 8u * (2 * S::SP + S::SU + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * S::SP + 2 * S::SU + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * S::SP + 2 * S::SU + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + S::BAR_OFF + S::NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + S::BAR_OFF + S::NUM_BARS * 8 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int total_tiles = p.tiles_m * p.tiles_n;    // 256 x 256 pair tiles
  const int my_tiles = pair < total_tiles ? (total_tiles - pair + npairs - 1) / npairs : 0;  // tiles pair, pair + npairs, ...
  const int kbt = p.kb_total;
  const int G = my_tiles * kbt;                     // K slices this pair goes through, over all its tiles
  const int look = kbt < P_LOOK ? kbt : P_LOOK;
  auto lead = [&](uint32_t bar) { return map_to_cta(bar, 0u); };  // the leader's barrier at this offset
  const bool has_tail = p.has_tail != 0;
  const int uses = has_tail ? 3 : 1;                // slot uses per K slice: INT8 operands, then two bf16 halves
  constexpr uint32_t TMEM_COLS = 2 * BN;  // int32 accumulator, then fp32 tail accumulator

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_a8)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_b4)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_d)) : "memory");
    for (int s = 0; s < S::SP; ++s) {
      mbar_init(full_p(s), 1);
      mbar_init(empty_p(s), 4);
    }
    for (int s = 0; s < S::SU; ++s) {
      mbar_init(full_u(s), 8 + 1);  // four warps of each CTA + the leader producer's expect_tx (leader's copy is used)
      mbar_init(empty_u(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      // the epilogue warps of both CTAs (leader's copy is used): all twelve with a tail, warps 10..13 without
      mbar_init(acc_empty(b), p.has_tail ? 2 * (4 + P_BUILD_WARPS) : 2 * 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();  // both CTAs have initialised their barriers before anyone arrives on a peer's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // slot use number q -> (slot, parity)
  auto slot_of = [](int q) { return q % S::SU; };
  auto par_of = [](int q) { return (uint32_t)((q / S::SU) & 1); };
  // local tile number i -> tile coordinates
  auto tile_mt = [&](int i) { return (pair + i * npairs) % p.tiles_m; };
  auto tile_nt = [&](int i) { return (pair + i * npairs) / p.tiles_m; };

  // Epilogue share of one warp (2..13) for local tile i: column chunks [c_lo, c_hi) of 32 channels each, rows of
  // the warp's tensor-memory lane quadrant.  y = bf16((float(acc) * s_x) * s_w + tail + bias).
  // Accumulator buffers: with a tail the int32 and the fp32 accumulator fill the tensor memory (one set; a tile's
  // MMAs wait for the previous epilogue).  Without a tail the second half holds a second int32 accumulator: tile
  // i uses buffer i & 1, and its epilogue (warps 10..13) runs under the next tile's main loop.
  auto acc_buf = [&](int i) { return has_tail ? 0 : (i & 1); };
  auto acc_use = [&](int i) { return has_tail ? i : (i >> 1); };
  auto epilogue = [&](int i, int c_lo, int c_hi) -> bool {
    const int ab = acc_buf(i);
    if (!TQ_WAIT(6, mbar_wait(acc_full(ab), (uint32_t)(acc_use(i) & 1), abort_flag, 0x40000u))) return false;
    tc_fence_after();
    const int mt = tile_mt(i), nt = tile_nt(i);
    const int quad = warp & 3;
    const int row = (2 * mt + (int)rank) * P_BM + quad * 32 + lane;
    const bool row_ok = row < p.M;
    const float sx = row_ok ? p.sx[row] : 0.0f;
    const size_t rowoff = (size_t)row * p.N;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ab * BN);
#pragma unroll 1
    for (int c = c_lo; c < c_hi; ++c) {
      const int c0 = c * 32;
      uint32_t ri[32], rf[32];
      __syncwarp();
      tmem_ld32(lane_addr + (uint32_t)c0, ri);
      if (has_tail) {
        tmem_ld32(lane_addr + (uint32_t)(BN + c0), rf);
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) rf[k] = 0u;
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
          for (int k = 0; k < 8; ++k) {
            const float dense = __fmul_rn(__fmul_rn((float)((int)ri[8 * j + k] >> 4), sx), ws[k]);
            d[k] = has_tail ? __fadd_rn(dense, __uint_as_float(rf[8 * j + k])) : dense;
          }
          if (p.bias) {
            const float4 b0 = *reinterpret_cast<const float4*>(p.bias + n);
            const float4 b1 = *reinterpret_cast<const float4*>(p.bias + n + 4);
            const float bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) d[k] = __fadd_rn(d[k], bs[k]);
          }
          if (ACT) {
            uint2 o;
            o.x = swiglu_bf16_bits(d[0], d[1]) | (swiglu_bf16_bits(d[2], d[3]) << 16);
            o.y = swiglu_bf16_bits(d[4], d[5]) | (swiglu_bf16_bits(d[6], d[7]) << 16);
            *reinterpret_cast<uint2*>(p.out + ((size_t)row * p.N + n) / 2) = o;
          } else {
            uint4 o;
            o.x = pack_bf16x2(d[0], d[1]);
            o.y = pack_bf16x2(d[2], d[3]);
            o.z = pack_bf16x2(d[4], d[5]);
            o.w = pack_bf16x2(d[6], d[7]);
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
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(lead(acc_empty(ab)));
    return true;
  };
  // the eight 32-channel chunks of a tile are split 3 / 3 / 2 over the three warps of a lane quadrant
  // (without a tail warps 10..13 take all eight chunks and the others none)
  const int ethird = (warp - 2) >> 2;
  const int c_lo = has_tail ? ethird * 3 : 0, c_hi = has_tail ? (ethird == 2 ? 8 : ethird * 3 + 3) : 8;
  bool ok = true;
  int epi_done = 0;  // tiles whose epilogue share this warp has done
  auto catch_up = [&](int upto) {
    while (ok && epi_done < upto) ok = epilogue(epi_done++, c_lo, c_hi);
  };
  // INT4 -> INT8 (x16) of K slice g's weight tile by four warps (wtid = 0..127): staging buffer -> B region of
  // the slice's INT8 slot.  One group of four warps sees every phase of the staging barriers it waits on.
  auto widen_one = [&](int g, int wtid) -> bool {
    const int q = g * uses, s = slot_of(q), sp = g % S::SP;
    const uint32_t php = (uint32_t)((g / S::SP) & 1);
    if (wtid == 0) TQ_TRACE(3, q, 0);
    if (!TQ_WAIT(7, mbar_wait(full_p(sp), php, abort_flag, 0x80000u))) return false;
    if (wtid == 0) TQ_TRACE(3, q, 1);
    if (!TQ_WAIT(8, mbar_wait(empty_u(s), par_of(q) ^ 1u, abort_flag, 0x100000u))) return false;
    if (wtid == 0) TQ_TRACE(3, q, 2);
    tc_fence_after();
    const unsigned char* src = sm + S::STAGE_OFF + sp * S::STAGE;
    unsigned char* dst = sm + s * S::SLOT + S::B_OFF;
#pragma unroll
    for (int task = wtid; task < P_BH * 4; task += 128) {
      const int row = task >> 2, piece = task & 3;
      const uint4 w = *reinterpret_cast<const uint4*>(src + row * (P_BK / 2) + piece * 16);
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
      mbar_arrive_cluster(lead(full_u(s)));
      mbar_arrive(empty_p(sp));
    }
    if (wtid == 0) TQ_TRACE(3, q, 3);
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer: packed INT4 weights
    if (lane == 0) {
      for (int g = 0; g < G; ++g) {
        const int sp = g % S::SP;
        const uint32_t php = (uint32_t)((g / S::SP) & 1);
        TQ_TRACE(6, g * uses, 0);
        if (!TQ_WAIT(0, mbar_wait(empty_p(sp), php ^ 1u, abort_flag, 0x1000u))) break;
        TQ_TRACE(6, g * uses, 1);
        const int i = g / kbt, kb = g - i * kbt;
        mbar_arrive_expect_tx(full_p(sp), S::STAGE);
        tma_load_2d(base + S::STAGE_OFF + sp * S::STAGE, &tmap_b4, kb * (P_BK / 2), tile_nt(i) * BN + (int)rank * P_BH,
                    full_p(sp));
      }
    }
  } else if (warp == 6 + P_BUILD_WARPS) {
    // ------------------------------------------------------------------ TMA producer: INT8 activations
    if (lane == 0) {
      for (int g = 0; g < G; ++g) {
        const int q = g * uses, s = slot_of(q);
        TQ_TRACE(1, q, 0);
        if (!TQ_WAIT(1, mbar_wait(empty_u(s), par_of(q) ^ 1u, abort_flag, 0x2000u))) break;
        TQ_TRACE(1, q, 1);
        const int i = g / kbt, kb = g - i * kbt;
        if (rank == 0) mbar_arrive_expect_tx(full_u(s), 2 * P_BM * 128);  // the A tiles of both CTAs
        tma_load_2d_pair(base + s * S::SLOT, &tmap_a8, kb * P_BK, (2 * tile_mt(i) + (int)rank) * P_BM, lead(full_u(s)));
        TQ_TRACE(1, q, 2);
      }
    }
  } else if (warp == 6 + P_BUILD_WARPS + 1) {
    // ------------------------------------------------------------------ TMA producer: bf16 weight rows
    if (lane == 0 && has_tail) {
      bool ok = true;
      for (int g = 0; g < G && ok; ++g) {
        const int i = g / kbt, kb = g - i * kbt;
        const int nrow = tile_nt(i) * BN + (int)rank * P_BH;
        for (int h = 0; h < 2; ++h) {
          const int q = 3 * g + 1 + h, s = slot_of(q);
          TQ_TRACE(2, q, 0);
          if (!(ok = TQ_WAIT(2, mbar_wait(empty_u(s), par_of(q) ^ 1u, abort_flag, 0x4000u)))) break;
          TQ_TRACE(2, q, 1);
          if (rank == 0) mbar_arrive_expect_tx(full_u(s), BN * 128);  // both halves of the bf16 B tile
          tma_load_2d_pair(base + s * S::SLOT + S::B_OFF, &tmap_w, kb * P_BK + h * 64, nrow, lead(full_u(s)));
          TQ_TRACE(2, q, 2);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_i8 = make_idesc_i8<BN, 256>();
      constexpr uint32_t idesc_bf = make_idesc_bf16<BN, 256>();
      int q = 0;
      bool ok = true;
      for (int i = 0; ok && i < my_tiles; ++i) {
        const int ab = acc_buf(i);
        const uint32_t acc_tmem = tmem_base + (uint32_t)(ab * BN);
        if (!(ok = TQ_WAIT(3, mbar_wait(acc_empty(ab), (uint32_t)(acc_use(i) & 1) ^ 1u, abort_flag, 0x8000u)))) break;
        tc_fence_after();
        for (int kb = 0; kb < kbt && ok; ++kb) {
          {
            const int s = slot_of(q);
            TQ_TRACE(0, q, 0);
            if (!(ok = TQ_WAIT(4, mbar_wait(full_u(s), par_of(q), abort_flag, 0x10000u)))) break;
            TQ_TRACE(0, q, 1);
            tc_fence_after();
            const uint32_t a_addr = base + s * S::SLOT, b_addr = a_addr + S::B_OFF;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_i8_pair(acc_tmem, make_smem_desc(a_addr + k * 32), make_smem_desc(b_addr + k * 32), idesc_i8,
                      (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit_pair(empty_u(s));
            TQ_TRACE(0, q, 2);
            ++q;
          }
          if (has_tail) {
            for (int h = 0; h < 2; ++h) {
              const int s = slot_of(q);
              TQ_TRACE(0, q, 0);
              if (!(ok = TQ_WAIT(5, mbar_wait(full_u(s), par_of(q), abort_flag, 0x20000u)))) break;
              TQ_TRACE(0, q, 1);
              tc_fence_after();
              const uint32_t a_addr = base + s * S::SLOT, b_addr = a_addr + S::B_OFF;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_bf16_pair(tmem_base + BN, make_smem_desc(a_addr + k * 32), make_smem_desc(b_addr + k * 32), idesc_bf,
                          (kb > 0 || h > 0 || k > 0) ? 1u : 0u);
              umma_commit_pair(empty_u(s));
              TQ_TRACE(0, q, 2);
              ++q;
            }
          }
        }
        if (!ok) break;
        umma_commit_pair(acc_full(ab));
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ wideners (+ epilogue share)
    // INT4 -> INT8 (x16) of the pair's weight tiles, one K slice after the other over all its tiles.  The
    // epilogue of a tile is taken up once the first slices of the NEXT tile are widened, so that the MMAs
    // restart as soon as the accumulators are drained.  Without a tail these warps take the even slices and
    // four of the idle builder warps the odd ones.
    const int etid = threadIdx.x - 2 * 32;  // 0..127
    const int step = has_tail ? 1 : 2;
    for (int g = 0; g < G && ok; g += step) {
      if (!(ok = widen_one(g, etid))) break;
      const int i = g / kbt, kb = g - i * kbt;
      if (has_tail && (kb >= look - 1 || kb + step >= kbt)) catch_up(i);  // (second case: this group's last slice of the tile)
    }
    if (has_tail) catch_up(my_tiles);
  } else {
    // ------------------------------------------------------------------ tail builders (+ epilogue share)
    // 256 threads = 128 rows x the two 64-wide halves of a K slice: each builds its row of the zero-filled
    // bf16 tail tile of that half.  The row's entries of a half slice come as one record of TQ_TAIL_REC_CAP words
    // ([half slice][row][j]: 128-bit loads, a warp reads one contiguous run), fetched one slice ahead; a word
    // already holds the swizzled position of the value inside the 128-byte tile row.
    if (has_tail) {
      constexpr int C = TQ_TAIL_REC_CAP;
      const int btid = threadIdx.x - 6 * 32;
      const int brow = btid & 127, half = btid >> 7;
      const uint32_t roff = (uint32_t)((brow >> 3) * 1024 + (brow & 7) * 128);
      // records and count of this thread's 64-wide half of K slice g (g runs over all tiles of the pair), requested
      // right after the previous fill.  This kernel runs at the 128-register cap and its builders sit on the
      // critical path: ONE register set (a second set, or gating the loads on a count fetched earlier, spilled
      // and measured 10-40 % slower), all sixteen records requested whatever the count is.
      // (fi, fkb): local tile and slice of the NEXT slice to fetch, advanced without divisions -- this code runs
      // between two fills; fhs: its position in the record arrays.
      int fi = 0, fkb = 0;
      // (The record arrays cover 2 * ceil(M / 256) row tiles, and rows at or beyond M have zero counts: no bounds
      // checks here.)
      size_t fhs = my_tiles > 0 ? ((size_t)(2 * tile_mt(0) + (int)rank) * kbt) * 2 + half : 0;
      // The count of a half slice is requested one fetch ahead of its record (npre), so that the record's third
      // 128-bit word -- entries 8..11, needed by one row in two hundred -- is only loaded where it exists.
      auto load_cnt = [&](size_t hs) -> int {
        uint32_t n16;
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(n16) : "l"(p.cnt + hs * 128 + brow));
        return (int)n16;
      };
      int npre = my_tiles > 0 ? load_cnt(fhs) : 0;
      auto fetch = [&](uint32_t(&r)[C], int& n) {
        if (fi < my_tiles) {
          const uint4* recb = reinterpret_cast<const uint4*>(p.rec + (fhs * 128 + brow) * C);
          n = npre;
#pragma unroll
          for (int j = 0; j < C / 4; ++j)  // the row's record: C words in a row, a warp reads 32 C contiguous words
            if (j < 2 || n > 4 * j)
              asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(r[4 * j]), "=r"(r[4 * j + 1]), "=r"(r[4 * j + 2]), "=r"(r[4 * j + 3])
                           : "l"(recb + j));
          fhs += 2;
          if (++fkb == kbt) {  // next tile of the pair
            fkb = 0;
            ++fi;
            if (fi < my_tiles) fhs = ((size_t)(2 * tile_mt(fi) + (int)rank) * kbt) * 2 + half;
          }
          if (fi < my_tiles) npre = load_cnt(fhs);
        } else {
          n = 0;
        }
      };
      auto fill = [&](int g, const uint32_t(&r)[C], int n) -> bool {
        const int q = 3 * g + 1 + half, s = slot_of(q);
        if (brow == 0) TQ_TRACE(4, q, 0);
        if (!TQ_WAIT(9, mbar_wait(empty_u(s), par_of(q) ^ 1u, abort_flag, 0x200000u))) return false;
        if (brow == 0) TQ_TRACE(4, q, 1);
        tc_fence_after();
        const int nwmax = __reduce_max_sync(0xffffffffu, n);
        if (p.dense && nwmax > C) {
          // a run longer than the record among the warp's 32 rows and the zero-filled tail matrix at hand: its 32 x 64
          // block is the operand itself -- one tiled load (same 128-byte swizzle as the tile), whose bytes the slot's
          // barrier counts on top of this warp's arrival
          if (lane == 0) {
            const int i = g / kbt, kb = g - i * kbt;
            mbar_arrive_expect_tx_cluster(lead(full_u(s)), 32u * 128u);
            tma_load_2d_pair(base + s * S::SLOT + (uint32_t)(brow >> 5) * 4096u, &tmap_d, kb * P_BK + 64 * half,
                             (2 * tile_mt(i) + (int)rank) * P_BM + (brow & ~31), lead(full_u(s)));
          }
          return true;
        }
        unsigned char* arow = sm + s * S::SLOT + roff;
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(arow + ((c ^ (brow & 7)) << 4)) = z;
        if (brow == 0) TQ_TRACE(5, q, 2);
        const int nmax = min(nwmax, C);  // warp-uniform trip count
#pragma unroll
        for (int j = 0; j < C; ++j) {
          if (j < nmax) {
            if (j < n) *reinterpret_cast<uint16_t*>(arow + ((r[j] & 63u) << 1)) = (uint16_t)(r[j] >> 16);
          }
        }
        if (n > C) {  // a run longer than the record: the rest comes from the row's sorted list, 8 entries a load
          const int i = g / kbt, kb = g - i * kbt;
          const size_t lrow = (size_t)(2 * tile_mt(i) + (int)rank) * P_BM + brow;  // < M: other rows have zero counts
          int e0 = (int)__ldg(p.ptr + lrow * p.ptr_ld + kb);
          if (half)  // entries of the slice's first half
            e0 += (int)__ldg(p.cnt + (((size_t)(2 * tile_mt(i) + (int)rank) * kbt + kb) * 2) * 128 + brow);
          const int lo = e0 + C, hi = e0 + n;  // list positions [lo, hi)
          const int kb0 = kb * P_BK + 64 * half;
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
        if (brow == 0) TQ_TRACE(4, q, 3);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (brow == 0) TQ_TRACE(5, q, 0);
        __syncwarp();
        if (brow == 0) TQ_TRACE(5, q, 1);
        if (lane == 0) mbar_arrive_cluster(lead(full_u(s)));
        if (brow == 0) TQ_TRACE(4, q, 2);
        return true;
      };
      // a tile's epilogue share comes after the first slices of the next tile, as for the wideners
      int ci = 0, ckb = 0;  // local tile and slice of the slice just filled
      auto after = [&]() -> bool {
        if (ckb >= look - 1) catch_up(ci);
        if (++ckb == kbt) {
          ckb = 0;
          ++ci;
        }
        return ok;
      };
      uint32_t ra[C];
      int na = 0;
      fetch(ra, na);
      for (int g = 0; g < G && ok; ++g) {
        ok = fill(g, ra, na) && after();
        if (!ok) break;
        fetch(ra, na);
      }
      catch_up(my_tiles);
    } else {
      if (warp < 10) {  // warps 6..9: the odd K slices of the weight widening
        const int wtid = threadIdx.x - 6 * 32;
        for (int g = 1; g < G && ok; g += 2) {
          if (!(ok = widen_one(g, wtid))) break;
        }
      } else {
        catch_up(my_tiles);  // warps 10..13: the epilogues, each under the next tile's main loop
      }
    }
  }

  tc_fence_before();
  cluster_sync_all();  // the peer's MMAs, arrivals and loads are done with this CTA's memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int ACT>
int launch_pair_gemm(const int8_t* a_q8, const uint8_t* b_col, const void* w_rot, const void* tail_dense, PairGemmParams p,
                     cudaStream_t st) {
  using S = PS;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(dev < 64 && configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(pair_gemm_kernel<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::DYN);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return TQ_ERR_CUDA;
    }
    if (dev < 64) configured[dev] = true;
  }
  CUtensorMap ma, mb, mw, md;
  if (!make_tensor_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a_q8, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)p.K, 128,
                          P_BM, true))
    return TQ_ERR_CUDA;
  if (!make_tensor_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b_col, (uint64_t)(p.K / 2), (uint64_t)p.N,
                          (uint64_t)(p.K / 2), P_BK / 2, P_BH))
    return TQ_ERR_CUDA;
  const void* wsrc = p.has_tail ? w_rot : (const void*)b_col;  // never loaded without a tail; kept valid
  if (!make_tensor_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, wsrc, (uint64_t)(p.has_tail ? p.K : p.K / 4),
                          (uint64_t)p.N, (uint64_t)(p.has_tail ? p.K * 2 : p.K / 2), 64, P_BH, true))
    return TQ_ERR_CUDA;
  // the zero-filled tail matrix, 32 rows x one 64-wide half slice per load (rows beyond M read as zeros)
  p.dense = (p.has_tail && tail_dense) ? 1 : 0;
  if (p.dense) {
    if (!make_tensor_map_2d(&md, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, tail_dense, (uint64_t)p.K, (uint64_t)p.M,
                            (uint64_t)p.K * 2, 64, 32, true))
      return TQ_ERR_CUDA;
  } else {
    md = mw;  // never used; kept valid
  }
  p.tiles_m = (p.M + 2 * P_BM - 1) / (2 * P_BM);
  p.tiles_n = (p.N + P_BN - 1) / P_BN;
  p.kb_total = p.K / P_BK;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int total = p.tiles_m * p.tiles_n;
  const int pairs = total < sms / 2 ? total : sms / 2;
  pair_gemm_kernel<ACT><<<2 * pairs, P_THREADS, S::DYN, st>>>(ma, mb, mw, md, p);
  return check_launch();
}

}  // namespace

// Runs the pair kernel when the problem has enough 256 x 256 tiles to fill the machine; `*used` says whether it did.
int run_pair_gemm(const int8_t* a_q8, const float* body_scale, const uint8_t* b_col, const float* w_scale,
                  const void* w_rot, const uint16_t* tail_idx16, const void* tail_val, int tail_ld,
                  const uint16_t* tail_ptr, int ptr_ld, const uint32_t* tail_rec, const uint16_t* tail_cnt,
                  const void* tail_dense, int R, const float* bias, void* out_bf16, int32_t* dbg_acc, float* dbg_tail,
                  int M, int N, int K, int act, cudaStream_t st) {
  PairGemmParams p = {};
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
  if (tail_dense && !aligned16(tail_dense)) return TQ_ERR_MISALIGNED;
  return act ? launch_pair_gemm<1>(a_q8, b_col, w_rot, tail_dense, p, st)
             : launch_pair_gemm<0>(a_q8, b_col, w_rot, tail_dense, p, st);
}

}  // namespace tq
