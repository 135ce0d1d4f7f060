// Fused prologue of the split W4A4 + tail linear, the kernel for the layer widths of the benchmarked models
// (K = 4096, 12288, 14336; sm_100a).  Same outputs, bit for bit, as the general kernel in tq_prologue.cu.
//
// One CTA of K/64 threads works on one row at a time (grid-stride over rows).
//   * The row arrives by ONE tiled TMA load into shared memory ([K/64 rows of 64 elements], 128-byte swizzle), so a
//     thread reads its 64 contiguous elements with eight conflict-free 128-bit loads.
//   * Rotation in fp32, ascending butterfly strides, 64 elements per thread held as 32 packed fp32 pairs
//     (add / sub / mul / fma .f32x2).  K = 4096: strides 1..32 in registers, one transposing exchange through a
//     swizzled fp32 buffer, strides 64..2048 in registers.  K = 12288 (12 (x) 1024): strides 1..32, exchange, strides
//     64..512, exchange, the 12-point mix.  K = 14336 (block-128): strides 1..32 in registers, stride 64 by one
//     shuffle with the neighbouring lane -- no exchange at all.
//   * One multiply by the normalisation, one rounding to bf16; the bf16 row goes back to the row buffer and from
//     there on thread t owns elements [64 t, 64 t + 64), i.e. exactly one 64-wide half of a K slice: tie-breaking
//     by index, positions of the tail entries and the per-half-slice records need one block scan and nothing else.
//   * Exact rank selection on the 15-bit magnitude keys: distances from the row maximum are histogrammed in
//     windows of 256 key values with shared-memory atomics (the first window holds the threshold for any
//     Gaussian-like row; further windows follow until the rank is reached, so every input is handled exactly).
//   * Membership masks from two subtractions per pair of elements (the borrow lands in the top bit of each half).
//   * INT4 codes by reciprocal multiply + magic-number rounding on packed pairs; elements within 2e-6 of a rounding
//     boundary are redone with the IEEE division (exact rint(x / scale) semantics, a handful per million).
//
// Reference behaviour covered: tools/fused_threshold_topr_pack_ext_v57.py:96-194 (select, scales, pack),
// tools/fused_topr_pack_ext_v55.py:21-26,73-109 (clamp_s4, scale = max(key, eps)/7, body nibble 0 at tail
// positions, nibble order; fp16 input as there), plus the online rotation that the reference runs as a separate
// kernel.
#include "tq_common.cuh"
#include "tq_ptx.cuh"
#include "tq_prologue.cuh"

namespace tq {
namespace {

typedef unsigned long long u64;
constexpr unsigned FM = 0xffffffffu;

// ------------------------------------------------------------------------------------ packed fp32 pairs
__device__ __forceinline__ u64 pk2(float lo, float hi) {
  u64 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void up2(u64 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
  u64 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ u64 sub2(u64 a, u64 b) {
  u64 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
  u64 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
  u64 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {  // (lo -> bits 0..15, hi -> bits 16..31), RNE
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// shared-memory accesses through plain pointers: the compiler folds constant offsets into the instructions
typedef unsigned char* smp;
__device__ __forceinline__ uint4 lds128(const unsigned char* a) { return *reinterpret_cast<const uint4*>(a); }
__device__ __forceinline__ void sts128(unsigned char* a, uint4 v) { *reinterpret_cast<uint4*>(a) = v; }
__device__ __forceinline__ void sts32(unsigned char* a, uint32_t v) { *reinterpret_cast<uint32_t*>(a) = v; }
__device__ __forceinline__ void sts16(unsigned char* a, uint32_t v) { *reinterpret_cast<unsigned short*>(a) = (unsigned short)v; }
__device__ __forceinline__ uint32_t lds16(const unsigned char* a) { return (uint32_t)*reinterpret_cast<const unsigned short*>(a); }

// 64-point Walsh-Hadamard butterflies, strides 1, 2, ..., 32 in that order, on 32 packed pairs (elements 2j, 2j+1)
__device__ __forceinline__ void wht64(u64 (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float a, b;
    up2(v[j], a, b);
    v[j] = pk2(__fadd_rn(a, b), __fsub_rn(a, b));
  }
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if ((j & s) == 0) {
        const u64 a = v[j], b = v[j + s];
        v[j] = add2(a, b);
        v[j + s] = sub2(a, b);
      }
    }
  }
}

// 16-bit input word (bf16 or fp16) -> fp32
template <int DT>
__device__ __forceinline__ void unpack_word(uint32_t w, float& lo, float& hi) {
  if (DT == TQ_BF16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
}
template <int DT>
__device__ __forceinline__ float key_to_f32(uint32_t key) {  // 15-bit magnitude key -> value
  if (DT == TQ_BF16) return __uint_as_float(key << 16);
  return __half2float(__ushort_as_half((unsigned short)key));
}

struct Sel {
  int kp;       // distance from the row maximum of the key at the requested rank
  int cnt_lt;   // keys strictly larger (distance strictly smaller)
  int cnt_eq;   // keys equal to it
  int next_kp;  // next larger distance present in the same window, or -1
};

// rank is 1-based in (key descending) order; dd[j] holds the distances kmax - key of elements 2j (low half) and
// 2j + 1 (high half).  Uniform over the CTA; uses `hist` (256 words) and `res` (8 words).
template <int NT>
__device__ __forceinline__ Sel select_rank(const uint32_t (&dd)[32], int rank, uint32_t* hist, int* res, int tid) {
  const uint32_t hist_s = smem_u32(hist);
  int below = 0;  // keys at a distance below the window
  for (int base = 0; base < 32768; base += 256) {
    for (int i = tid; i < 256; i += NT) hist[i] = 0u;
    __syncthreads();
    const uint32_t b4 = (uint32_t)base << 2;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const uint32_t lo = ((dd[j] << 2) & 0x3fffcu) - b4;   // 4 * (distance - base); wraps to a large value below the window
      const uint32_t hi = ((dd[j] >> 14) & 0x3fffcu) - b4;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.lt.u32 p, %1, 1024;\n\t"
          "setp.lt.u32 q, %2, 1024;\n\t"
          "@p red.shared.add.u32 [%0], 1;\n\t"
          "@q red.shared.add.u32 [%3], 1;\n\t}"
          ::"r"(hist_s + lo), "r"(lo), "r"(hi), "r"(hist_s + hi)
          : "memory");
    }
    __syncthreads();
    if (tid < 32) {
      const int lane = tid;
      const uint4 ha = *reinterpret_cast<const uint4*>(hist + 8 * lane);
      const uint4 hb = *reinterpret_cast<const uint4*>(hist + 8 * lane + 4);
      const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
      uint32_t s = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += h[i];
      uint32_t incl = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(FM, incl, o);
        if (lane >= o) incl += t;
      }
      const uint32_t total = __shfl_sync(FM, incl, 31);
      const uint32_t r2 = (uint32_t)(rank - below);
      const unsigned hit = __ballot_sync(FM, incl >= r2);
      const unsigned nonempty = __ballot_sync(FM, s > 0);
      if (lane == 0) {
        res[0] = hit != 0u;
        res[4] = -1;
        res[5] = -1;
        res[6] = (int)total;
      }
      __syncwarp();
      if (hit) {
        const int fl = __ffs(hit) - 1;
        if (lane == fl) {
          uint32_t acc = incl - s;
          int f = 7;
          uint32_t lt = 0;
          bool done = false;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (!done && acc + h[i] >= r2) {
              f = i;
              lt = acc;
              done = true;
            }
            acc += h[i];
          }
          res[1] = 8 * lane + f;
          res[2] = below + (int)lt;
          res[3] = (int)h[f];
          int nx = -1;
#pragma unroll
          for (int i = 7; i >= 0; --i)
            if (i > f && h[i] > 0) nx = 8 * lane + i;
          res[4] = nx;
        }
        const unsigned later = (fl < 31) ? (nonempty & ~((2u << fl) - 1u)) : 0u;
        if (later && lane == __ffs(later) - 1) {
          int nx = -1;
#pragma unroll
          for (int i = 7; i >= 0; --i)
            if (h[i] > 0) nx = 8 * lane + i;
          res[5] = nx;
        }
      }
    }
    __syncthreads();
    if (res[0]) {
      Sel out;
      out.kp = base + res[1];
      out.cnt_lt = res[2];
      out.cnt_eq = res[3];
      const int nb = res[4] >= 0 ? res[4] : res[5];
      out.next_kp = nb >= 0 ? base + nb : -1;
      return out;  // (the caller's next use of hist / res lies behind barriers)
    }
    below += res[6];
  }
  Sel none;
  none.kp = 32767;
  none.cnt_lt = below;
  none.cnt_eq = 0;
  none.next_kp = -1;
  return none;
}

// shared-memory carve-up (offsets from the 1024-byte aligned base)
template <int KIND, int K>
struct FS {
  static constexpr int NT = K / 64;
  static constexpr bool XBUF = (KIND == TQ_HAD_WHT || KIND == TQ_HAD_KRON12);
  // K = 4096: the fp32 exchange buffer starts AT the row buffer (the 16-bit row is dead between the first register
  // pass and the write-back of the rotated row; one barrier after the second pass's loads keeps the two apart)
  static constexpr bool ALIAS = (KIND == TQ_HAD_WHT);
  static constexpr int ROW_OFF = 0;                        // [K] 16-bit row, [K/64][8 chunks of 16 B], chunk ^= row & 7
  static constexpr int X_OFF = ALIAS ? 0 : K * 2;          // [K] fp32 exchange buffer, rows of 256 B, same swizzle
  // after the rotation: [K] u16 list of the row's tail indices, then [K/64] u32 list position of each half slice
  static constexpr int LIST_OFF = K * 2;
  static constexpr int HST_OFF = LIST_OFF + K * 2;
  static constexpr int AUX_END = HST_OFF + (K / 64) * 4;
  static constexpr int X_END = XBUF ? X_OFF + K * 4 : 0;
  static constexpr int HIST_OFF = (AUX_END > X_END ? AUX_END : X_END);
  static constexpr int RED_OFF = HIST_OFF + 1024;          // 16 words: block max / sums
  static constexpr int RES_OFF = RED_OFF + 64;             // 8 words: select result
  static constexpr int SCAN_OFF = RES_OFF + 32;            // 8 words: warp totals of the scan
  static constexpr int BAR_OFF = SCAN_OFF + 32;            // mbarrier (8 B) + abort flag
  static constexpr int DYN = BAR_OFF + 16 + 1024;          // + alignment slack
};

constexpr int fast_min_ctas(int K) { return K <= 4096 ? 10 : (K <= 12288 ? 3 : 2); }

template <int KIND, int K, int DT, bool NORM>
__global__ void __launch_bounds__(K / 64, fast_min_ctas(K))
prologue_fast_kernel(const __grid_constant__ CUtensorMap tmap_x, const PrologueParams p) {
  using S = FS<KIND, K>;
  constexpr int NT = S::NT;
  constexpr int NW = (NT + 31) / 32;
  constexpr int NHS = K / 64;   // one thread per 64-wide half slice
  constexpr int NSL = K / 128;
  static_assert(K % 2048 == 0 && NT <= 256, "row width");
  static_assert((KIND == TQ_HAD_NONE && !NORM) || DT == TQ_BF16, "rotation and RMSNorm take bf16 input");
  static_assert(KIND != TQ_HAD_WHT || K == 4096, "full transform: K = 4096");
  static_assert(KIND != TQ_HAD_KRON12 || K == 12288, "12 (x) 2^n: K = 12288");

  extern __shared__ unsigned char smem_dyn[];
  const uint32_t raw = smem_u32(smem_dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* sm = smem_dyn + (base - raw);
  const uint32_t rowbuf_s = base + S::ROW_OFF;  // (shared-window address, for the TMA load)
  const smp rowbuf = sm + S::ROW_OFF;
  const smp xbuf = sm + S::X_OFF;
  uint32_t* hist = reinterpret_cast<uint32_t*>(sm + S::HIST_OFF);
  uint32_t* red = reinterpret_cast<uint32_t*>(sm + S::RED_OFF);
  int* res = reinterpret_cast<int*>(sm + S::RES_OFF);
  uint32_t* scanw = reinterpret_cast<uint32_t*>(sm + S::SCAN_OFF);
  const uint32_t bar = base + S::BAR_OFF;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + S::BAR_OFF + 8);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int R = p.R;
  const smp my_row = rowbuf + tid * 128;
  const uint32_t my_sw = (uint32_t)(tid & 7) << 4;

  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
    mbar_init(bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  uint32_t phase = 0;
  for (int m = blockIdx.x; m < p.M; m += gridDim.x, phase ^= 1u) {
    // ---- the row: one tiled TMA load.  (The previous row's last reads of the row buffer lie before the barrier
    // that ends its iteration; the proxy fence orders them before the asynchronous write.)
    if (tid == 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_expect_tx(bar, (uint32_t)K * 2u);
      tma_load_2d(rowbuf_s, &tmap_x, 0, m * (K / 64), bar);
    }
    {
      const bool ok = mbar_wait(bar, phase, abort_flag, 0x400000u);
      if (!__syncthreads_and(ok)) break;  // a bounded wait ran out: every thread leaves (status word set)
    }
    uint32_t w[32];  // the thread's 64 elements of the rotated row, two 16-bit values per word
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 q = lds128(my_row + (((uint32_t)c << 4) ^ my_sw));
      w[4 * c] = q.x;
      w[4 * c + 1] = q.y;
      w[4 * c + 2] = q.z;
      w[4 * c + 3] = q.w;
    }

    if (KIND != TQ_HAD_NONE || NORM) {
      u64 v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float lo, hi;
        unpack_word<TQ_BF16>(w[j], lo, hi);
        v[j] = pk2(lo, hi);
      }
      if (NORM) {
        // RMSNorm in front of the rotation: inv = 1 / sqrt(mean(x^2) + eps) with the squares summed per thread in
        // index order over its 64 contiguous elements, a butterfly over the warp and the warp sums added in order
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float lo, hi;
          up2(v[j], lo, hi);
          ss = __fadd_rn(ss, __fmul_rn(lo, lo));
          ss = __fadd_rn(ss, __fmul_rn(hi, hi));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(FM, ss, o));
        float* redf = reinterpret_cast<float*>(red);
        if (lane == 0) redf[warp] = ss;
        __syncthreads();
        float tot = redf[0];
#pragma unroll
        for (int q = 1; q < NW; ++q) tot = __fadd_rn(tot, redf[q]);
        __syncthreads();  // (red is reused by the block maximum)
        const float rms_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.rms_eps)));
        // y = bf16(bf16(x * inv) * gamma), as a bf16 framework's RMSNorm rounds
        const uint4* gp = reinterpret_cast<const uint4*>(p.gamma + 64 * tid);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 g4 = __ldg(gp + c);
          const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float lo, hi, gl, gh;
            up2(v[4 * c + i], lo, hi);
            unpack_word<TQ_BF16>(gw[i], gl, gh);
            lo = bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn(lo, rms_inv)));
            hi = bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn(hi, rms_inv)));
            lo = bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn(lo, gl)));
            hi = bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn(hi, gh)));
            v[4 * c + i] = pk2(lo, hi);
          }
        }
      }
      const u64 hs2 = pk2(p.hscale, p.hscale);
      if (KIND != TQ_HAD_NONE) wht64(v);  // strides 1 .. 32

      if (KIND == TQ_HAD_NONE) {
        // (normalised, not rotated) the values are bf16 already: back into words and into the row buffer
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float lo, hi;
          up2(v[j], lo, hi);
          w[j] = cvt_bf16x2(lo, hi);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          sts128(my_row + (((uint32_t)c << 4) ^ my_sw), make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
      } else if (KIND == TQ_HAD_BLOCK128) {
        // stride 64: the other half of the 128-block sits in the neighbouring lane
        const float sg = (tid & 1) ? -1.0f : 1.0f;
        const u64 sg2 = pk2(sg, sg);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float lo, hi;
          up2(v[j], lo, hi);
          const float plo = __shfl_xor_sync(FM, lo, 1), phi = __shfl_xor_sync(FM, hi, 1);
          v[j] = fma2(sg2, v[j], pk2(plo, phi));  // even lane: v + partner; odd lane: partner - v (exact products)
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float lo, hi;
          up2(mul2(v[j], hs2), lo, hi);
          w[j] = cvt_bf16x2(lo, hi);
        }
        // the thread's own row goes back to the row buffer (the tail emission reads single values from it)
#pragma unroll
        for (int c = 0; c < 8; ++c)
          sts128(my_row + (((uint32_t)c << 4) ^ my_sw), make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]));
      } else if (KIND == TQ_HAD_WHT) {
        // ---- transpose through the fp32 buffer: element i of thread t -> (row i, column t)
        if (S::ALIAS) __syncthreads();  // (the buffer overlays the 16-bit row: every thread has read its part)
        {
          const smp wb = xbuf + (tid & 3) * 4;
          const uint32_t ch = (uint32_t)(tid >> 2);
          smp wa[8];  // the eight swizzled column positions of this thread
#pragma unroll
          for (int q = 0; q < 8; ++q) wa[q] = wb + ((ch ^ (uint32_t)q) << 4);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float lo, hi;
            up2(v[j], lo, hi);
            const int i0 = 2 * j, i1 = 2 * j + 1;
            sts32(wa[i0 & 7] + i0 * 256, __float_as_uint(lo));
            sts32(wa[i1 & 7] + i1 * 256, __float_as_uint(hi));
          }
        }
        __syncthreads();
        {
          const smp rb = xbuf + tid * 256;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const uint4 q = lds128(rb + ((((uint32_t)(c & 7)) << 4) ^ my_sw) + (uint32_t)(c >> 3) * 128u);
            v[2 * c] = pk2(__uint_as_float(q.x), __uint_as_float(q.y));
            v[2 * c + 1] = pk2(__uint_as_float(q.z), __uint_as_float(q.w));
          }
        }
        if (S::ALIAS) __syncthreads();  // every thread has its values: the rotated row may overwrite the exchange buffer
        wht64(v);  // strides 64 .. 2048: the thread holds elements 64 j + t
        // ---- normalise, round, park the bf16 row in index order: element 64 j + t -> (row j, position t)
        {
          const smp wb = rowbuf + (tid & 7) * 2;
          const uint32_t ch = (uint32_t)(tid >> 3);
          smp wa[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) wa[q] = wb + ((ch ^ (uint32_t)q) << 4);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float lo, hi;
            up2(mul2(v[j], hs2), lo, hi);
            const uint32_t b2 = cvt_bf16x2(lo, hi);
            const int j0 = 2 * j, j1 = 2 * j + 1;
            sts16(wa[j0 & 7] + j0 * 128, b2);
            sts16(wa[j1 & 7] + j1 * 128, b2 >> 16);
          }
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 q = lds128(my_row + (((uint32_t)c << 4) ^ my_sw));
          w[4 * c] = q.x;
          w[4 * c + 1] = q.y;
          w[4 * c + 2] = q.z;
          w[4 * c + 3] = q.w;
        }
      } else {  // TQ_HAD_KRON12, K = 12288: thread t = (segment a = t / 16, block p = t % 16)
        // ---- own 64 values -> own 256-byte row of the fp32 buffer
        {
          const smp rb = xbuf + tid * 256;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float a0, a1, a2, a3;
            up2(v[2 * c], a0, a1);
            up2(v[2 * c + 1], a2, a3);
            sts128(rb + ((((uint32_t)(c & 7)) << 4) ^ my_sw) + (uint32_t)(c >> 3) * 128u,
                   make_uint4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3)));
          }
        }
        __syncthreads();
        // ---- strides 64 .. 512 inside the segment: thread (a, u) holds positions 64 h + 4 u + c, h < 16, c < 4
        {
          const int u = tid & 15;
          const smp segb = xbuf + (tid >> 4) * 4096 + (u >> 3) * 128;
          const uint32_t usw = (uint32_t)(u & 7) << 4;
          u64 b[16][2];
#pragma unroll
          for (int h = 0; h < 16; ++h) {
            const uint4 q = lds128(segb + (usw ^ ((uint32_t)(h & 7) << 4)) + (uint32_t)h * 256u);
            b[h][0] = pk2(__uint_as_float(q.x), __uint_as_float(q.y));
            b[h][1] = pk2(__uint_as_float(q.z), __uint_as_float(q.w));
          }
#pragma unroll
          for (int s = 1; s < 16; s <<= 1) {
#pragma unroll
            for (int h = 0; h < 16; ++h) {
              if ((h & s) == 0) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const u64 x0 = b[h][e], x1 = b[h + s][e];
                  b[h][e] = add2(x0, x1);
                  b[h + s][e] = sub2(x0, x1);
                }
              }
            }
          }
#pragma unroll
          for (int h = 0; h < 16; ++h) {
            float a0, a1, a2, a3;
            up2(b[h][0], a0, a1);
            up2(b[h][1], a2, a3);
            sts128(segb + (usw ^ ((uint32_t)(h & 7) << 4)) + (uint32_t)h * 256u,
                   make_uint4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3)));
          }
        }
        __syncthreads();
        // ---- the 12-point mix across segments: thread t takes positions 6 t .. 6 t + 5 of every segment
        // (threads 171 .. 191 have none), sums in the fixed order a = 0 .. 11
        {
          const int q0 = 6 * tid;
          uint32_t roff[3], woff[3];
#pragma unroll
          for (int k = 0; k < 3; ++k) {
            const int q = q0 + 2 * k;
            const uint32_t r = (uint32_t)(q >> 6);
            roff[k] = r * 256u + (((((uint32_t)q >> 2) & 15u) ^ (r & 7u)) << 4) + ((uint32_t)q & 3u) * 4u;
            woff[k] = r * 128u + (((((uint32_t)q >> 3) & 7u) ^ (r & 7u)) << 4) + ((uint32_t)q & 7u) * 2u;
          }
#pragma unroll
          for (int k = 0; k < 3; ++k) {
            if (q0 + 2 * k < 1024) {
              u64 c[12];
#pragma unroll
              for (int a = 0; a < 12; ++a) {
                float lo, hi;
                const float2 f = *reinterpret_cast<const float2*>(xbuf + a * 4096 + roff[k]);
                lo = f.x;
                hi = f.y;
                c[a] = pk2(lo, hi);
              }
              float n0, n1;
              up2(c[0], n0, n1);
              const u64 neg0 = pk2(-n0, -n1);
#pragma unroll
              for (int a2 = 0; a2 < 12; ++a2) {
                u64 acc = (H12_NEG[a2] & 1) ? neg0 : c[0];
#pragma unroll
                for (int a = 1; a < 12; ++a) acc = ((H12_NEG[a2] >> a) & 1) ? sub2(acc, c[a]) : add2(acc, c[a]);
                float lo, hi;
                up2(mul2(acc, hs2), lo, hi);
                sts32(rowbuf + a2 * 2048 + woff[k], cvt_bf16x2(lo, hi));
              }
            }
          }
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 q = lds128(my_row + (((uint32_t)c << 4) ^ my_sw));
          w[4 * c] = q.x;
          w[4 * c + 1] = q.y;
          w[4 * c + 2] = q.z;
          w[4 * c + 3] = q.w;
        }
      }
    }

    // =============================================================== thread t owns elements [64 t, 64 t + 64)
    if (p.x_rot) {
      uint4* dst = reinterpret_cast<uint4*>(p.x_rot + (size_t)m * K + 64 * tid);
#pragma unroll
      for (int c = 0; c < 8; ++c) dst[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
    }
    // ---- row maximum of the 15-bit magnitude keys
    uint32_t kmax;
    {
      uint32_t mx = 0u;
#pragma unroll
      for (int j = 0; j < 32; ++j) mx = max_u16x2(mx, w[j] & 0x7fff7fffu);
      mx = max(mx & 0xffffu, mx >> 16);
      mx = __reduce_max_sync(FM, mx);
      if (lane == 0) red[warp] = mx;
      __syncthreads();
      kmax = red[0];
#pragma unroll
      for (int q = 1; q < NW; ++q) kmax = max(kmax, red[q]);
    }
    uint32_t dd[32];  // distances from the maximum, two per word
    {
      const uint32_t km2 = kmax | (kmax << 16);
#pragma unroll
      for (int j = 0; j < 32; ++j) dd[j] = km2 - (w[j] & 0x7fff7fffu);
    }

    // ---- rank selection (one inlined call site: first the tail rank, then, if it does not follow from that
    // result, the body rank)
    int Tkp = -1, cnt_lt = 0, body_kp = 0;
    {
      int want = R > 0 ? R : (p.dr > 1 ? p.dr : 0);
      bool tail_pass = R > 0;
      while (want) {  // uniform over the CTA
        const Sel s = select_rank<NT>(dd, want, hist, res, tid);
        want = 0;
        if (tail_pass) {
          tail_pass = false;
          Tkp = s.kp;
          cnt_lt = s.cnt_lt;
          if (p.dr > s.cnt_lt && p.dr <= s.cnt_lt + s.cnt_eq) {
            body_kp = s.kp;
          } else if (p.dr == s.cnt_lt + s.cnt_eq + 1 && s.next_kp >= 0) {
            body_kp = s.next_kp;
          } else {
            want = p.dr;
          }
        } else {
          body_kp = s.kp;
        }
      }
    }
    const int need = R - cnt_lt;  // keys equal to the threshold that still belong to the tail (lowest indices)
    const float tscale = make_scale(key_to_f32<DT>(kmax), p.eps, p.scale_mode);
    const float bscale = make_scale(key_to_f32<DT>(kmax - (uint32_t)body_kp), p.eps, p.scale_mode);
    const float brinv = __fdiv_rn(1.0f, bscale);

    // ---- tail membership.  Mask layout: mask[h] covers elements 32 h .. 32 h + 31; bit i = element 2 i (low half of
    // word i), bit 16 + i = element 2 i + 1.
    uint32_t tm[2] = {0u, 0u};
    int tail_before = 0;  // tail entries of the row in front of this thread's elements
    if (R > 0) {
      const uint32_t T2 = (uint32_t)Tkp | ((uint32_t)Tkp << 16);
      const uint32_t c_le = 0x80008000u + T2, c_lt = 0x7fff7fffu + T2;  // per half: top bit set <=> d <= T, d < T
      uint32_t le[2] = {0u, 0u}, lt[2] = {0u, 0u};
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int h = j >> 4, i = j & 15;
        le[h] |= ((c_le - dd[j]) >> (15 - i)) & (0x00010001u << i);
        lt[h] |= ((c_lt - dd[j]) >> (15 - i)) & (0x00010001u << i);
      }
      const uint32_t eq[2] = {le[0] ^ lt[0], le[1] ^ lt[1]};
      const uint32_t cnt = (uint32_t)(__popc(lt[0]) + __popc(lt[1])) | ((uint32_t)(__popc(eq[0]) + __popc(eq[1])) << 16);
      uint32_t incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(FM, incl, o);
        if (lane >= o) incl += t;
      }
      if (lane == 31 || tid == NT - 1) scanw[warp] = incl;
      __syncthreads();
      uint32_t pre = incl - cnt;
#pragma unroll
      for (int q = 0; q < NW - 1; ++q)
        if (q < warp) pre += scanw[q];
      const int gt_before = (int)(pre & 0xffffu), eq_before = (int)(pre >> 16);
      tail_before = gt_before + min(eq_before, need);
      tm[0] = lt[0];
      tm[1] = lt[1];
      int take = need - eq_before;  // ties of this thread that join the tail: its first `take` in index order
      if (take > 0 && (eq[0] | eq[1])) {
        if (take >= (int)(cnt >> 16)) {
          tm[0] |= eq[0];
          tm[1] |= eq[1];
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t ev = eq[h] & 0xffffu, od = eq[h] >> 16;
            while ((ev | od) && take > 0) {
              const int a = ev ? __ffs(ev) - 1 : 32, b = od ? __ffs(od) - 1 : 32;
              if (a <= b) {
                tm[h] |= 1u << a;
                ev &= ev - 1u;
              } else {
                tm[h] |= 0x10000u << b;
                od &= od - 1u;
              }
              --take;
            }
          }
        }
      }
      const int ntail = __popc(tm[0]) + __popc(tm[1]);
      if (p.tail_dense) {
        // the row with everything outside the tail zeroed: the operand rows that the fused GEMM loads by TMA where a
        // half slice holds more entries than a record
        uint4* dst = reinterpret_cast<uint4*>(p.tail_dense + (size_t)m * K + 64 * tid);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int j = 4 * c + i;
            o[i] = w[j] & (((tm[j >> 4] >> (j & 15)) & 0x00010001u) * 0xffffu);
          }
          dst[c] = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      if (p.tail_ptr) {  // run boundaries of the row's ascending index list at multiples of 128
        if ((tid & 1) == 0) p.tail_ptr[(size_t)m * p.ptr_ld + (tid >> 1)] = (uint16_t)tail_before;
        if (tid == 0) p.tail_ptr[(size_t)m * p.ptr_ld + NSL] = (uint16_t)R;
      }
      if (p.tail_cnt) {
        p.tail_cnt[((size_t)(m >> 7) * NHS + tid) * 128 + (m & 127)] = (uint16_t)ntail;
        if (m == p.M - 1) {
          // the rows that pad M to a multiple of 256 (the CTA-pair GEMM's tile height) have no entries: the GEMM
          // kernels rely on these zeros instead of checking rows
          const int last = (p.M + 255) / 256 * 256;
          for (int r = p.M; r < last; ++r) p.tail_cnt[((size_t)(r >> 7) * NHS + tid) * 128 + (r & 127)] = 0;
        }
      }
      // ---- tail entries: every thread writes the indices of its own entries to the row's list in shared memory
      // (ascending), then the threads share the list evenly -- entry r goes to thread r mod NT -- so that the global
      // stores of the lists are coalesced and no thread waits for the one with the most entries
      {
        const smp list_s = sm + S::LIST_OFF;
        uint32_t* const hst = reinterpret_cast<uint32_t*>(sm + S::HST_OFF);
        hst[tid] = (uint32_t)tail_before;
        smp lp = list_s + 2 * tail_before;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t ev = tm[h] & 0xffffu, od = tm[h] >> 16;
          while (ev | od) {
            const int a = ev ? __ffs(ev) - 1 : 32, b = od ? __ffs(od) - 1 : 32;
            int e;
            if (a <= b) {
              e = 2 * a;
              ev &= ev - 1u;
            } else {
              e = 2 * b + 1;
              od &= od - 1u;
            }
            sts16(lp, (uint32_t)(64 * tid + 32 * h + e));
            lp += 2;
          }
        }
        __syncthreads();
        const size_t rl = (size_t)m * p.tail_ld, rb = (size_t)m * R;
        for (int r = tid; r < R; r += NT) {
          const uint32_t i = lds16(list_s + 2 * r);
          const uint32_t hs = i >> 6, e = i & 63u;
          const uint32_t vb = lds16(rowbuf + hs * 128u + (((e >> 3) ^ (hs & 7u)) << 4) + (e & 7u) * 2u);
          if (p.tail_idx16) p.tail_idx16[rl + r] = (uint16_t)i;
          if (p.tail_val) p.tail_val[rl + r] = (uint16_t)vb;
          if (p.idx32) p.idx32[rb + r] = (int32_t)i;
          if (p.top_q) {
            float xv, dummy;
            unpack_word<DT>(vb, xv, dummy);
            const float q = fminf(fmaxf(rintf(__fdiv_rn(xv, tscale)), -8.0f), 7.0f);
            p.top_q[rb + r] = (int8_t)(int)q;
          }
          if (p.tail_rec) {
            const int jr = r - (int)hst[hs];  // place of the entry in the record of its half slice
            if (jr < TQ_TAIL_REC_CAP)
              // bits 0..5: half the byte offset of the value inside its 128-byte row of the swizzled operand tile
              // (16-byte chunk index XOR row & 7, then the element); bits 16..31: the bf16 value
              p.tail_rec[(((size_t)(m >> 7) * NHS + hs) * 128 + (m & 127)) * TQ_TAIL_REC_CAP + jr] =
                  ((((e >> 3) ^ ((uint32_t)m & 7u)) << 3) | (e & 7u)) | (vb << 16);
          }
        }
      }
    }

    // ---- INT4 codes of the body: t = x * (1 / scale), rounded by adding 1.5 * 2^23 (the low byte of the sum is the
    // two's-complement code); |t - rint(t)| within 2e-6 of one half marks an element whose IEEE quotient may round
    // the other way -- those are redone with the division afterwards
    const bool clampq = p.dr != R + 1;  // (body scale below the body maximum: codes can leave [-8, 7])
    uint32_t fm[2] = {0u, 0u};  // elements on a rounding boundary, mask layout as tm
    {
      const u64 rinv2 = pk2(brinv, brinv);
      const u64 magic2 = pk2(12582912.0f, 12582912.0f), nmagic2 = pk2(-12582912.0f, -12582912.0f);
      // byte masks of the tail elements of an 8-group: 4 flag bits -> 4 bytes of 0xff
      auto bytemask = [](uint32_t nib) -> uint32_t { return (((nib & 0xfu) * 0x00204081u) & 0x01010101u) * 0xffu; };
#pragma unroll
      for (int g4 = 0; g4 < 2; ++g4) {  // 32 elements (16 words, four 8-groups) at a time
        uint32_t ul[16], uh[16];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          float lo, hi;
          unpack_word<DT>(w[16 * g4 + jj], lo, hi);
          u64 t2 = mul2(pk2(lo, hi), rinv2);
          if (clampq) {
            float a, b;
            up2(t2, a, b);
            t2 = pk2(fminf(fmaxf(a, -8.0f), 7.0f), fminf(fmaxf(b, -8.0f), 7.0f));
          }
          const u64 u2 = add2(t2, magic2);
          const u64 e2 = sub2(t2, add2(u2, nmagic2));
          float el, eh, fl, fh;
          up2(e2, el, eh);
          if (fabsf(el) >= 0.499998f) fm[g4] |= 1u << jj;
          if (fabsf(eh) >= 0.499998f) fm[g4] |= 0x10000u << jj;
          up2(u2, fl, fh);
          ul[jj] = __float_as_uint(fl);
          uh[jj] = __float_as_uint(fh);
        }
        uint32_t ev[4], od[4];  // byte k of ev[s] / od[s] = code of element 2 k / 2 k + 1 of group 4 g4 + s, tail -> 0
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const int j0 = 4 * s, sh = 4 * s;
          ev[s] = prmt(prmt(ul[j0], ul[j0 + 1], 0x0040u), prmt(ul[j0 + 2], ul[j0 + 3], 0x0040u), 0x5410u) &
                  ~bytemask(tm[g4] >> sh);
          od[s] = prmt(prmt(uh[j0], uh[j0 + 1], 0x0040u), prmt(uh[j0 + 2], uh[j0 + 3], 0x0040u), 0x5410u) &
                  ~bytemask(tm[g4] >> (16 + sh));
        }
        if (p.a_q8) {
          // INT8 form: even elements of the group first, then the odd ones -- the order in which the GEMM's
          // widening of the packed INT4 weights lays out K
          uint4* dst = reinterpret_cast<uint4*>(p.a_q8 + (size_t)m * K + 64 * tid + 32 * g4);
          dst[0] = make_uint4(ev[0], od[0], ev[1], od[1]);
          dst[1] = make_uint4(ev[2], od[2], ev[3], od[3]);
        }
        if (p.a_pack) {
          // packed form: byte k of a group's word = nibbles of elements (2 k, 2 k + 1)
          uint4 q;
          q.x = (ev[0] & 0x0f0f0f0fu) | ((od[0] & 0x0f0f0f0fu) << 4);
          q.y = (ev[1] & 0x0f0f0f0fu) | ((od[1] & 0x0f0f0f0fu) << 4);
          q.z = (ev[2] & 0x0f0f0f0fu) | ((od[2] & 0x0f0f0f0fu) << 4);
          q.w = (ev[3] & 0x0f0f0f0fu) | ((od[3] & 0x0f0f0f0fu) << 4);
          *reinterpret_cast<uint4*>(p.a_pack + (size_t)m * (K / 2) + 32 * tid + 16 * g4) = q;
        }
      }
    }
    // ---- the elements on a rounding boundary of the reciprocal product (exact half-integer quotients are common
    // with 8-bit mantissas: about one element in 400) get the IEEE division, and their code is patched in place
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t mk = fm[h] & ~tm[h];
      while (mk) {
        const int b = __ffs(mk) - 1;
        mk &= mk - 1u;
        const int e = 32 * h + (b < 16 ? 2 * b : 2 * (b - 16) + 1);
        const uint32_t vb = lds16(my_row + ((((uint32_t)e >> 3) << 4) ^ my_sw) + ((uint32_t)e & 7u) * 2u);
        float xv, dummy;
        unpack_word<DT>(vb, xv, dummy);
        const int code = (int)fminf(fmaxf(rintf(__fdiv_rn(xv, bscale)), -8.0f), 7.0f);
        if (p.a_q8) {
          const int c = e & 7;
          p.a_q8[(size_t)m * K + 64 * tid + (e & ~7) + ((c & 1) ? 4 + (c >> 1) : (c >> 1))] = (int8_t)code;
        }
        if (p.a_pack) {
          uint8_t* bp = p.a_pack + (size_t)m * (K / 2) + 32 * tid + (e >> 1);
          const uint8_t old = *bp;
          *bp = (e & 1) ? (uint8_t)((old & 0x0fu) | ((code & 0xf) << 4)) : (uint8_t)((old & 0xf0u) | (code & 0xf));
        }
      }
    }
    if (tid == 0) {
      p.body_scale[m] = bscale;
      if (p.top_scale) p.top_scale[m] = tscale;
    }
    __syncthreads();  // the next row's load overwrites the row buffer; hist / res / red / scanw start over
  }
}

template <int KIND, int K, int DT, bool NORM>
int launch_fast(const PrologueParams& p, cudaStream_t st) {
  using S = FS<KIND, K>;
  auto kern = prologue_fast_kernel<KIND, K, DT, NORM>;
  static bool configured[64] = {};
  static int grid_per_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(dev < 64 && configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::DYN);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return TQ_ERR_CUDA;
    }
    int sms = 148, per_sm = 1;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, S::NT, S::DYN);
    if (per_sm < 1) per_sm = 1;
    if (dev < 64) {
      grid_per_dev[dev] = sms * per_sm;
      configured[dev] = true;
    }
  }
  CUtensorMap mx;
  // the [M, K] matrix as [M K / 64] rows of 64 elements; the box is one row of the matrix
  if (!make_tensor_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, p.x, 64, (uint64_t)p.M * (K / 64), 128, 64, K / 64, true))
    return TQ_ERR_CUDA;
  int grid = dev < 64 ? grid_per_dev[dev] : 148;
  if (grid > p.M) grid = p.M;
  kern<<<grid, S::NT, S::DYN, st>>>(mx, p);
  return check_launch();
}

}  // namespace

int run_prologue_fast(int kind, int K, int dtype, const PrologueParams& p, cudaStream_t st) {
  const bool norm = p.gamma != nullptr;
  if (dtype == TQ_FP16) {
    if (kind != TQ_HAD_NONE || norm) return TQ_ERR_UNSUPPORTED;
    if (K == 4096) return launch_fast<TQ_HAD_NONE, 4096, TQ_FP16, false>(p, st);
    if (K == 12288) return launch_fast<TQ_HAD_NONE, 12288, TQ_FP16, false>(p, st);
    return TQ_ERR_UNSUPPORTED;
  }
#define TQ_FAST(KIND, KK)                        \
  if (kind == KIND && K == KK)                   \
    return norm ? launch_fast<KIND, KK, TQ_BF16, true>(p, st) : launch_fast<KIND, KK, TQ_BF16, false>(p, st);
  TQ_FAST(TQ_HAD_WHT, 4096)
  TQ_FAST(TQ_HAD_KRON12, 12288)
  TQ_FAST(TQ_HAD_BLOCK128, 14336)
  TQ_FAST(TQ_HAD_NONE, 4096)
  TQ_FAST(TQ_HAD_NONE, 12288)
  TQ_FAST(TQ_HAD_NONE, 14336)
#undef TQ_FAST
  return TQ_ERR_UNSUPPORTED;
}

}  // namespace tq
