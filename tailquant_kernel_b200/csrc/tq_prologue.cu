// Fused prologue of the split W4A4 + tail linear (sm_100a).
//
// One CTA of 256 threads works on one row at a time (grid-stride over rows):
//   1. rotation in fp32 with ascending butterfly strides: radix-16 register passes, the row
//      travelling between passes through a swizzled fp32 buffer in shared memory;
//   2. one fp32 multiply by the normalisation and one rounding to bf16;
//      -- the bf16 row is parked in shared memory and from here on a thread owns groups of 8
//      consecutive indices (group tid + 256 j), so that packing and prefixes need no exchange;
//   3. exact rank selection on the 15-bit magnitude keys (distance from the row maximum:
//      128-wide coarse bins counted in registers, then a 128-bin shared histogram);
//   4. tail membership with ties broken by lowest index (per-group masks + one block scan in
//      index order), tail entries emitted in ascending index order;
//   5. INT4 codes of the body with true-division semantics, packed / INT8 words stored straight
//      to global memory (4 or 8 contiguous bytes per lane).
//
// Reference behaviour covered: tools/fused_threshold_topr_pack_ext_v57.py:96-194 (select,
// scales, pack), tools/fused_topr_pack_ext_v55.py:21-26,73-109 (clamp_s4, scale = max(key,
// eps)/7, body nibble 0 at tail positions, nibble order), plus the online rotation that the
// reference runs as a separate kernel.
#include <cmath>

#include "tq_common.cuh"
#include "tq_prologue.cuh"

namespace tq {
namespace {

constexpr int NT = 256;
constexpr unsigned FULL = 0xffffffffu;

// fp32 word index -> physical word index of the row buffer.  Chosen so that the 128-bit
// stores of pass 1 and the 32-bit accesses of the later passes are bank-conflict free.
template <int SWB>
__device__ __forceinline__ int swz(int i) {
  return i ^ (((i >> 5) & 3) << 2) ^ (((i >> SWB) & 1) << 4);
}

template <int N>
__device__ __forceinline__ void butterflies(float* v) {
#pragma unroll
  for (int s = 1; s < N; s <<= 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if ((i & s) == 0) {
        float a = v[i], b = v[i + s];
        v[i] = a + b;
        v[i + s] = a - b;
      }
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4& a, float* v) {
  v[0] = __uint_as_float(a.x << 16);
  v[1] = __uint_as_float(a.x & 0xffff0000u);
  v[2] = __uint_as_float(a.y << 16);
  v[3] = __uint_as_float(a.y & 0xffff0000u);
  v[4] = __uint_as_float(a.z << 16);
  v[5] = __uint_as_float(a.z & 0xffff0000u);
  v[6] = __uint_as_float(a.w << 16);
  v[7] = __uint_as_float(a.w & 0xffff0000u);
}

__device__ __forceinline__ uint32_t block_max(uint32_t v, uint32_t* red, int tid) {
  v = __reduce_max_sync(FULL, v);
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  uint32_t r = red[0];
#pragma unroll
  for (int w = 1; w < NT / 32; ++w) r = max(r, red[w]);
  return r;  // red[0..7] stay untouched until the next row: the rank selection uses red[16..31]
}

struct SelRes {
  int kp;       // distance from the row maximum of the key at the requested rank
  int cnt_lt;   // keys strictly larger (distance strictly smaller)
  int cnt_eq;   // keys equal to it
  int next_kp;  // next larger distance present in the same coarse bin, or -1
};

// rank is 1-based in (key descending) order.  pk[e] holds (bf16 bits << 16) | distance.
template <int E>
__device__ __forceinline__ SelRes select_rank(const uint32_t (&pk)[E], int rank, uint32_t* red,
                                              uint32_t* hist, int* res, int tid) {
  const int lane = tid & 31, warp = tid >> 5;
  int below = 0, base = 0, dstar = 0, cum_prev = 0;
  red += 16;                      // (the first half of `red` belongs to block_max)
  if (tid < 128) hist[tid] = 0;   // ordered before the histogram adds by the barrier(s) of the loop below
  while (true) {  // uniform across the block: every value below comes from shared memory
    uint32_t c = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      int dd = (int)((pk[e] & 0xffffu) >> 7) - base;
      if (dd >= 0 && dd < 4) c += 0x01010101u << (dd * 8);
    }
    uint32_t lo = __reduce_add_sync(FULL, c & 0x00ff00ffu);
    uint32_t hi = __reduce_add_sync(FULL, (c >> 8) & 0x00ff00ffu);
    if (lane == 0) {
      red[warp * 2] = lo;
      red[warp * 2 + 1] = hi;
    }
    __syncthreads();
    lo = 0;
    hi = 0;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) {
      lo += red[w * 2];
      hi += red[w * 2 + 1];
    }
    int cum[4] = {below + (int)(lo & 0xffffu), below + (int)(hi & 0xffffu), below + (int)(lo >> 16),
                  below + (int)(hi >> 16)};
    bool found = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (!found && cum[j] >= rank) {
        found = true;
        dstar = base + j;
        cum_prev = j ? cum[j - 1] : below;
      }
    }
    if (found || base >= 256) break;
    __syncthreads();  // every thread has read the counters before the next round overwrites them
    below = cum[3];
    base += 4;
  }

#pragma unroll
  for (int e = 0; e < E; ++e) {
    uint32_t kp = pk[e] & 0xffffu;
    if ((int)(kp >> 7) == dstar) atomicAdd(&hist[kp & 127u], 1u);
  }
  __syncthreads();
  if (warp == 0) {
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = hist[lane * 4 + j];
    uint32_t s = h[0] + h[1] + h[2] + h[3];
    uint32_t incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t t = __shfl_up_sync(FULL, incl, o);
      if (lane >= o) incl += t;
    }
    const uint32_t r2 = (uint32_t)(rank - cum_prev);
    unsigned hit = __ballot_sync(FULL, incl >= r2);
    unsigned nonempty = __ballot_sync(FULL, s > 0);
    int fl = hit ? (__ffs(hit) - 1) : 31;
    if (lane == 0) {
      res[3] = -1;
      res[4] = -1;
    }
    __syncwarp();
    if (lane == fl) {
      uint32_t acc = incl - s;
      int f = 3;
#pragma unroll
      for (int j = 3; j >= 0; --j) {  // smallest j whose running sum reaches r2
        uint32_t upto = acc;
#pragma unroll
        for (int i = 0; i <= j; ++i) upto += h[i];
        if (upto >= r2) f = j;
      }
      uint32_t lt = acc;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < f) lt += h[i];
      res[0] = lane * 4 + f;
      res[1] = (int)lt;
      res[2] = (int)h[f];
      int nx = -1;
#pragma unroll
      for (int i = 3; i >= 0; --i)
        if (i > f && h[i] > 0) nx = lane * 4 + i;
      res[3] = nx;
    }
    unsigned later = (fl < 31) ? (nonempty & ~((2u << fl) - 1u)) : 0u;
    if (later && lane == __ffs(later) - 1) {
      int nx = -1;
#pragma unroll
      for (int i = 3; i >= 0; --i)
        if (h[i] > 0) nx = lane * 4 + i;
      res[4] = nx;
    }
  }
  __syncthreads();
  SelRes out;
  out.kp = dstar * 128 + res[0];
  out.cnt_lt = cum_prev + res[1];
  out.cnt_eq = res[2];
  int nb = res[3] >= 0 ? res[3] : res[4];
  out.next_kp = nb >= 0 ? dstar * 128 + nb : -1;
  return out;  // (a later call rewrites hist / res only behind its own barriers)
}

// resident CTAs per SM the register budget is tuned for
constexpr int min_ctas(int K) { return K <= 4096 ? 4 : 2; }

template <int KIND, int K, bool NORM>  // NORM: RMSNorm in front of the rotation (p.gamma, p.rms_eps)
__global__ void __launch_bounds__(NT, min_ctas(K)) prologue_kernel(const PrologueParams p) {
  constexpr bool BLOCK = (KIND == TQ_HAD_BLOCK128);
  constexpr int SWB = BLOCK ? 7 : 8;
  constexpr int E = K / NT;
  constexpr int L = (KIND == TQ_HAD_KRON12) ? K / 12 : K;
  static_assert(K % NT == 0 && K % 32 == 0, "K must be a multiple of 256");
  static_assert(!BLOCK || K % 2048 == 0, "block-128 rotation needs K % 2048 == 0");
  static_assert(KIND != TQ_HAD_KRON12 || (L % 256 == 0), "kron12 needs K = 12 * 2^n, n >= 8");

  constexpr int GN = K / 8;                  // groups of 8 consecutive indices
  constexpr int J = (GN + NT - 1) / NT;      // groups per thread: g = tid + NT * j
  constexpr int EJ = 8 * J;
  constexpr int NSL = K / 128;               // 128-wide slices (K % 128 == 0 for every built K)
  constexpr int NHS = K / 64;                // 64-wide half slices: the unit of the tail records
  static_assert(J * (NT / 32) <= 64, "scan scratch");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* buf = reinterpret_cast<float*>(smem_raw);                           // [K] fp32, rotation passes
  uint16_t* rowb = reinterpret_cast<uint16_t*>(smem_raw + (size_t)K * 4);    // [K] rotated row as bf16 bits
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw + (size_t)K * 6);
  uint32_t* red = hist + 128;
  int* res = reinterpret_cast<int*>(red + 32);
  uint32_t* scan_a = reinterpret_cast<uint32_t*>(res + 8);  // [J][8] warp totals, then their exclusive scan
  uint32_t* scan_b = scan_a + 64;
  uint32_t* slice_pre = scan_b + 64;                         // [NHS] packed prefix at the start of each half slice
  const int Rpad = (p.R + 7) & ~7;
  uint16_t* st_idx = reinterpret_cast<uint16_t*>(slice_pre + ((NHS + 4) & ~3));
  uint16_t* st_val = st_idx + Rpad;
  int8_t* st_q = reinterpret_cast<int8_t*>(st_val + Rpad);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int R = p.R;
  const int fbase = BLOCK ? ((tid & 15) + 128 * (tid >> 4)) : tid;  // index = fbase + eoff(e)
  auto eoff = [](int e) -> int { return BLOCK ? (2048 * (e >> 3) + 16 * (e & 7)) : 256 * e; };

  for (int m = blockIdx.x; m < p.M; m += gridDim.x) {
    const __nv_bfloat16* xrow = p.x + (size_t)m * K;
    // ---- optional RMSNorm in front of the rotation: inv = 1 / sqrt(mean(x^2) + eps) with the squares summed per
    // thread in index order (16 contiguous elements, then the thread's next chunks), a butterfly over the warp
    // and the eight warp sums added in order -- the order the CPU oracle states
    float rms_inv = 0.0f;
    if (NORM) {
      float ss = 0.0f;
#pragma unroll
      for (int w0 = 0; w0 < K / 16; w0 += NT) {
        const int w = w0 + tid;
        if ((K / 16) % NT == 0 || w < K / 16) {
          const uint4* src = reinterpret_cast<const uint4*>(xrow + 16 * w);
          uint4 a = ldg_nc_128(src), b = ldg_nc_128(src + 1);
          float v[16];
          unpack8(a, v);
          unpack8(b, v + 8);
#pragma unroll
          for (int e = 0; e < 16; ++e) ss = __fadd_rn(ss, __fmul_rn(v[e], v[e]));
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(FULL, ss, o));
      float* redf = reinterpret_cast<float*>(red);
      if (lane == 0) redf[warp] = ss;
      __syncthreads();
      float tot = redf[0];
#pragma unroll
      for (int w = 1; w < NT / 32; ++w) tot = __fadd_rn(tot, redf[w]);
      __syncthreads();
      rms_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)K), p.rms_eps)));
    }
    // ---- pass 1: strides 1,2,4,8 on 16 contiguous elements straight from global memory
#pragma unroll
    for (int w0 = 0; w0 < K / 16; w0 += NT) {
      const int w = w0 + tid;
      if ((K / 16) % NT == 0 || w < K / 16) {
        const uint4* src = reinterpret_cast<const uint4*>(xrow + 16 * w);
        uint4 a = ldg_nc_128(src), b = ldg_nc_128(src + 1);
        float v[16];
        unpack8(a, v);
        unpack8(b, v + 8);
        if (NORM) {  // y = bf16(bf16(x * inv) * gamma), as a bf16 framework's RMSNorm rounds
          const uint4 ga = *reinterpret_cast<const uint4*>(p.gamma + 16 * w);
          const uint4 gb = *reinterpret_cast<const uint4*>(p.gamma + 16 * w + 8);
          float gm[16];
          unpack8(ga, gm);
          unpack8(gb, gm + 8);
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float xn = bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn(v[e], rms_inv)));
            v[e] = bf16_bits_to_f32(f32_to_bf16_bits(__fmul_rn(xn, gm[e])));
          }
        }
        if (KIND != TQ_HAD_NONE) butterflies<16>(v);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<float4*>(buf + swz<SWB>(16 * w + 4 * j)) =
              make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
    }
    __syncthreads();
    // ---- pass 2: strides 16..128 (full transform and 12 (x) 2^n only)
    if (KIND == TQ_HAD_WHT || KIND == TQ_HAD_KRON12) {
#pragma unroll
      for (int w0 = 0; w0 < K / 16; w0 += NT) {
        const int w = w0 + tid;
        if ((K / 16) % NT == 0 || w < K / 16) {
          const int i0 = (w & 15) + ((w >> 4) << 8);
          float v[16];
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] = buf[swz<SWB>(i0 + 16 * q)];
          butterflies<16>(v);
#pragma unroll
          for (int q = 0; q < 16; ++q) buf[swz<SWB>(i0 + 16 * q)] = v[q];
        }
      }
      __syncthreads();
    }
    // ---- final pass, ends in registers
    float v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) v[e] = buf[swz<SWB>(fbase + eoff(e))];
    if (KIND == TQ_HAD_WHT) {
      butterflies<E>(v);  // strides 256 .. K/2
    } else if (KIND == TQ_HAD_KRON12) {
      constexpr int EQ = E / 12;  // elements per 2^n segment held by this thread
#pragma unroll
      for (int a = 0; a < 12; ++a) butterflies<EQ>(v + a * EQ);
#pragma unroll
      for (int q = 0; q < EQ; ++q) {
        float c[12], o[12];
#pragma unroll
        for (int a = 0; a < 12; ++a) c[a] = v[a * EQ + q];
#pragma unroll
        for (int a2 = 0; a2 < 12; ++a2) {
          float acc = (H12_NEG[a2] & 1) ? -c[0] : c[0];
#pragma unroll
          for (int a = 1; a < 12; ++a) acc = ((H12_NEG[a2] >> a) & 1) ? acc - c[a] : acc + c[a];
          o[a2] = acc;
        }
#pragma unroll
        for (int a = 0; a < 12; ++a) v[a * EQ + q] = o[a];
      }
    } else if (BLOCK) {
#pragma unroll
      for (int g = 0; g < E / 8; ++g) butterflies<8>(v + g * 8);  // strides 16, 32, 64
    }

    // ---- normalise, round to bf16; the row goes to shared memory in index order
    uint32_t kmax = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const uint32_t b = f32_to_bf16_bits(v[e] * p.hscale);
      rowb[fbase + eoff(e)] = (uint16_t)b;
      kmax = max(kmax, b & 0x7fffu);
    }
    kmax = block_max(kmax, red, tid);  // its barriers also publish rowb and retire the last reads of buf

    // ---- keys of this thread's groups: (bf16 bits << 16) | distance from the row maximum
    uint32_t pk[EJ];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int g = tid + NT * j;
      const bool act = (GN % NT == 0) || g < GN;
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      if (act) {
        w = *reinterpret_cast<const uint4*>(rowb + 8 * g);
        if (p.x_rot) *reinterpret_cast<uint4*>(p.x_rot + (size_t)m * K + 8 * g) = w;
      }
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t b = (ww[c >> 1] >> (16 * (c & 1))) & 0xffffu;
        pk[8 * j + c] = act ? ((b << 16) | (kmax - (b & 0x7fffu))) : 0xffffu;  // idle groups: beyond every bin
      }
    }

    // ---- rank selection
    int Tkp = -1, cnt_lt = 0, body_kp = 0;
    if (R > 0) {
      SelRes s = select_rank<EJ>(pk, R, red, hist, res, tid);
      Tkp = s.kp;
      cnt_lt = s.cnt_lt;
      if (p.dr > s.cnt_lt && p.dr <= s.cnt_lt + s.cnt_eq) {
        body_kp = s.kp;
      } else if (p.dr == s.cnt_lt + s.cnt_eq + 1 && s.next_kp >= 0) {
        body_kp = s.next_kp;
      } else {
        body_kp = select_rank<EJ>(pk, p.dr, red, hist, res, tid).kp;
      }
    } else if (p.dr > 1) {
      body_kp = select_rank<EJ>(pk, p.dr, red, hist, res, tid).kp;
    }
    const int need = R - cnt_lt;  // keys equal to the threshold that still belong to the tail (lowest indices)
    const float tscale = make_scale(bf16_bits_to_f32(kmax), p.eps, p.scale_mode);
    const float bscale = make_scale(bf16_bits_to_f32(kmax - (uint32_t)body_kp), p.eps, p.scale_mode);
    const float brinv = __fdiv_rn(1.0f, bscale), trinv = __fdiv_rn(1.0f, tscale);

    // ---- tail membership: per-group masks, block scan of (larger | equal << 16) counts in index order
    uint32_t mg[J], me[J], tm[J], pre[J];
#pragma unroll
    for (int j = 0; j < J; ++j) mg[j] = me[j] = tm[j] = pre[j] = 0u;
    if (R > 0) {
      uint32_t cnt[J], incl[J];
#pragma unroll
      for (int j = 0; j < J; ++j) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int kp = (int)(pk[8 * j + c] & 0xffffu);
          mg[j] |= (uint32_t)(kp < Tkp) << c;
          me[j] |= (uint32_t)(kp == Tkp) << c;
        }
        cnt[j] = (uint32_t)__popc(mg[j]) | ((uint32_t)__popc(me[j]) << 16);
        incl[j] = cnt[j];
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const uint32_t t = __shfl_up_sync(FULL, incl[j], o);
          if (lane >= o) incl[j] += t;
        }
      }
      if (lane == 31) {
#pragma unroll
        for (int j = 0; j < J; ++j) scan_a[j * (NT / 32) + warp] = incl[j];
      }
      __syncthreads();
      if (warp == 0) {  // exclusive scan of the J x 8 warp totals, two per lane
        constexpr int NTOT = J * (NT / 32);
        const uint32_t a0 = (2 * lane < NTOT) ? scan_a[2 * lane] : 0u;
        const uint32_t a1 = (2 * lane + 1 < NTOT) ? scan_a[2 * lane + 1] : 0u;
        uint32_t sc = a0 + a1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t t = __shfl_up_sync(FULL, sc, o);
          if (lane >= o) sc += t;
        }
        const uint32_t ex = sc - (a0 + a1);
        scan_b[2 * lane] = ex;
        scan_b[2 * lane + 1] = ex + a0;
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < J; ++j) {
        const int g = tid + NT * j;
        pre[j] = scan_b[j * (NT / 32) + warp] + incl[j] - cnt[j];
        if (((GN % NT == 0) || g < GN) && (g & 7) == 0) slice_pre[g >> 3] = pre[j];
        tm[j] = mg[j];
        if (me[j]) {  // ties at the threshold: the `need` lowest indices of the row join the tail
          int neq = (int)(pre[j] >> 16);
          uint32_t mm = me[j];
          while (mm) {
            const int c = __ffs(mm) - 1;
            mm &= mm - 1u;
            if (neq < need) tm[j] |= 1u << c;
            ++neq;
          }
        }
      }
      if (p.tail_dense) {
        // the row with everything outside the tail zeroed (operand rows for the fused GEMM's dense half slices)
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const int g = tid + NT * j;
          if ((GN % NT == 0) || g < GN) {
            uint32_t o[4];
#pragma unroll
            for (int c = 0; c < 4; ++c)
              o[c] = (((tm[j] >> (2 * c)) & 1u) ? (pk[8 * j + 2 * c] >> 16) : 0u) |
                     (((tm[j] >> (2 * c + 1)) & 1u) ? (pk[8 * j + 2 * c + 1] & 0xffff0000u) : 0u);
            *reinterpret_cast<uint4*>(p.tail_dense + (size_t)m * K + 8 * g) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
      __syncthreads();
      // entries of the row's ascending list before a half slice: the larger keys, plus the ties that made it
      auto half_start = [&](int hs) -> int {
        const uint32_t ps = slice_pre[hs];
        return (int)(ps & 0xffffu) + min((int)(ps >> 16), need);
      };
      if (p.tail_ptr) {  // run boundaries of the row's ascending index list at multiples of 128
        for (int sl = tid; sl <= NSL; sl += NT)
          p.tail_ptr[(size_t)m * p.ptr_ld + sl] = (uint16_t)(sl < NSL ? half_start(2 * sl) : R);
      }
      if (p.tail_cnt) {
        for (int hs = tid; hs < NHS; hs += NT) {
          const int ea = half_start(hs), eb = hs + 1 < NHS ? half_start(hs + 1) : R;
          p.tail_cnt[((size_t)(m >> 7) * NHS + hs) * 128 + (m & 127)] = (uint16_t)(eb - ea);
        }
        if (m == p.M - 1) {
          // the rows that pad M to a multiple of 256 (the CTA-pair GEMM's tile height) have no entries: the GEMM
          // kernels rely on these zeros instead of checking rows
          const int first = p.M, last = (p.M + 255) / 256 * 256;
          for (int i = tid; i < NHS * (last - first); i += NT) {
            const int hs = i / (last - first), r = first + i % (last - first);
            p.tail_cnt[((size_t)(r >> 7) * NHS + hs) * 128 + (r & 127)] = 0;
          }
        }
      }
      // ---- tail entries, ascending index order
#pragma unroll
      for (int j = 0; j < J; ++j) {
        const int g = tid + NT * j;
        uint32_t mm = tm[j];
        while (mm) {
          const int c = __ffs(mm) - 1;
          mm &= mm - 1u;
          const uint32_t below = (1u << c) - 1u;
          const int i = 8 * g + c;
          const int pos = (int)(pre[j] & 0xffffu) + __popc(mg[j] & below) +
                          min((int)(pre[j] >> 16) + __popc(me[j] & below), need);
          const uint32_t vb = rowb[i];
          st_idx[pos] = (uint16_t)i;
          st_val[pos] = (uint16_t)vb;
          if (p.tail_rec) {  // the entry's place in the record of its 64-wide half slice
            const int jr = pos - half_start(i >> 6);
            if (jr < TQ_TAIL_REC_CAP)
              // bits 0..5: half the byte offset of the value inside its 128-byte row of the swizzled operand
              // tile (16-byte chunk index XOR row & 7, then the element); bits 16..31: the bf16 value
              p.tail_rec[(((size_t)(m >> 7) * NHS + (i >> 6)) * 128 + (m & 127)) * TQ_TAIL_REC_CAP + jr] =
                  (uint32_t)(((((i & 63) >> 3) ^ (m & 7)) << 3) | (i & 7)) | (vb << 16);
          }
          if (p.top_q) st_q[pos] = (int8_t)quant_s4(bf16_bits_to_f32(vb), tscale, trinv);
        }
      }
    }

    // ---- INT4 codes of the body: 8 nibbles (packed form) and 8 bytes (INT8 form) per group, stored directly
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int g = tid + NT * j;
      if ((GN % NT == 0) || g < GN) {
        uint32_t qlo = 0u, qhi = 0u;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const float xv = __uint_as_float(pk[8 * j + c] & 0xffff0000u);
          const int code = ((tm[j] >> c) & 1u) ? 0 : quant_s4(xv, bscale, brinv);
          // INT8 form: even elements of the group first, then the odd ones -- the order in which the GEMM's
          // widening of the packed INT4 weights lays out K
          if (c & 1)
            qhi |= ((uint32_t)code & 0xffu) << (8 * (c >> 1));
          else
            qlo |= ((uint32_t)code & 0xffu) << (8 * (c >> 1));
        }
        // packed form: nibble c = element c, i.e. the low nibbles of the even bytes interleaved with the odd ones
        const uint32_t packw = (qlo & 0x0f0f0f0fu) | ((qhi & 0x0f0f0f0fu) << 4);
        if (p.a_pack) *reinterpret_cast<uint32_t*>(p.a_pack + (size_t)m * (K / 2) + 4 * g) = packw;
        if (p.a_q8) *reinterpret_cast<uint2*>(p.a_q8 + (size_t)m * K + 8 * g) = make_uint2(qlo, qhi);
      }
    }
    __syncthreads();

    // ---- coalesced copy-out of the tail lists
    {
      const size_t rb = (size_t)m * R, rl = (size_t)m * p.tail_ld;
      for (int r = tid; r < R; r += NT) {
        const uint16_t ix = st_idx[r];
        if (p.tail_idx16) p.tail_idx16[rl + r] = ix;
        if (p.tail_val) p.tail_val[rl + r] = st_val[r];
        if (p.idx32) p.idx32[rb + r] = (int32_t)ix;
        if (p.top_q) p.top_q[rb + r] = st_q[r];
      }
      if (tid == 0) {
        p.body_scale[m] = bscale;
        if (p.top_scale) p.top_scale[m] = tscale;
      }
    }
    // (no barrier here: the next row touches the tail staging, the bf16 row, `red` and `res` only behind several
    // of its own barriers, which every thread of this row reaches after its copy-out)
  }
}

template <int KIND, int K, bool NORM>
int launch(const PrologueParams& p, cudaStream_t st) {
  auto kern = prologue_kernel<KIND, K, NORM>;
  const int Rpad = (p.R + 7) & ~7;
  const size_t smem = (size_t)K * 6 + (128 + 32 + 8 + 64 + 64 + ((K / 64 + 4) & ~3)) * 4 + (size_t)Rpad * 5 + 16;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && !(dev < 64 && configured[dev])) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return TQ_ERR_CUDA;
    }
    if (dev < 64) configured[dev] = true;
  }
  if (smem > 160 * 1024) return TQ_ERR_UNSUPPORTED;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int per_sm = 1;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NT, smem);
  if (per_sm < 1) per_sm = 1;
  int grid = sms * per_sm;
  if (grid > p.M) grid = p.M;
  kern<<<grid, NT, smem, st>>>(p);
  return check_launch();
}

#define TQ_CASE(KIND, KK) \
  if (kind == KIND && K == KK) return p.gamma ? launch<KIND, KK, true>(p, st) : launch<KIND, KK, false>(p, st);

int dispatch(int kind, int K, const PrologueParams& p, cudaStream_t st) {
  TQ_CASE(TQ_HAD_WHT, 512)
  TQ_CASE(TQ_HAD_WHT, 1024)
  TQ_CASE(TQ_HAD_WHT, 2048)
  TQ_CASE(TQ_HAD_WHT, 4096)
  TQ_CASE(TQ_HAD_WHT, 8192)
  TQ_CASE(TQ_HAD_KRON12, 6144)
  TQ_CASE(TQ_HAD_KRON12, 12288)
  TQ_CASE(TQ_HAD_BLOCK128, 2048)
  TQ_CASE(TQ_HAD_BLOCK128, 14336)
  TQ_CASE(TQ_HAD_NONE, 512)
  TQ_CASE(TQ_HAD_NONE, 1024)
  TQ_CASE(TQ_HAD_NONE, 2048)
  TQ_CASE(TQ_HAD_NONE, 6144)
  TQ_CASE(TQ_HAD_NONE, 4096)
  TQ_CASE(TQ_HAD_NONE, 8192)
  TQ_CASE(TQ_HAD_NONE, 12288)
  TQ_CASE(TQ_HAD_NONE, 14336)
  return TQ_ERR_UNSUPPORTED;
}
#undef TQ_CASE

float had_scale(int kind, int K) {
  if (kind == TQ_HAD_NONE) return 1.0f;
  const double n = (kind == TQ_HAD_BLOCK128) ? 128.0 : (double)K;
  return (float)(1.0 / sqrt(n));
}

}  // namespace

static int g_prologue_mode = -1;  // -1: specialised kernel where it is built; 0: general kernel only

int run_prologue(const void* x, int M, int K, int had_kind, int R, int dr, float eps, int scale_mode,
                 uint8_t* a_pack, int8_t* a_q8, float* body_scale, float* top_scale, uint16_t* tail_idx16,
                 void* tail_val, int tail_ld, uint16_t* tail_ptr, int ptr_ld, uint32_t* tail_rec, uint16_t* tail_cnt,
                 int32_t* idx32, int8_t* top_q, void* x_rot, const void* gamma, float rms_eps, cudaStream_t st,
                 int dtype, void* tail_dense) {
  if ((tail_idx16 || tail_val) && tail_ld < R) return TQ_ERR_BAD_ARG;
  if (gamma && !aligned16(gamma)) return TQ_ERR_MISALIGNED;
  if (tail_ptr && (ptr_ld < K / 128 + 1 || K % 128 != 0)) return TQ_ERR_BAD_ARG;
  if ((tail_rec != nullptr) != (tail_cnt != nullptr) || (tail_rec && K % 128 != 0)) return TQ_ERR_BAD_ARG;
  if (!x || (!a_pack && !a_q8) || !body_scale || M < 0 || K <= 0 || R < 0 || R >= K) return TQ_ERR_BAD_ARG;
  if (dr < 1 || dr > K) return TQ_ERR_BAD_ARG;
  if (!aligned16(x) || (a_pack && !aligned16(a_pack)) || (a_q8 && !aligned16(a_q8)) || (x_rot && !aligned16(x_rot)) ||
      (tail_dense && !aligned16(tail_dense)))
    return TQ_ERR_MISALIGNED;
  if (M == 0) return TQ_OK;
  PrologueParams p;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.M = M;
  p.R = R;
  p.dr = dr;
  p.tail_ld = tail_ld;
  p.ptr_ld = ptr_ld;
  p.tail_ptr = tail_ptr;
  p.tail_rec = tail_rec;
  p.tail_cnt = tail_cnt;
  p.eps = eps;
  p.hscale = had_scale(had_kind, K);
  p.scale_mode = scale_mode;
  p.a_pack = a_pack;
  p.a_q8 = a_q8;
  p.body_scale = body_scale;
  p.top_scale = top_scale;
  p.tail_idx16 = tail_idx16;
  p.tail_val = reinterpret_cast<uint16_t*>(tail_val);
  p.idx32 = idx32;
  p.top_q = top_q;
  p.x_rot = reinterpret_cast<uint16_t*>(x_rot);
  p.tail_dense = reinterpret_cast<uint16_t*>(tail_dense);
  p.gamma = reinterpret_cast<const uint16_t*>(gamma);
  p.rms_eps = rms_eps;
  // the kernel specialised for the benchmarked widths first (same outputs bit for bit); everything else, and
  // everything when tq_set_prologue_mode(0) asked for it, takes the general kernel
  // (A handful of rows -- decode -- is a latency problem, not a throughput one: the general kernel puts 256 threads
  // on a row and finishes a single 4096-wide row about 2 us earlier (a 12288-wide one 4 us later), so it keeps those
  // calls up to K = 8192 when it can serve them.  With
  // the fused RMSNorm the specialised kernel always runs: the two sum their squares in different orders, and a
  // row's result must not depend on how many rows came with it.)
  const bool few_rows = M <= 64 && K <= 8192 && !gamma && dtype == TQ_BF16;
  if (g_prologue_mode != 0 && !few_rows) {
    const int rc = run_prologue_fast(had_kind, K, dtype, p, st);
    if (rc != TQ_ERR_UNSUPPORTED) return rc;
  }
  if (dtype != TQ_BF16) return TQ_ERR_UNSUPPORTED;
  {
    const int rc = dispatch(had_kind, K, p, st);
    if (rc != TQ_ERR_UNSUPPORTED || g_prologue_mode == 0 || !few_rows) return rc;
  }
  return run_prologue_fast(had_kind, K, dtype, p, st);
}

}  // namespace tq

extern "C" int tq_split_prologue(const void* x, int M, int K, int had_kind, int R, int descending_rank,
                                 float eps, uint8_t* a_pack, int8_t* a_q8, float* body_scale, float* top_scale,
                                 uint16_t* tail_idx16, void* tail_val, int tail_ld, uint16_t* tail_ptr,
                                 int ptr_ld, uint32_t* tail_rec, uint16_t* tail_cnt, void* tail_dense, int32_t* idx32,
                                 int8_t* top_q, void* x_rot, void* stream) {
  return tq::run_prologue(x, M, K, had_kind, R, descending_rank, eps, 0, a_pack, a_q8, body_scale, top_scale,
                          tail_idx16, tail_val, tail_ld, tail_ptr, ptr_ld, tail_rec, tail_cnt, idx32, top_q, x_rot,
                          nullptr, 0.0f, (cudaStream_t)stream, TQ_BF16, tail_dense);
}

extern "C" int tq_set_prologue_mode(int mode) {
  if (mode < -1 || mode > 0) return TQ_ERR_BAD_ARG;
  tq::g_prologue_mode = mode;
  return TQ_OK;
}

extern "C" int tq_split_prologue_rmsnorm(const void* x, const void* gamma, float rms_eps, int M, int K, int had_kind,
                                         int R, int descending_rank, float eps, uint8_t* a_pack, int8_t* a_q8,
                                         float* body_scale, float* top_scale, uint16_t* tail_idx16, void* tail_val,
                                         int tail_ld, uint16_t* tail_ptr, int ptr_ld, uint32_t* tail_rec,
                                         uint16_t* tail_cnt, void* tail_dense, void* x_rot, void* stream) {
  if (!gamma) return TQ_ERR_BAD_ARG;
  return tq::run_prologue(x, M, K, had_kind, R, descending_rank, eps, 0, a_pack, a_q8, body_scale, top_scale,
                          tail_idx16, tail_val, tail_ld, tail_ptr, ptr_ld, tail_rec, tail_cnt, nullptr, nullptr, x_rot,
                          gamma, rms_eps, (cudaStream_t)stream, TQ_BF16, tail_dense);
}

extern "C" int tq_topr_pack(const void* A, int dtype, int M, int K, int R, int descending_rank,
                            uint8_t* A_pack, float* body_scale, float* top_scale, int8_t* top_q,
                            int32_t* idx, float eps, void* stream) {
  if (dtype != TQ_BF16 && dtype != TQ_FP16) return TQ_ERR_BAD_ARG;
  if (R > 0 && (!top_q || !idx || !top_scale)) return TQ_ERR_BAD_ARG;
  return tq::run_prologue(A, M, K, TQ_HAD_NONE, R, descending_rank, eps, 0, A_pack, nullptr, body_scale, top_scale,
                          nullptr, nullptr, 0, nullptr, 0, nullptr, nullptr, idx, top_q, nullptr, nullptr, 0.0f,
                          (cudaStream_t)stream, dtype, nullptr);
}
