// Fused quantise + pack kernels (bf16/fp16/fp32 -> packed signed int4 + fp32 scales).
//
// One pass over HBM: every element is loaded once with 128-bit loads, stays in registers
// between the absmax reduction (warp shuffles) and the quantise step, and leaves as packed
// 32-bit words (8 codes each).  The reference reads each row twice and uses one 256-thread
// block per 128-element group (int4_native_tc/csrc/int4_quant.cu:100-182, 759-803).
//
// Code arithmetic (shared with the CPU oracle): s = absmax / 7 (IEEE), q = clamp(rint(x / s), -8, 7)
// with IEEE division and round-half-even, q = 0 when absmax == 0.  The returned scale is
// max(s, 1/(7*512)) for activations (int4_quant.cu:97,142) and s or 1.0 (all-zero slice) for
// weights (int4_quant.cu:267).
#include "common.cuh"

namespace i4tc {

__device__ __forceinline__ float min_scale() { return 1.0f / (7.0f * 512.0f); }

__device__ __forceinline__ float scale_out(float absmax, int role) {
  float s = __fdiv_rn(absmax, 7.0f);
  if (role == I4TC_ROLE_ACTIVATION) return fmaxf(s, min_scale());
  return absmax == 0.0f ? 1.0f : s;
}

// Eight consecutive elements.  bf16 keeps the raw 128 bits (4 registers) and widens on use; the
// absmax is taken on the packed halves (|x| and max are exact in bf16).  Other types are widened
// at load time.
template <typename T>
struct Vec8 {
  float v[8];
  __device__ __forceinline__ void load(const T* p);
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
  __device__ __forceinline__ float get(int i) const { return v[i]; }
  __device__ __forceinline__ void set_all(const float (&f)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = f[i];
  }
  __device__ __forceinline__ float absmax() const {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
  }
};

template <>
struct Vec8<__nv_bfloat16> {
  uint32_t w[4];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    w[0] = u.x; w[1] = u.y; w[2] = u.z; w[3] = u.w;
  }
  __device__ __forceinline__ void zero() { w[0] = w[1] = w[2] = w[3] = 0u; }
  __device__ __forceinline__ float get(int i) const {
    return (i & 1) ? __uint_as_float(w[i >> 1] & 0xFFFF0000u) : __uint_as_float(w[i >> 1] << 16);
  }
  __device__ __forceinline__ void set_all(const float (&f)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  // |x| maxima of the two 16-bit halves, still packed (max and abs are exact in bf16)
  __device__ __forceinline__ __nv_bfloat162 absmax2() const {
    __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[0]));
#pragma unroll
    for (int i = 1; i < 4; ++i) m = __hmax2(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i])));
    return m;
  }
  __device__ __forceinline__ float absmax() const { return widen_max(absmax2()); }
  // bf16 -> fp32 by moving the 16 bits up (integer pipe; the conversion instruction is much slower)
  static __device__ __forceinline__ float widen_max(__nv_bfloat162 m) {
    const uint32_t b = *reinterpret_cast<const uint32_t*>(&m);
    return fmaxf(__uint_as_float(b << 16), __uint_as_float(b & 0xFFFF0000u));
  }
};

template <>
__device__ __forceinline__ void Vec8<__half>::load(const __half* p) {
  uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __half22float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void Vec8<float>::load(const float* p) {
  float4 a = __ldg(reinterpret_cast<const float4*>(p));
  float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename T>
__device__ __forceinline__ float absmax8(const Vec8<T>& x) { return x.absmax(); }

// Eight codes -> one 32-bit word, element 0 in the lowest nibble.  Exact-division path.
template <typename T>
__device__ __forceinline__ uint32_t pack8_div(const Vec8<T>& x, float s) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) w |= code4(x.get(i), s) << (4 * i);
  return w;
}

// Reciprocal of the divisor for the fast path.  rcp.approx is within 2^-23 of 1/s; `fast` is false
// when r is not a normal number of moderate size, and then every vector takes the exact path.
struct Recip {
  float r;      // approximately 1 / divisor
  float base;   // absmax (FROM_ABSMAX) or the divisor itself
  bool fast;
};
// FROM_ABSMAX: the divisor is absmax / 7, so r = 7 * rcp(absmax) (within 2^-22 of 1 / RN(absmax/7));
// the IEEE division absmax / 7 is then only needed on the rare exact path.
template <bool FROM_ABSMAX>
__device__ __forceinline__ Recip make_recip(float base) {
  Recip q;
  q.base = base;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(q.r) : "f"(base));
  if (FROM_ABSMAX) q.r *= 7.0f;
  q.fast = (q.r > 7.8886090522e-31f) && (q.r < 1.2676506002e30f);  // 2^-100 < r < 2^100
  return q;
}
template <bool FROM_ABSMAX>
__device__ __forceinline__ float exact_divisor(const Recip& q) {
  return FROM_ABSMAX ? __fdiv_rn(q.base, 7.0f) : q.base;
}

// Exact code (+8) of an element whose quotient lies within ~1e-5 of a rounding boundary h = k + 0.5.
// No division: with a = |x|, e1 = h*s - a is exactly representable (a is that close to h*s), and
// RN(a/s) <= h, = h or >= h is decided by comparing e1 with half an ulp of h times s, also exact.
// rint's tie-to-even then picks k or k+1.  (a/s can never equal the 25-bit midpoint h +- ulp/2.)
__device__ __forceinline__ float exact_tie_code8(float x, float y8, float s) {
  const float a = fabsf(x);
  const float kf = rintf(fabsf(y8 - 8.0f) - 0.5f);      // k >= 0
  const float h = kf + 0.5f;
  const float e1 = fmaf(h, s, -a);                       // exact
  const float pw = __uint_as_float(__float_as_uint(h) & 0x7F800000u);
  const float cs = pw * (s * 5.9604644775390625e-08f);   // (ulp(h) / 2) * s, exact
  const bool odd = (__float2int_rn(kf) & 1) != 0;
  // k even: RN(a/s) <= h rounds to k, above h to k+1.  k odd: RN(a/s) >= h rounds to k+1, below to k.
  const float mag = odd ? ((e1 > cs) ? kf : kf + 1.0f) : ((-e1 > cs) ? kf + 1.0f : kf);
  return copysignf(mag, x) + 8.0f;
}

// Same result as pack8_div, bit for bit, at a fraction of the instructions (packed f32x2 math).
//   y8 = x*r + 8 (one FMA)      u = y8 + 1.5*2^23 rounds y8 to the nearest-even integer n+8 in [0,15]
//   v  = u - 1.5*2^23 = n+8     the eight v's are combined with exact FMAs (16 bits per half)
// |y8 - 8 - RN(x/s)| < 3e-6 for |x/s| <= 8 (r within 2^-22 of 1/s, one rounding in the FMA, one in
// the exact quotient), so unless y8 lies within 1e-5 of a rounding boundary (k + 0.5) the rounded
// integer is that of the exact division.  Elements inside that window (bf16 data produce exact
// ties in about one element per thousand) are decided exactly by exact_tie_code8.
// CLAMP: the caller supplied the divisor, so x/s may leave [-8, 7].
template <typename T, bool CLAMP>
__device__ __forceinline__ uint32_t pack8(const Vec8<T>& x, const Recip& q, bool zero) {
  if (zero) return 0u;
  if (!q.fast) return pack8_div(x, exact_divisor<!CLAMP>(q));
  constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
  constexpr float kThr = 0.5f - 1e-5f;
  const float2 r2 = make_float2(q.r, q.r), eight = make_float2(8.f, 8.f), mg = make_float2(kMagic, kMagic);
  const float2 nmg = make_float2(-kMagic, -kMagic);
  float2 v[4];  // v[i] = (n_i + 8, n_{i+4} + 8)
  float2 e[CLAMP ? 4 : 1];   // CLAMP: e[i] = y8 - v[i] (exact), kept for the rare path
  float worst = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 y8 = __ffma2_rn(make_float2(x.get(i), x.get(i + 4)), r2, eight);
    if (CLAMP) {
      y8.x = fminf(fmaxf(y8.x, 0.0f), 15.0f);
      y8.y = fminf(fmaxf(y8.y, 0.0f), 15.0f);
    }
    v[i] = __fadd2_rn(__fadd2_rn(y8, mg), nmg);
    const float2 d = __ffma2_rn(v[i], make_float2(-1.f, -1.f), y8);
    if (CLAMP) e[i] = d;
    worst = fmaxf(worst, fmaxf(fabsf(d.x), fabsf(d.y)));
  }
  if (!(worst <= kThr)) {
    // rare: some element sits on a rounding boundary
    const float s = exact_divisor<!CLAMP>(q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (CLAMP) {
        // y8 = v + e exactly (v is y8 rounded to an integer, e the exact remainder): nothing is recomputed
        if (!(fabsf(e[i].x) <= kThr)) v[i].x = exact_tie_code8(x.get(i), v[i].x + e[i].x, s);
        if (!(fabsf(e[i].y) <= kThr)) v[i].y = exact_tie_code8(x.get(i + 4), v[i].y + e[i].y, s);
      } else {
        // (the absmax kernels run at four blocks per SM with 64 registers: recomputing is cheaper than keeping e)
        const float y0 = fmaf(x.get(i), q.r, 8.0f), y1 = fmaf(x.get(i + 4), q.r, 8.0f);
        if (!(fabsf(y0 - v[i].x) <= kThr)) v[i].x = exact_tie_code8(x.get(i), y0, s);
        if (!(fabsf(y1 - v[i].y) <= kThr)) v[i].y = exact_tie_code8(x.get(i + 4), y1, s);
      }
    }
  }
  // (lo, hi) = v0 + 16 v1 + 256 v2 + 4096 v3 for elements 0..3 and 4..7: exact, below 2^16
  float2 lh = __ffma2_rn(v[3], make_float2(4096.f, 4096.f),
                         __ffma2_rn(v[2], make_float2(256.f, 256.f), __ffma2_rn(v[1], make_float2(16.f, 16.f), v[0])));
  lh = __fadd2_rn(lh, mg);
  const uint32_t wl = __float_as_uint(lh.x) & 0xFFFFu;
  const uint32_t wh = __float_as_uint(lh.y) << 16;
  return (wl | wh) ^ 0x88888888u;  // offset-binary nibbles (n+8) -> two's complement
}

// e**t for t clamped to [-87, 87] as a fixed sequence of correctly rounded fp32 operations (never contracted into
// fused multiply-adds): n = rint(t * log2(e)); r = (t - n * ln2_hi) - n * ln2_lo; degree-7 Taylor polynomial of r by
// Horner's rule; times 2**n.  A CPU repeats it bit for bit with plain IEEE single-precision arithmetic.
__device__ __forceinline__ float exp_reproducible(float t) {
  t = fminf(fmaxf(t, -87.0f), 87.0f);
  const float n = rintf(__fmul_rn(t, 1.4426950408889634f));
  const float r = __fsub_rn(__fsub_rn(t, __fmul_rn(n, 0.693145751953125f)), __fmul_rn(n, 1.428606765330187045e-06f));
  float p = 1.0f / 5040.0f;
  p = __fadd_rn(__fmul_rn(p, r), 1.0f / 720.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f / 120.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f / 24.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f / 6.0f);
  p = __fadd_rn(__fmul_rn(p, r), 0.5f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  return __fmul_rn(p, __int_as_float(((int)n + 127) << 23));   // |n| <= 126: an exact power of two
}

// (g * sigmoid(g)) * u with sigmoid(g) = 1 / (1 + exp_reproducible(-g)): the definition of SwiGLU here.
__device__ __forceinline__ float silu_mul_reproducible(float g, float u) {
  const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_reproducible(-g)));
  return __fmul_rn(__fmul_rn(g, sig), u);
}

// silu(g) * u rounded to bf16 and widened again: the value the next quantiser sees, bit-identical to
// bf16(silu_mul_reproducible(g, u)).  The fast evaluation (exp through the special-function unit, documented error
// 2 + |1.173 x| ulp, and a correctly rounded reciprocal) is within ~17 ulp of that definition for |g| <= 8; it decides
// the bf16 rounding unless the fp32 value lies within 32 ulp of a rounding boundary (one element in a thousand),
// and only those elements and the rare |g| > 8 are evaluated by the definition itself.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  const float sig = __frcp_rn(1.0f + __expf(-g));
  float y = __fmul_rn(__fmul_rn(g, sig), u);
  const uint32_t low = __float_as_uint(y) & 0xFFFFu;
  const bool near_boundary = (low - (0x8000u - 32u)) <= 64u;
  if (near_boundary || !(fabsf(g) <= 8.0f)) y = silu_mul_reproducible(g, u);
  return __bfloat162float(__float2bfloat16_rn(y));
}

// ------------------------------------------------------------------------------------------
// Grouped kernel.  Block = 8 warps = 8 consecutive rows; each warp owns a 1024-element segment
// of its row (4 x 128-bit loads per lane, all issued before the first use).  A group of
// 8*LPG elements lives in LPG adjacent lanes, so its absmax is log2(LPG) shuffles.
// MODE 0: rows of x.  MODE 1: rows gathered through row_index[r] / index_div.
// MODE 2: input is bf16 [rows, 2*K] laid out [gate | up]; the quantised value is
//         bf16(silu(gate) * up).
// MODE 3: RMSNorm first: the quantised value is bf16(bf16(x * rsqrt(mean(x^2) + eps)) * aux[k]); a warp then
//         needs its whole row (the grid is not split along K).
// GIVEN: divisors come from `given_scale` (group-major) instead of the absmax.
// ------------------------------------------------------------------------------------------
constexpr int kQRows = 8;
constexpr int kQVecs = 4;                 // 8-element vectors per lane per segment
constexpr int kQLane = 8 * kQVecs;        // 32 consecutive elements per lane
constexpr int kQSeg = 32 * kQLane;        // 1024 elements per warp per segment

// round to bf16 and widen again
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <typename T, int MODE>
__device__ __forceinline__ void load_segment(Vec8<T> (&v)[kQVecs], const T* src, int k, int K, bool row_ok,
                                             const T* aux = nullptr, float row_factor = 0.f) {
  // k = first element of this lane; K % 32 == 0, so the lane's 32 elements are all in range or none
  if (row_ok && k < K) {
#pragma unroll
    for (int j = 0; j < kQVecs; ++j) {
      if (MODE == 2) {
        Vec8<T> g, u;
        g.load(src + k + 8 * j);
        u.load(src + K + k + 8 * j);
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = silu_mul_bf16(g.get(i), u.get(i));
        v[j].set_all(f);
      } else if (MODE == 3) {
        // RMSNorm in front of the quantiser: bf16(bf16(x * inv_rms) * weight), the roundings of an unfused
        // normalisation that works in fp32 and returns the input's type
        Vec8<T> xv, wv;
        xv.load(src + k + 8 * j);
        wv.load(aux + k + 8 * j);
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = bf16_round(bf16_round(xv.get(i) * row_factor) * wv.get(i));
        v[j].set_all(f);
      } else {
        v[j].load(src + k + 8 * j);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < kQVecs; ++j) v[j].zero();
  }
}

template <typename T>
__device__ __forceinline__ float absmax_of(const Vec8<T> (&v)[kQVecs]) {
  float m = 0.f;
#pragma unroll
  for (int j = 0; j < kQVecs; ++j) m = fmaxf(m, v[j].absmax());
  return m;
}
template <>
__device__ __forceinline__ float absmax_of<__nv_bfloat16>(const Vec8<__nv_bfloat16> (&v)[kQVecs]) {
  __nv_bfloat162 m = v[0].absmax2();
#pragma unroll
  for (int j = 1; j < kQVecs; ++j) m = __hmax2(m, v[j].absmax2());
  return Vec8<__nv_bfloat16>::widen_max(m);
}

// Block = 8 warps = 8 consecutive rows (the warps are independent).  In a segment every lane owns 32 consecutive elements
// (64 bytes of bf16), so a group of GS elements is LPG = GS/32 adjacent lanes: its absmax costs
// log2(LPG) shuffles, its reciprocal is formed once per lane, and each lane leaves 16 packed bytes
// with one 128-bit store.  The block walks `segs_per_block` segments of its rows and loads segment
// s+1 while it quantises segment s.
// OUTMAP (expert-parallel MoE): output row r goes to row out.row_map[r] (skipped when negative) of a layout given by
// byte / float strides instead of the group-major default, and rows at or beyond *out.rows_dev are skipped.
struct QuantOutMap {
  const int32_t* row_map;   // nullptr: identity
  const int32_t* rows_dev;  // nullptr: all `rows`
  long long pk_gstride, pk_rstride;   // bytes between groups / rows of the packed output
  long long sc_gstride, sc_rstride;   // floats between groups / rows of the scale output
  // Peer destinations (nullptr: one local buffer).  Mapped row m lies in block m / block_rows; that block's rows go
  // to the buffer at dest_bases[block] (another GPU's memory, written with plain stores over NVLink), where this
  // rank's block is number my_block: row my_block * block_rows + m % block_rows.  scale_offset = bytes from a row's
  // codes to its scales.
  const unsigned long long* dest_bases;
  int block_rows, my_block;
  long long scale_offset;
};

template <typename T, int LPG, int MODE, bool GIVEN, bool OUTMAP = false>
__global__ void __launch_bounds__(256) quant_grouped_kernel(
    const T* __restrict__ x, int64_t rows, int K, int64_t ldx, const int32_t* __restrict__ row_index,
    int index_div, int64_t src_rows, const float* __restrict__ given_scale, uint8_t* __restrict__ packed,
    float* __restrict__ scale, int role, int segs_per_block, const T* __restrict__ aux, float eps,
    QuantOutMap out = QuantOutMap{nullptr, nullptr, 0, 0, 0, 0, nullptr, 1, 0, 0}) {
  constexpr int GS = LPG * kQLane;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = (int64_t)blockIdx.x * kQRows;
  const int64_t r = r0 + warp;
  bool row_ok = r < rows;
  int64_t orow = r;
  if (OUTMAP) {
    if (out.rows_dev != nullptr && r >= (int64_t)__ldg(out.rows_dev)) row_ok = false;
    if (row_ok && out.row_map != nullptr) {
      orow = __ldg(out.row_map + r);
      if (orow < 0) row_ok = false;
    }
  }
  const int nseg = (K + kQSeg - 1) / kQSeg;
  const int seg_begin = blockIdx.y * segs_per_block;
  const int seg_end = min(nseg, seg_begin + segs_per_block);

  const T* src = nullptr;
  bool src_ok = row_ok;   // MODE 1: false for a pair index that names no row of x (such a row is quantised as zeros)
  if (row_ok) {
    int64_t sr = r;
    if (MODE == 1) {
      const int idx = row_index[r];
      sr = idx / index_div;
      src_ok = idx >= 0 && sr < src_rows;
    }
    if (src_ok) src = x + sr * ldx;
  }
  float row_factor = 0.f;
  if (MODE == 3) {
    // first pass over the row: sum of squares in fp32 (the second pass below hits L1/L2)
    float ss = 0.f;
    if (row_ok) {
      for (int k = lane * kQLane; k < K; k += kQSeg) {
#pragma unroll
        for (int j = 0; j < kQVecs; ++j) {
          Vec8<T> xv;
          xv.load(src + k + 8 * j);
#pragma unroll
          for (int i = 0; i < 8; ++i) ss = fmaf(xv.get(i), xv.get(i), ss);
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    // correctly rounded division, addition and reciprocal square root: a CPU can repeat the row statistic exactly
    row_factor = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps));
  }
  Vec8<T> cur[kQVecs], nxt[kQVecs];
  load_segment<T, MODE>(cur, src, seg_begin * kQSeg + lane * kQLane, K, src_ok, aux, row_factor);
  for (int seg = seg_begin; seg < seg_end; ++seg) {
    const int k = seg * kQSeg + lane * kQLane;
    if (seg + 1 < seg_end) load_segment<T, MODE>(nxt, src, k + kQSeg, K, src_ok, aux, row_factor);
    const bool ok = row_ok && k < K;
    const int g = k / GS;
    Recip q;
    float absmax = 0.f;
    if (GIVEN) {
      q = make_recip<false>(ok ? __ldg(given_scale + (int64_t)g * rows + r) : 1.f);
    } else {
      absmax = absmax_of(cur);
#pragma unroll
      for (int o = 1; o < LPG; o <<= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, o));
      q = make_recip<true>(absmax);
      // one lane per group writes the scale (the IEEE division absmax / 7 happens here, off the
      // per-element path); neighbouring rows fill the same 32-byte sector from other warps
      if (ok && (lane % LPG) == 0) {
        if (OUTMAP) {
          float* sdst = scale + (int64_t)g * out.sc_gstride + orow * out.sc_rstride;
          if (out.dest_bases != nullptr) {
            const int blk = (int)(orow / out.block_rows);
            const int64_t prow = (int64_t)out.my_block * out.block_rows + (orow - (int64_t)blk * out.block_rows);
            sdst = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(out.dest_bases[blk]) + prow * out.pk_rstride +
                                            out.scale_offset) + (int64_t)g * out.sc_gstride;
          }
          *sdst = scale_out(absmax, role);
        } else {
          scale[(int64_t)g * rows + r] = scale_out(absmax, role);
        }
      }
    }
    if (ok) {
      const bool zero = !GIVEN && absmax == 0.f;
      uint4 w;
      w.x = pack8<T, GIVEN>(cur[0], q, zero);
      w.y = pack8<T, GIVEN>(cur[1], q, zero);
      w.z = pack8<T, GIVEN>(cur[2], q, zero);
      w.w = pack8<T, GIVEN>(cur[3], q, zero);
      uint8_t* dst = OUTMAP ? packed + (int64_t)g * out.pk_gstride + orow * out.pk_rstride + (lane % LPG) * 16
                            : packed + ((int64_t)g * rows + r) * (GS / 2) + (lane % LPG) * 16;
      if (OUTMAP && out.dest_bases != nullptr) {
        const int blk = (int)(orow / out.block_rows);
        const int64_t prow = (int64_t)out.my_block * out.block_rows + (orow - (int64_t)blk * out.block_rows);
        dst = reinterpret_cast<uint8_t*>(out.dest_bases[blk]) + prow * out.pk_rstride + (int64_t)g * out.pk_gstride +
              (lane % LPG) * 16;
      }
      *reinterpret_cast<uint4*>(dst) = w;
    }
#pragma unroll
    for (int j = 0; j < kQVecs; ++j) cur[j] = nxt[j];
  }
}

// ------------------------------------------------------------------------------------------
// Clipped symmetric and asymmetric per-group quantisers on the layout of the grouped kernel above (a lane owns 32
// consecutive elements, a group is LPG adjacent lanes, 128-bit loads and stores, next segment loaded while this one is
// quantised).  Arithmetic per group, IEEE fp32:
//   t = max|x| * clip
//   symmetric:  s = t / 7;  code = clamp(rint(x / s), -8, 7), 0 when s == 0;  scale = max(s, 1/(7*512))
//   asymmetric: c = clamp(x, -t, t);  s = max((max c - min c) / 15, 1/(7*512));  azp = clamp(rint(-min c / s), 0, 15);
//               u = clamp(rint(c / s + azp), 0, 15);  stored nibble = u - 8;  azp_adj = 8 - azp
// ------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void minmax_of(const Vec8<T> (&v)[kQVecs], float& mn, float& mx) {
  mn = INFINITY;
  mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kQVecs; ++j) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mn = fminf(mn, v[j].v[i]);
      mx = fmaxf(mx, v[j].v[i]);
    }
  }
}
template <>
__device__ __forceinline__ void minmax_of<__nv_bfloat16>(const Vec8<__nv_bfloat16> (&v)[kQVecs], float& mn, float& mx) {
  // min and max of packed bf16 halves are exact
  __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v[0].w[0]), hi = lo;
#pragma unroll
  for (int j = 0; j < kQVecs; ++j) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&v[j].w[i]);
      lo = __hmin2(lo, h);
      hi = __hmax2(hi, h);
    }
  }
  const uint32_t bl = *reinterpret_cast<const uint32_t*>(&lo), bh = *reinterpret_cast<const uint32_t*>(&hi);
  mn = fminf(__uint_as_float(bl << 16), __uint_as_float(bl & 0xFFFF0000u));
  mx = fmaxf(__uint_as_float(bh << 16), __uint_as_float(bh & 0xFFFF0000u));
}

// Parameters of one asymmetric group, the same in all its lanes.
struct AsymGroup {
  float thr, s, r, azp;   // clip range, step, ~1/step, zero point
  float ylo, yhi;         // images of -thr / +thr under y = c * r + azp, intersected with [0, 15]
  bool fast;
};

// Eight unsigned codes u (stored as u - 8).  Fast path: y = x * r + azp in one FMA.  The FMA is monotone in x, so
// clamping y to [y(-thr), y(thr)] equals clamping x first; intersected with [0, 15] that is one clamp per element.
// For |c / s| < 64 the FMA lies within 2e-5 of RN(RN(c / s) + azp), so outside 1e-4 of a rounding boundary both round to
// the same integer; for |c / s| >= 64 both saturate on the same side.  Elements inside the window take the IEEE
// division.
template <typename T>
__device__ __forceinline__ uint32_t pack8_asym(const Vec8<T>& x, const AsymGroup& q) {
  constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
  constexpr float kThr = 0.5f - 1e-4f;
  const float2 r2 = make_float2(q.r, q.r), az = make_float2(q.azp, q.azp), mg = make_float2(kMagic, kMagic);
  const float2 nmg = make_float2(-kMagic, -kMagic);
  float2 v[4], y[4];
  float worst = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    y[i] = __ffma2_rn(make_float2(x.get(i), x.get(i + 4)), r2, az);
    y[i].x = fminf(fmaxf(y[i].x, q.ylo), q.yhi);
    y[i].y = fminf(fmaxf(y[i].y, q.ylo), q.yhi);
    v[i] = __fadd2_rn(__fadd2_rn(y[i], mg), nmg);
    const float2 e = __ffma2_rn(v[i], make_float2(-1.f, -1.f), y[i]);
    worst = fmaxf(worst, fmaxf(fabsf(e.x), fabsf(e.y)));
  }
  if (!q.fast || !(worst <= kThr)) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (!q.fast || !(fabsf(y[i].x - v[i].x) <= kThr)) {
        const float c = fminf(fmaxf(x.get(i), -q.thr), q.thr);
        v[i].x = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(c, q.s), q.azp)), 0.0f), 15.0f);
      }
      if (!q.fast || !(fabsf(y[i].y - v[i].y) <= kThr)) {
        const float c = fminf(fmaxf(x.get(i + 4), -q.thr), q.thr);
        v[i].y = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(c, q.s), q.azp)), 0.0f), 15.0f);
      }
    }
  }
  float2 lh = __ffma2_rn(v[3], make_float2(4096.f, 4096.f),
                         __ffma2_rn(v[2], make_float2(256.f, 256.f), __ffma2_rn(v[1], make_float2(16.f, 16.f), v[0])));
  lh = __fadd2_rn(lh, mg);
  const uint32_t wl = __float_as_uint(lh.x) & 0xFFFFu;
  const uint32_t wh = __float_as_uint(lh.y) << 16;
  return (wl | wh) ^ 0x88888888u;   // u - 8 as a two's-complement nibble is u ^ 8
}

template <typename T, int LPG, bool ASYM>
__global__ void __launch_bounds__(256) quant_grouped_ext_kernel(const T* __restrict__ x, int64_t rows, int K,
                                                                int64_t ldx, float clip, uint8_t* __restrict__ packed,
                                                                float* __restrict__ scale,
                                                                float* __restrict__ azp_adj, int segs_per_block) {
  constexpr int GS = LPG * kQLane;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * kQRows + warp;
  const bool row_ok = r < rows;
  const int nseg = (K + kQSeg - 1) / kQSeg;
  const int seg_begin = blockIdx.y * segs_per_block;
  const int seg_end = min(nseg, seg_begin + segs_per_block);
  const T* src = row_ok ? x + r * ldx : nullptr;
  Vec8<T> cur[kQVecs], nxt[kQVecs];
  load_segment<T, 0>(cur, src, seg_begin * kQSeg + lane * kQLane, K, row_ok);
  for (int seg = seg_begin; seg < seg_end; ++seg) {
    const int k = seg * kQSeg + lane * kQLane;
    if (seg + 1 < seg_end) load_segment<T, 0>(nxt, src, k + kQSeg, K, row_ok);
    const bool ok = row_ok && k < K;
    const int g = k / GS;
    float mn, mx;
    minmax_of(cur, mn, mx);
#pragma unroll
    for (int o = 1; o < LPG; o <<= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    const float thr = __fmul_rn(fmaxf(-mn, mx), clip);
    uint4 w;
    if (ASYM) {
      AsymGroup q;
      q.thr = thr;
      const float cmn = fminf(fmaxf(mn, -thr), thr), cmx = fminf(fmaxf(mx, -thr), thr);
      q.s = fmaxf(__fdiv_rn(__fsub_rn(cmx, cmn), 15.0f), min_scale());
      q.azp = fminf(fmaxf(rintf(__fdiv_rn(-cmn, q.s)), 0.0f), 15.0f);
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(q.r) : "f"(q.s));
      q.fast = (q.r > 7.8886090522e-31f) && (q.r < 1.2676506002e30f);
      q.ylo = fmaxf(fmaf(-thr, q.r, q.azp), 0.0f);
      q.yhi = fminf(fmaf(thr, q.r, q.azp), 15.0f);
      if (ok && (lane % LPG) == 0) {
        scale[(int64_t)g * rows + r] = q.s;
        azp_adj[(int64_t)g * rows + r] = 8.0f - q.azp;
      }
      w.x = pack8_asym<T>(cur[0], q);
      w.y = pack8_asym<T>(cur[1], q);
      w.z = pack8_asym<T>(cur[2], q);
      w.w = pack8_asym<T>(cur[3], q);
    } else {
      const float s = __fdiv_rn(thr, 7.0f);
      const bool zero = !(s > 0.0f);
      const Recip q = make_recip<false>(zero ? 1.0f : s);
      if (ok && (lane % LPG) == 0) scale[(int64_t)g * rows + r] = fmaxf(s, min_scale());
      w.x = pack8<T, true>(cur[0], q, zero);
      w.y = pack8<T, true>(cur[1], q, zero);
      w.z = pack8<T, true>(cur[2], q, zero);
      w.w = pack8<T, true>(cur[3], q, zero);
    }
    if (ok) *reinterpret_cast<uint4*>(packed + ((int64_t)g * rows + r) * (GS / 2) + (lane % LPG) * 16) = w;
#pragma unroll
    for (int j = 0; j < kQVecs; ++j) cur[j] = nxt[j];
  }
}

template <typename T, bool ASYM>
static int launch_grouped_ext_t(const T* x, int64_t rows, int64_t K, int64_t ldx, int gs, float clip, uint8_t* packed,
                                float* scale, float* azp_adj, cudaStream_t st) {
  const int64_t row_blocks = (rows + kQRows - 1) / kQRows;
  const int nseg = (int)((K + kQSeg - 1) / kQSeg);
  int spb = nseg;
  if (row_blocks < 2048) spb = (int)((int64_t)nseg * row_blocks / 2048);
  if (spb < 1) spb = 1;
  dim3 grid((unsigned)row_blocks, (unsigned)((nseg + spb - 1) / spb));
  I4TC_REQUIRE(grid.y <= 65535, I4TC_EINVAL, "K=%lld too large for the grouped quantiser", (long long)K);
  switch (gs) {
    case 64: quant_grouped_ext_kernel<T, 2, ASYM><<<grid, 256, 0, st>>>(x, rows, (int)K, ldx, clip, packed, scale, azp_adj, spb); break;
    case 128: quant_grouped_ext_kernel<T, 4, ASYM><<<grid, 256, 0, st>>>(x, rows, (int)K, ldx, clip, packed, scale, azp_adj, spb); break;
    case 256: quant_grouped_ext_kernel<T, 8, ASYM><<<grid, 256, 0, st>>>(x, rows, (int)K, ldx, clip, packed, scale, azp_adj, spb); break;
    default: return fail(I4TC_EUNSUPPORTED, "group_size=%d not supported (64, 128 or 256)", gs);
  }
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

// Whether the vectorised kernel can take this call: 16-byte aligned rows and outputs (it moves 128 bits per lane).
bool grouped_ext_fast_ok(const void* x, int64_t ldx, const uint8_t* packed) {
  return aligned_to(x, 16) && (ldx * 2) % 16 == 0 && aligned_to(packed, 16);
}

int launch_grouped_ext(bool asym, const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, int gs, float clip,
                       uint8_t* packed, float* scale, float* azp_adj, cudaStream_t st) {
  if (dtype == I4TC_BF16) {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(x);
    return asym ? launch_grouped_ext_t<__nv_bfloat16, true>(p, rows, K, ldx, gs, clip, packed, scale, azp_adj, st)
                : launch_grouped_ext_t<__nv_bfloat16, false>(p, rows, K, ldx, gs, clip, packed, scale, azp_adj, st);
  }
  if (dtype == I4TC_FP16) {
    const __half* p = static_cast<const __half*>(x);
    return asym ? launch_grouped_ext_t<__half, true>(p, rows, K, ldx, gs, clip, packed, scale, azp_adj, st)
                : launch_grouped_ext_t<__half, false>(p, rows, K, ldx, gs, clip, packed, scale, azp_adj, st);
  }
  return fail(I4TC_EUNSUPPORTED, "input must be bf16 or fp16 (dtype %d)", dtype);
}

// ------------------------------------------------------------------------------------------
// Row-wise kernel.  One 256-thread block per row; the row is cached in registers
// (NCH chunks of 2048 elements, 8 per thread per chunk), so HBM is read once.
// ------------------------------------------------------------------------------------------
template <typename T, int NCH, bool GIVEN>
__global__ void __launch_bounds__(256) quant_rowwise_kernel(const T* __restrict__ x, int K, int64_t ldx,
                                                            const float* __restrict__ given_scale,
                                                            uint8_t* __restrict__ packed,
                                                            float* __restrict__ scale, int role) {
  __shared__ float s_max[8];
  const int64_t r = blockIdx.x;
  const T* src = x + r * ldx;
  const int t = threadIdx.x;
  Vec8<T> v[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = c * 2048 + t * 8;
    if (k < K) v[c].load(src + k); else v[c].zero();
  }
  float divisor, absmax = 0.f;
  if (GIVEN) {
    divisor = __ldg(given_scale + r);
  } else {
#pragma unroll
    for (int c = 0; c < NCH; ++c) absmax = fmaxf(absmax, absmax8(v[c]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, o));
    if ((t & 31) == 0) s_max[t >> 5] = absmax;
    __syncthreads();
    absmax = s_max[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) absmax = fmaxf(absmax, s_max[i]);
    if (t == 0) scale[r] = scale_out(absmax, role);
  }
  uint8_t* dst = packed + r * (int64_t)(K / 2);
  const Recip rcp = GIVEN ? make_recip<false>(divisor) : make_recip<true>(absmax);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = c * 2048 + t * 8;
    if (k < K) *reinterpret_cast<uint32_t*>(dst + k / 2) = pack8<T, GIVEN>(v[c], rcp, !GIVEN && absmax == 0.f);
  }
}

// Any even K, any alignment, any row length: two passes (the second one hits L2).
template <typename T, bool GIVEN>
__global__ void __launch_bounds__(256) quant_rowwise_generic_kernel(const T* __restrict__ x, int64_t K,
                                                                    int64_t ldx,
                                                                    const float* __restrict__ given_scale,
                                                                    uint8_t* __restrict__ packed,
                                                                    float* __restrict__ scale, int role) {
  __shared__ float s_max[8];
  const int64_t r = blockIdx.x;
  const T* src = x + r * ldx;
  const int t = threadIdx.x;
  float divisor, absmax = 0.f;
  if (GIVEN) {
    divisor = __ldg(given_scale + r);
  } else {
    for (int64_t k = t; k < K; k += 256) absmax = fmaxf(absmax, fabsf(to_f32(src[k])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, o));
    if ((t & 31) == 0) s_max[t >> 5] = absmax;
    __syncthreads();
    absmax = s_max[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) absmax = fmaxf(absmax, s_max[i]);
    divisor = __fdiv_rn(absmax, 7.0f);
    if (t == 0) scale[r] = scale_out(absmax, role);
  }
  const bool zero = !GIVEN && absmax == 0.f;
  uint8_t* dst = packed + r * (K / 2);
  for (int64_t i = t; i < K / 2; i += 256) {
    uint32_t lo = zero ? 0u : code4(to_f32(src[2 * i]), divisor);
    uint32_t hi = zero ? 0u : code4(to_f32(src[2 * i + 1]), divisor);
    dst[i] = (uint8_t)((hi << 4) | lo);
  }
}

// packed [n_words*4 bytes] -> int8, eight codes per thread-iteration.
__global__ void unpack_int4_kernel(const uint8_t* __restrict__ packed, int64_t n_bytes, int8_t* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t n_words = n_bytes / 4;
  const bool al = ((reinterpret_cast<uintptr_t>(packed) & 3) == 0) && ((reinterpret_cast<uintptr_t>(out) & 7) == 0);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
    if (al) {
      const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(packed) + i);
      // byte b of w holds codes 2b (low nibble) and 2b+1 (high nibble)
      uint32_t o[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t acc = 0;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const uint32_t byte = (w >> (8 * (2 * h + b))) & 0xFFu;
          const int lo = ((int)(byte << 28)) >> 28;
          const int hi = ((int)(byte << 24)) >> 28;
          acc |= ((uint32_t)lo & 0xFFu) << (16 * b);
          acc |= ((uint32_t)hi & 0xFFu) << (16 * b + 8);
        }
        o[h] = acc;
      }
      *reinterpret_cast<uint2*>(out + 8 * i) = make_uint2(o[0], o[1]);
    } else {
      for (int b = 0; b < 4; ++b) {
        const uint32_t byte = packed[4 * i + b];
        out[8 * i + 2 * b] = (int8_t)(((int)(byte << 28)) >> 28);
        out[8 * i + 2 * b + 1] = (int8_t)(((int)(byte << 24)) >> 28);
      }
    }
  }
  // tail bytes
  for (int64_t i = n_words * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_bytes; i += stride) {
    const uint32_t byte = packed[i];
    out[2 * i] = (int8_t)(((int)(byte << 28)) >> 28);
    out[2 * i + 1] = (int8_t)(((int)(byte << 24)) >> 28);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
template <typename T, int MODE, bool GIVEN>
static int launch_grouped_t(const T* x, int64_t rows, int64_t K, int64_t ldx, int gs, const int32_t* row_index,
                            int index_div, int64_t src_rows, const float* given, uint8_t* packed, float* scale, int role,
                            cudaStream_t st, const void* aux = nullptr, float eps = 0.f) {
  if (rows == 0 || K == 0) return I4TC_OK;
  // Enough blocks to fill the GPU several times over; beyond that a block walks several segments
  // of its rows so that loads of the next segment overlap the arithmetic of the current one.
  const int64_t row_blocks = (rows + kQRows - 1) / kQRows;
  const int nseg = (int)((K + kQSeg - 1) / kQSeg);
  int spb = nseg;
  if (row_blocks < 2048) spb = (int)((int64_t)nseg * row_blocks / 2048);
  if (spb < 1) spb = 1;
  if (MODE == 3) spb = nseg;   // a warp normalises with the statistics of its whole row
  dim3 grid((unsigned)row_blocks, (unsigned)((nseg + spb - 1) / spb));
  I4TC_REQUIRE(grid.y <= 65535, I4TC_EINVAL, "K=%lld too large for the grouped quantiser", (long long)K);
#define I4TC_LAUNCH_G(LPG)                                                                             \
  quant_grouped_kernel<T, LPG, MODE, GIVEN><<<grid, 256, 0, st>>>(x, rows, (int)K, ldx, row_index,     \
                                                                   index_div, src_rows, given, packed, scale, role, spb, \
                                                                   static_cast<const T*>(aux), eps)
  switch (gs) {
    case 32: I4TC_LAUNCH_G(1); break;
    case 64: I4TC_LAUNCH_G(2); break;
    case 128: I4TC_LAUNCH_G(4); break;
    case 256: I4TC_LAUNCH_G(8); break;
    default: return fail(I4TC_EUNSUPPORTED, "group_size=%d not supported (32, 64, 128 or 256)", gs);
  }
#undef I4TC_LAUNCH_G
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

// Mapped-output launches (bf16 input, group size 128): MODE 1 = gather rows through row_index, MODE 2 = SwiGLU first.
template <int MODE>
static int launch_grouped_mapped(const __nv_bfloat16* x, int64_t rows, int64_t K, int64_t ldx, const int32_t* row_index,
                                 int index_div, int64_t src_rows, uint8_t* packed, float* scale, const QuantOutMap& out,
                                 cudaStream_t st) {
  if (rows == 0 || K == 0) return I4TC_OK;
  const int64_t row_blocks = (rows + kQRows - 1) / kQRows;
  const int nseg = (int)((K + kQSeg - 1) / kQSeg);
  int spb = nseg;
  if (row_blocks < 2048) spb = (int)((int64_t)nseg * row_blocks / 2048);
  if (spb < 1) spb = 1;
  dim3 grid((unsigned)row_blocks, (unsigned)((nseg + spb - 1) / spb));
  quant_grouped_kernel<__nv_bfloat16, 4, MODE, false, true><<<grid, 256, 0, st>>>(
      x, rows, (int)K, ldx, row_index, index_div, src_rows, nullptr, packed, scale, I4TC_ROLE_ACTIVATION, spb, nullptr, 0.f,
      out);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

static int check_vec_input(const void* x, int dtype, int64_t ldx, const char* who) {
  const size_t es = dtype == I4TC_FP32 ? 4 : 2;
  I4TC_REQUIRE(aligned_to(x, 16) && (ldx * es) % 16 == 0, I4TC_EALIGN,
               "%s: input base and row stride must be 16-byte aligned", who);
  return I4TC_OK;
}

template <int MODE, bool GIVEN>
static int launch_grouped(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, int64_t gs,
                          const int32_t* row_index, int index_div, const float* given, uint8_t* packed,
                          float* scale, int role, int device, void* stream, const void* aux = nullptr, float eps = 0.f,
                          int64_t src_rows = 0) {
  I4TC_REQUIRE(rows >= 0 && K >= 0 && gs > 0, I4TC_EINVAL, "negative size");
  I4TC_REQUIRE(gs % 2 == 0, I4TC_EINVAL, "group_size must be even");
  I4TC_REQUIRE(K % gs == 0, I4TC_EINVAL, "K must be divisible by group_size");
  I4TC_REQUIRE(K < (1ll << 31), I4TC_EINVAL, "K too large");
  I4TC_REQUIRE(role == I4TC_ROLE_ACTIVATION || role == I4TC_ROLE_WEIGHT, I4TC_EINVAL, "bad role");
  if (rows == 0 || K == 0) return I4TC_OK;
  I4TC_REQUIRE(x && packed && (GIVEN ? given != nullptr : scale != nullptr), I4TC_EINVAL, "null pointer");
  if (int rc = check_vec_input(x, dtype, ldx, "quant_grouped")) return rc;
  I4TC_REQUIRE(aligned_to(packed, 16), I4TC_EALIGN, "packed output must be 16-byte aligned");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case I4TC_BF16:
      return launch_grouped_t<__nv_bfloat16, MODE, GIVEN>(static_cast<const __nv_bfloat16*>(x), rows, K, ldx,
                                                          (int)gs, row_index, index_div, src_rows, given, packed, scale,
                                                          role, st, aux, eps);
    case I4TC_FP16:
      if (MODE >= 2) break;
      return launch_grouped_t<__half, MODE >= 2 ? 0 : MODE, GIVEN>(static_cast<const __half*>(x), rows, K, ldx,
                                                                  (int)gs, row_index, index_div, src_rows, given, packed,
                                                                  scale, role, st);
    case I4TC_FP32:
      if (MODE >= 2) break;
      return launch_grouped_t<float, MODE >= 2 ? 0 : MODE, GIVEN>(static_cast<const float*>(x), rows, K, ldx,
                                                                 (int)gs, row_index, index_div, src_rows, given, packed,
                                                                 scale, role, st);
    default: break;
  }
  return fail(I4TC_EUNSUPPORTED, "unsupported input dtype %d", dtype);
}

template <typename T, bool GIVEN>
static int launch_rowwise_t(const T* x, int64_t rows, int64_t K, int64_t ldx, const float* given, uint8_t* packed,
                            float* scale, int role, cudaStream_t st) {
  const bool vec_ok = (K % 8 == 0) && K <= 16384 && aligned_to(x, 16) && (ldx * sizeof(T)) % 16 == 0 &&
                      aligned_to(packed, 4) && (K / 2) % 4 == 0;
  const unsigned grid = (unsigned)rows;
  if (!vec_ok) {
    quant_rowwise_generic_kernel<T, GIVEN><<<grid, 256, 0, st>>>(x, K, ldx, given, packed, scale, role);
  } else if (K <= 2048) {
    quant_rowwise_kernel<T, 1, GIVEN><<<grid, 256, 0, st>>>(x, (int)K, ldx, given, packed, scale, role);
  } else if (K <= 4096) {
    quant_rowwise_kernel<T, 2, GIVEN><<<grid, 256, 0, st>>>(x, (int)K, ldx, given, packed, scale, role);
  } else if (K <= 8192) {
    quant_rowwise_kernel<T, 4, GIVEN><<<grid, 256, 0, st>>>(x, (int)K, ldx, given, packed, scale, role);
  } else {
    quant_rowwise_kernel<T, 8, GIVEN><<<grid, 256, 0, st>>>(x, (int)K, ldx, given, packed, scale, role);
  }
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

template <bool GIVEN>
static int launch_rowwise(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, const float* given,
                          uint8_t* packed, float* scale, int role, int device, void* stream) {
  I4TC_REQUIRE(rows >= 0 && K >= 0, I4TC_EINVAL, "negative size");
  I4TC_REQUIRE(K % 2 == 0, I4TC_EINVAL, "K must be even for INT4 packing");
  I4TC_REQUIRE(rows < (1ll << 31), I4TC_EINVAL, "too many rows");
  I4TC_REQUIRE(role == I4TC_ROLE_ACTIVATION || role == I4TC_ROLE_WEIGHT, I4TC_EINVAL, "bad role");
  if (rows == 0) return I4TC_OK;
  I4TC_REQUIRE(x || K == 0, I4TC_EINVAL, "null input");
  I4TC_REQUIRE((packed || K == 0) && (GIVEN ? given != nullptr : scale != nullptr), I4TC_EINVAL, "null pointer");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case I4TC_BF16:
      return launch_rowwise_t<__nv_bfloat16, GIVEN>(static_cast<const __nv_bfloat16*>(x), rows, K, ldx, given,
                                                    packed, scale, role, st);
    case I4TC_FP16:
      return launch_rowwise_t<__half, GIVEN>(static_cast<const __half*>(x), rows, K, ldx, given, packed, scale,
                                             role, st);
    case I4TC_FP32:
      return launch_rowwise_t<float, GIVEN>(static_cast<const float*>(x), rows, K, ldx, given, packed, scale,
                                            role, st);
    default: break;
  }
  return fail(I4TC_EUNSUPPORTED, "unsupported input dtype %d", dtype);
}

}  // namespace i4tc

using namespace i4tc;

extern "C" int i4tc_quant_rowwise(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, uint8_t* packed,
                                  float* scale, int role, int device, void* stream) {
  return launch_rowwise<false>(x, dtype, rows, K, ldx, nullptr, packed, scale, role, device, stream);
}

extern "C" int i4tc_quant_grouped(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                                  int64_t group_size, uint8_t* packed, float* scale, int role, int device,
                                  void* stream) {
  return launch_grouped<0, false>(x, dtype, rows, K, ldx, group_size, nullptr, 1, nullptr, packed, scale, role,
                                  device, stream);
}

extern "C" int i4tc_quant_with_scales(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                                      int64_t group_size, const float* scale, uint8_t* packed, int device,
                                      void* stream) {
  if (group_size == 0)
    return launch_rowwise<true>(x, dtype, rows, K, ldx, scale, packed, nullptr, I4TC_ROLE_ACTIVATION, device,
                                stream);
  return launch_grouped<0, true>(x, dtype, rows, K, ldx, group_size, nullptr, 1, scale, packed, nullptr,
                                 I4TC_ROLE_ACTIVATION, device, stream);
}

extern "C" int i4tc_moe_gather_quant(const void* x, int dtype, int64_t num_tokens, int64_t K, int64_t ldx,
                                     const int32_t* sorted_pairs, int64_t num_pairs, int64_t top_k, uint8_t* packed,
                                     float* scale, int device, void* stream) {
  I4TC_REQUIRE(top_k > 0 && top_k < (1 << 20), I4TC_EINVAL, "bad top_k");
  I4TC_REQUIRE(num_tokens >= 0, I4TC_EINVAL, "negative num_tokens");
  I4TC_REQUIRE(sorted_pairs || num_pairs == 0, I4TC_EINVAL, "null sorted_pairs");
  return launch_grouped<1, false>(x, dtype, num_pairs, K, ldx, 128, sorted_pairs, (int)top_k, nullptr, packed,
                                  scale, I4TC_ROLE_ACTIVATION, device, stream, nullptr, 0.f, num_tokens);
}

extern "C" int i4tc_moe_ep_dispatch_quant(const void* x, int64_t num_tokens, int64_t K, int64_t ldx,
                                          const int32_t* sorted_pairs, int64_t num_pairs, int64_t top_k,
                                          const int32_t* slot, void* send_buf, int64_t row_bytes,
                                          const uint64_t* peer_bases, int64_t cap, int64_t my_rank, int device,
                                          void* stream) {
  I4TC_REQUIRE(top_k > 0 && top_k < (1 << 20) && num_tokens >= 0 && num_pairs >= 0, I4TC_EINVAL, "bad sizes");
  I4TC_REQUIRE(K > 0 && K % 128 == 0 && row_bytes == (K / 128) * 68, I4TC_EINVAL,
               "a row is 64 bytes of codes and one fp32 scale per 128 values");
  if (num_pairs == 0) return I4TC_OK;
  I4TC_REQUIRE(x && sorted_pairs && slot && (send_buf || peer_bases), I4TC_EINVAL, "null pointer");
  if (int rc = check_vec_input(x, I4TC_BF16, ldx, "moe_ep_dispatch_quant")) return rc;
  I4TC_REQUIRE(aligned_to(send_buf, 16), I4TC_EALIGN, "send buffer must be 16-byte aligned");
  I4TC_REQUIRE(peer_bases == nullptr || (cap > 0 && my_rank >= 0), I4TC_EINVAL, "peer destinations need cap and the rank");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  const int64_t G = K / 128;
  QuantOutMap out;
  out.row_map = slot;
  out.rows_dev = nullptr;
  out.pk_gstride = 64;
  out.pk_rstride = row_bytes;
  out.sc_gstride = 1;
  out.sc_rstride = row_bytes / 4;
  out.dest_bases = reinterpret_cast<const unsigned long long*>(peer_bases);
  out.block_rows = (int)(1 + cap);
  out.my_block = (int)my_rank;
  out.scale_offset = G * 64;
  uint8_t* base = static_cast<uint8_t*>(send_buf);
  return launch_grouped_mapped<1>(static_cast<const __nv_bfloat16*>(x), num_pairs, K, ldx, sorted_pairs, (int)top_k,
                                  num_tokens, base, reinterpret_cast<float*>(base + G * 64), out,
                                  static_cast<cudaStream_t>(stream));
}

extern "C" int i4tc_moe_silu_mul_quant_rows(const void* h, int64_t max_rows, const int32_t* rows_dev, int64_t I,
                                            uint8_t* packed, float* scale, int device, void* stream) {
  I4TC_REQUIRE(max_rows >= 0 && I > 0 && I % 128 == 0, I4TC_EINVAL, "intermediate size must be a positive multiple of 128");
  if (max_rows == 0) return I4TC_OK;
  I4TC_REQUIRE(h && rows_dev && packed && scale, I4TC_EINVAL, "null pointer");
  if (int rc = check_vec_input(h, I4TC_BF16, 2 * I, "moe_silu_mul_quant_rows")) return rc;
  I4TC_REQUIRE(aligned_to(packed, 16), I4TC_EALIGN, "packed output must be 16-byte aligned");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  QuantOutMap out;
  out.row_map = nullptr;
  out.rows_dev = rows_dev;
  out.pk_gstride = max_rows * 64;
  out.pk_rstride = 64;
  out.sc_gstride = max_rows;
  out.sc_rstride = 1;
  out.dest_bases = nullptr;
  out.block_rows = 1;
  out.my_block = 0;
  out.scale_offset = 0;
  return launch_grouped_mapped<2>(static_cast<const __nv_bfloat16*>(h), max_rows, I, 2 * I, nullptr, 1, 0, packed, scale,
                                  out, static_cast<cudaStream_t>(stream));
}

extern "C" int i4tc_moe_silu_mul_quant(const void* h, int64_t P, int64_t I, uint8_t* packed, float* scale,
                                       int device, void* stream) {
  return launch_grouped<2, false>(h, I4TC_BF16, P, I, 2 * I, 128, nullptr, 1, nullptr, packed, scale,
                                  I4TC_ROLE_ACTIVATION, device, stream);
}

extern "C" int i4tc_rmsnorm_quant_grouped(const void* x, int64_t rows, int64_t K, int64_t ldx, const void* norm_weight,
                                          float eps, int64_t group_size, uint8_t* packed, float* scale, int device,
                                          void* stream) {
  I4TC_REQUIRE(norm_weight != nullptr || rows == 0, I4TC_EINVAL, "null norm_weight");
  I4TC_REQUIRE(K % 32 == 0, I4TC_EINVAL, "K must be a multiple of 32");
  I4TC_REQUIRE(aligned_to(norm_weight, 16), I4TC_EALIGN, "norm_weight must be 16-byte aligned");
  I4TC_REQUIRE(eps >= 0.f, I4TC_EINVAL, "negative eps");
  return launch_grouped<3, false>(x, I4TC_BF16, rows, K, ldx, group_size, nullptr, 1, nullptr, packed, scale,
                                  I4TC_ROLE_ACTIVATION, device, stream, norm_weight, eps);
}

extern "C" int i4tc_unpack_int4_to_int8(const uint8_t* packed, int64_t rows, int64_t K, int8_t* out, int device,
                                        void* stream) {
  I4TC_REQUIRE(rows >= 0 && K >= 0 && K % 2 == 0, I4TC_EINVAL, "rows >= 0 and even K required");
  const int64_t n_bytes = rows * (K / 2);
  if (n_bytes == 0) return I4TC_OK;
  I4TC_REQUIRE(packed && out, I4TC_EINVAL, "null pointer");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  int64_t blocks = (n_bytes / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  const int64_t cap = (int64_t)info->sm_count * 16;
  if (blocks > cap) blocks = cap;
  unpack_int4_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(packed, n_bytes, out);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}
