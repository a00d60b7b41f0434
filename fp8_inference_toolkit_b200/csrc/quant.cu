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

// Eight consecutive elements as floats, loaded with 128-bit loads.
template <typename T>
struct Vec8 {
  float v[8];
  __device__ __forceinline__ void load(const T* p);
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
  }
};

template <>
__device__ __forceinline__ void Vec8<__nv_bfloat16>::load(const __nv_bfloat16* p) {
  uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
  uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
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
__device__ __forceinline__ float absmax8(const Vec8<T>& x) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(x.v[i]));
  return m;
}

// Eight codes -> one 32-bit word, element 0 in the lowest nibble.  Exact-division path.
template <typename T>
__device__ __forceinline__ uint32_t pack8_div(const Vec8<T>& x, float s) {
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) w |= code4(x.v[i], s) << (4 * i);
  return w;
}

// Per-slice constants of the fast path: r = RN(1/s).  `fast` is false when r is not a normal
// number of moderate size, in which case every vector takes the exact-division path.
struct Recip {
  float r;
  bool fast;
};
__device__ __forceinline__ Recip make_recip(float s) {
  Recip q;
  q.r = __frcp_rn(s);
  q.fast = (q.r > 7.8886090522e-31f) && (q.r < 1.2676506002e30f);  // 2^-100 < r < 2^100
  return q;
}

// Same result as pack8_div, bit for bit, at about a fifth of the instructions.
//   y8 = x*r + 8 (one FMA)      u = y8 + 1.5*2^23 rounds y8 to the nearest-even integer n+8 in [0,15]
//   v  = u - 1.5*2^23 = n+8     the eight v's are combined with exact FMAs (16 bits per half)
// |y8 - 8 - RN(x/s)| < 1.5e-6 for |x/s| <= 8, so unless some y8 lies within 1e-5 of a rounding
// boundary (k + 0.5) the rounded integers are those of the exact division.  Vectors with such an
// element (a few in 10^5) are redone with the exact division.  CLAMP: the caller supplied the
// divisor, so x/s may leave [-8, 7].
template <typename T, bool CLAMP>
__device__ __forceinline__ uint32_t pack8(const Vec8<T>& x, float s, Recip q, bool zero) {
  if (zero) return 0u;
  if (!q.fast) return pack8_div(x, s);
  constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
  float v[8], worst = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float y8 = fmaf(x.v[i], q.r, 8.0f);
    if (CLAMP) y8 = fminf(fmaxf(y8, 0.0f), 15.0f);
    const float u = y8 + kMagic;
    v[i] = u - kMagic;
    worst = fmaxf(worst, fabsf(y8 - v[i]));
  }
  if (!(worst <= 0.5f - 1e-5f)) return pack8_div(x, s);
  const float lo = fmaf(v[3], 4096.f, fmaf(v[2], 256.f, fmaf(v[1], 16.f, v[0])));
  const float hi = fmaf(v[7], 4096.f, fmaf(v[6], 256.f, fmaf(v[5], 16.f, v[4])));
  const uint32_t wl = __float_as_uint(lo + kMagic) & 0xFFFFu;
  const uint32_t wh = __float_as_uint(hi + kMagic) << 16;
  return (wl | wh) ^ 0x88888888u;  // offset-binary nibbles (n+8) -> two's complement
}

// silu(g) * u rounded to bf16 and widened again: the value the next quantiser sees.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  float sig = __fdiv_rn(1.0f, 1.0f + expf(-g));
  return __bfloat162float(__float2bfloat16_rn((g * sig) * u));
}

// ------------------------------------------------------------------------------------------
// Grouped kernel.  Block = 8 warps = 8 consecutive rows; each warp owns a 1024-element segment
// of its row (4 x 128-bit loads per lane, all issued before the first use).  A group of
// 8*LPG elements lives in LPG adjacent lanes, so its absmax is log2(LPG) shuffles.
// MODE 0: rows of x.  MODE 1: rows gathered through row_index[r] / index_div.
// MODE 2: input is bf16 [rows, 2*K] laid out [gate | up]; the quantised value is
//         bf16(silu(gate) * up).
// GIVEN: divisors come from `given_scale` (group-major) instead of the absmax.
// ------------------------------------------------------------------------------------------
constexpr int kQRows = 8;
constexpr int kQSteps = 4;
constexpr int kQSeg = 32 * 8 * kQSteps;  // 1024 elements

template <typename T, int LPG, int MODE, bool GIVEN>
__global__ void __launch_bounds__(256) quant_grouped_kernel(
    const T* __restrict__ x, int64_t rows, int K, int64_t ldx, const int32_t* __restrict__ row_index,
    int index_div, const float* __restrict__ given_scale, uint8_t* __restrict__ packed,
    float* __restrict__ scale, int role) {
  constexpr int GS = LPG * 8;
  constexpr int GROUPS_PER_STEP = 32 / LPG;
  constexpr int GROUPS_PER_SEG = GROUPS_PER_STEP * kQSteps;
  __shared__ float s_scale[GROUPS_PER_SEG][kQRows];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t r0 = (int64_t)blockIdx.x * kQRows;
  const int64_t r = r0 + warp;
  const int k0 = blockIdx.y * kQSeg;
  const bool row_ok = r < rows;

  Vec8<T> v[kQSteps];
  const T* src = nullptr;
  if (row_ok) {
    int64_t sr = r;
    if (MODE == 1) sr = row_index[r] / index_div;
    src = x + sr * ldx;
  }
#pragma unroll
  for (int j = 0; j < kQSteps; ++j) {
    const int k = k0 + j * 256 + lane * 8;
    if (row_ok && k < K) {
      if (MODE == 2) {
        Vec8<T> g, u;
        g.load(src + k);
        u.load(src + K + k);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j].v[i] = silu_mul_bf16(g.v[i], u.v[i]);
      } else {
        v[j].load(src + k);
      }
    } else {
      v[j].zero();
    }
  }

  const int gl = lane / LPG;  // group inside a step
#pragma unroll
  for (int j = 0; j < kQSteps; ++j) {
    const int k = k0 + j * 256 + lane * 8;
    const bool ok = row_ok && k < K;
    const int g = k / GS;
    float divisor, absmax = 0.f;
    if (GIVEN) {
      divisor = ok ? __ldg(given_scale + (int64_t)g * rows + r) : 1.f;
    } else {
      absmax = absmax8(v[j]);
#pragma unroll
      for (int o = 1; o < LPG; o <<= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, o));
      divisor = __fdiv_rn(absmax, 7.0f);
      if ((lane % LPG) == 0) s_scale[j * GROUPS_PER_STEP + gl][warp] = scale_out(absmax, role);
    }
    if (ok) {
      const uint32_t w = pack8<T, GIVEN>(v[j], divisor, make_recip(divisor), !GIVEN && absmax == 0.f);
      uint8_t* dst = packed + ((int64_t)g * rows + r) * (GS / 2) + (lane % LPG) * 4;
      *reinterpret_cast<uint32_t*>(dst) = w;
    }
  }
  if (!GIVEN) {
    __syncthreads();
    // 8 consecutive rows of one group are 32 contiguous bytes of the [G, rows] scale array.
    for (int t = threadIdx.x; t < GROUPS_PER_SEG * kQRows; t += 256) {
      const int gi = t / kQRows, rr = t % kQRows;
      const int g = k0 / GS + gi;
      if (g * GS < K && r0 + rr < rows) scale[(int64_t)g * rows + r0 + rr] = s_scale[gi][rr];
    }
  }
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
    divisor = __fdiv_rn(absmax, 7.0f);
    if (t == 0) scale[r] = scale_out(absmax, role);
  }
  uint8_t* dst = packed + r * (int64_t)(K / 2);
  const Recip rcp = make_recip(divisor);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = c * 2048 + t * 8;
    if (k < K) *reinterpret_cast<uint32_t*>(dst + k / 2) = pack8<T, GIVEN>(v[c], divisor, rcp, !GIVEN && absmax == 0.f);
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
                            int index_div, const float* given, uint8_t* packed, float* scale, int role,
                            cudaStream_t st) {
  if (rows == 0 || K == 0) return I4TC_OK;
  dim3 grid((unsigned)((rows + kQRows - 1) / kQRows), (unsigned)((K + kQSeg - 1) / kQSeg));
  I4TC_REQUIRE(grid.y <= 65535, I4TC_EINVAL, "K=%lld too large for the grouped quantiser", (long long)K);
#define I4TC_LAUNCH_G(LPG)                                                                             \
  quant_grouped_kernel<T, LPG, MODE, GIVEN><<<grid, 256, 0, st>>>(x, rows, (int)K, ldx, row_index,     \
                                                                   index_div, given, packed, scale, role)
  switch (gs) {
    case 32: I4TC_LAUNCH_G(4); break;
    case 64: I4TC_LAUNCH_G(8); break;
    case 128: I4TC_LAUNCH_G(16); break;
    case 256: I4TC_LAUNCH_G(32); break;
    default: return fail(I4TC_EUNSUPPORTED, "group_size=%d not supported (32, 64, 128 or 256)", gs);
  }
#undef I4TC_LAUNCH_G
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
                          float* scale, int role, int device, void* stream) {
  I4TC_REQUIRE(rows >= 0 && K >= 0 && gs > 0, I4TC_EINVAL, "negative size");
  I4TC_REQUIRE(gs % 2 == 0, I4TC_EINVAL, "group_size must be even");
  I4TC_REQUIRE(K % gs == 0, I4TC_EINVAL, "K must be divisible by group_size");
  I4TC_REQUIRE(K < (1ll << 31), I4TC_EINVAL, "K too large");
  I4TC_REQUIRE(role == I4TC_ROLE_ACTIVATION || role == I4TC_ROLE_WEIGHT, I4TC_EINVAL, "bad role");
  if (rows == 0 || K == 0) return I4TC_OK;
  I4TC_REQUIRE(x && packed && (GIVEN ? given != nullptr : scale != nullptr), I4TC_EINVAL, "null pointer");
  if (int rc = check_vec_input(x, dtype, ldx, "quant_grouped")) return rc;
  I4TC_REQUIRE(aligned_to(packed, 4), I4TC_EALIGN, "packed output must be 4-byte aligned");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case I4TC_BF16:
      return launch_grouped_t<__nv_bfloat16, MODE, GIVEN>(static_cast<const __nv_bfloat16*>(x), rows, K, ldx,
                                                          (int)gs, row_index, index_div, given, packed, scale,
                                                          role, st);
    case I4TC_FP16:
      if (MODE == 2) break;
      return launch_grouped_t<__half, MODE == 2 ? 0 : MODE, GIVEN>(static_cast<const __half*>(x), rows, K, ldx,
                                                                  (int)gs, row_index, index_div, given, packed,
                                                                  scale, role, st);
    case I4TC_FP32:
      if (MODE == 2) break;
      return launch_grouped_t<float, MODE == 2 ? 0 : MODE, GIVEN>(static_cast<const float*>(x), rows, K, ldx,
                                                                 (int)gs, row_index, index_div, given, packed,
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

extern "C" int i4tc_moe_gather_quant(const void* x, int dtype, int64_t K, int64_t ldx, const int32_t* sorted_pairs,
                                     int64_t num_pairs, int64_t top_k, uint8_t* packed, float* scale, int device,
                                     void* stream) {
  I4TC_REQUIRE(top_k > 0 && top_k < (1 << 20), I4TC_EINVAL, "bad top_k");
  I4TC_REQUIRE(sorted_pairs || num_pairs == 0, I4TC_EINVAL, "null sorted_pairs");
  return launch_grouped<1, false>(x, dtype, num_pairs, K, ldx, 128, sorted_pairs, (int)top_k, nullptr, packed,
                                  scale, I4TC_ROLE_ACTIVATION, device, stream);
}

extern "C" int i4tc_moe_silu_mul_quant(const void* h, int64_t P, int64_t I, uint8_t* packed, float* scale,
                                       int device, void* stream) {
  return launch_grouped<2, false>(h, I4TC_BF16, P, I, 2 * I, 128, nullptr, 1, nullptr, packed, scale,
                                  I4TC_ROLE_ACTIVATION, device, stream);
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
