// Clipped, asymmetric and smoothed per-group activation quantisers, the per-group sums of weight codes, and
// the zero-point pass that finishes a per-group linear whose activations were quantised asymmetrically.
//
// Quantisers: a warp works on four (row, K-group) slices at a time, all 32 lanes on each; a lane keeps its
// gs/32 consecutive elements of every slice in registers between the reductions (warp shuffles) and the quantise
// step, so the input is read once; per slice the warp writes gs/2 contiguous bytes.  The reference launches one 256-thread block per slice and reads it two or
// three times (int4_native_tc/csrc/int4_quant.cu:857-903, 1189-1259, 1324-1430).
//
// Code arithmetic (shared with the CPU oracle; IEEE fp32, round-half-even, no contraction):
//   v   = x                       (or x / smooth_scale[k] when given, IEEE division)
//   t   = max|v| * clip_ratio
//   symmetric clipped:  s = t / 7;  q = clamp(rint(v / s), -8, 7), 0 when t == 0;  scale = max(s, 1/(7*512))
//   asymmetric:         c = clamp(v, -t, t);  s = max((max c - min c) / 15, 1/(7*512));
//                       azp = clamp(rint(-min c / s), 0, 15);  u = clamp(rint(c / s + azp), 0, 15);
//                       stored nibble = u - 8;  azp_adj = 8 - azp
// The reference multiplies by reciprocals under fast-math; its torch restatements divide
// (int4_native_tc/test_enhanced_quantization.py:262-268), which is the reproducible form used here.
#include "gemm.cuh"

namespace i4tc {

namespace {

__device__ __forceinline__ float ext_min_scale() { return 1.0f / (7.0f * 512.0f); }

template <typename T>
__device__ __forceinline__ void widen2(uint32_t w, float& a, float& b);
template <>
__device__ __forceinline__ void widen2<__nv_bfloat16>(uint32_t w, float& a, float& b) {
  a = __uint_as_float(w << 16);
  b = __uint_as_float(w & 0xFFFF0000u);
}
template <>
__device__ __forceinline__ void widen2<__half>(uint32_t w, float& a, float& b) {
  const __half2 h = *reinterpret_cast<const __half2*>(&w);
  const float2 f = __half22float2(h);
  a = f.x;
  b = f.y;
}

// EPL consecutive 16-bit elements -> fp32.  `vec`: the address is a multiple of 2 * EPL bytes.
template <typename T, int EPL>
__device__ __forceinline__ void load_elems(const T* src, bool vec, float (&v)[EPL]) {
  if (vec) {
    uint32_t w[EPL / 2];
    if constexpr (EPL == 2) {
      w[0] = *reinterpret_cast<const uint32_t*>(src);
    } else if constexpr (EPL == 4) {
      const uint2 t = *reinterpret_cast<const uint2*>(src);
      w[0] = t.x; w[1] = t.y;
    } else {
      const uint4 t = *reinterpret_cast<const uint4*>(src);
      w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
    }
#pragma unroll
    for (int i = 0; i < EPL / 2; ++i) widen2<T>(w[i], v[2 * i], v[2 * i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i) v[i] = to_f32(src[i]);
  }
}

// clamp(rint(v / s + off), lo, hi) + 1.5 * 2^23: the code sits in the low mantissa bits (two's complement).
// Fast path (the caller guarantees |v / s + off| < 64): one FMA with r ~ 1/s (rcp.approx, within 2^-23) lies
// within 3e-5 of the two-rounding IEEE value, so unless it is within 1e-4 of a rounding boundary both round to
// the same integer; the rounding itself is an add and a subtract of 1.5 * 2^23 (round-half-even, no conversion
// instructions, which issue at a quarter of the FMA rate).  Everything else takes the IEEE division.
__device__ __forceinline__ uint32_t code_bits(float v, float s, float r, bool fast, float off, float lo, float hi) {
  constexpr float kMagic = 12582912.0f;
  const float y = fmaf(v, r, off);
  float q = __fadd_rn(__fadd_rn(y, kMagic), -kMagic);
  if (!fast || !(fabsf(__fsub_rn(y, q)) < 0.4999f)) q = rintf(__fadd_rn(__fdiv_rn(v, s), off));
  q = fminf(fmaxf(q, lo), hi);
  return __float_as_uint(__fadd_rn(q, kMagic));
}

constexpr int kSlicesPerWarp = 4;   // (row, group) slices a warp has in flight per iteration

template <typename T, int EPL, bool ASYM>
__global__ void __launch_bounds__(256) quant_ext_kernel(const T* __restrict__ x, unsigned rows, unsigned G, long long ldx,
                                                        float clip, const T* __restrict__ smooth, bool vec_x,
                                                        bool vec_s, uint8_t* __restrict__ packed,
                                                        float* __restrict__ scale, float* __restrict__ azp_adj) {
  constexpr int GS = EPL * 32;
  constexpr int U = kSlicesPerWarp;
  const int lane = threadIdx.x & 31;
  const unsigned items = rows * G;   // < 2^31, checked by the host
  for (unsigned w0 = (blockIdx.x * 8u + (threadIdx.x >> 5)) * U; w0 < items; w0 += gridDim.x * 8u * U) {
    float v[U][EPL];
    unsigned row[U], grp[U];
    // consecutive slices (same row, next group) are adjacent in memory; all loads are issued before anything
    // depends on them
    {
      unsigned r0 = w0 / G, g0 = w0 - r0 * G;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        row[u] = r0;
        grp[u] = g0;
        if (++g0 == G) { g0 = 0; ++r0; }
        if (w0 + u < items) {
          load_elems<T, EPL>(x + (long long)row[u] * ldx + (long long)grp[u] * GS + lane * EPL, vec_x, v[u]);
        } else {
#pragma unroll
          for (int i = 0; i < EPL; ++i) v[u][i] = 0.0f;
        }
      }
    }
    if (smooth != nullptr) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (w0 + u >= items) continue;
        float sm[EPL];
        load_elems<T, EPL>(smooth + (long long)grp[u] * GS + lane * EPL, vec_s, sm);
#pragma unroll
        for (int i = 0; i < EPL; ++i) v[u][i] = __fdiv_rn(v[u][i], sm[i]);
      }
    }
    // reductions of the U slices side by side (independent shuffle chains)
    float mn[U], mx[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      mn[u] = INFINITY; mx[u] = -INFINITY;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        mn[u] = fminf(mn[u], v[u][i]);
        mx[u] = fmaxf(mx[u], v[u][i]);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        mn[u] = fminf(mn[u], __shfl_xor_sync(0xffffffffu, mn[u], o));
        mx[u] = fmaxf(mx[u], __shfl_xor_sync(0xffffffffu, mx[u], o));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (w0 + u >= items) continue;   // warp-uniform
      // max|v| = max(-min, max); clamping to [-t, t] is monotone, so the clamped extremes are the clamped raw ones
      const float thr = __fmul_rn(fmaxf(-mn[u], mx[u]), clip);
      float s, off, out_scale;
      bool zero = false;
      if (ASYM) {
        const float cmn = fminf(fmaxf(mn[u], -thr), thr), cmx = fminf(fmaxf(mx[u], -thr), thr);
        s = fmaxf(__fdiv_rn(__fsub_rn(cmx, cmn), 15.0f), ext_min_scale());
        off = fminf(fmaxf(rintf(__fdiv_rn(-cmn, s)), 0.0f), 15.0f);
        out_scale = s;
      } else {
        s = __fdiv_rn(thr, 7.0f);
        zero = !(s > 0.0f);
        off = 0.0f;
        out_scale = fmaxf(s, ext_min_scale());
        if (zero) s = 1.0f;
      }
      const float lo = ASYM ? 0.0f : -8.0f, hi = ASYM ? 15.0f : 7.0f;
      float r;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(s));
      // fast path only while every |v / s + off| of the slice stays below 64 (the error bound of code_bits);
      // an unclipped symmetric slice may exceed the clip range by 1 / clip_ratio
      const float vmax = ASYM ? thr : fmaxf(-mn[u], mx[u]);
      const bool fast = (r > 1e-30f) && (r < 1e30f) && (vmax * r < 48.0f);
      const long long slot = (long long)grp[u] * rows + row[u];
      if (lane == 0) {
        scale[slot] = out_scale;
        if (ASYM) azp_adj[slot] = 8.0f - off;
      }
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const float c = ASYM ? fminf(fmaxf(v[u][i], -thr), thr) : v[u][i];
        const uint32_t bits = zero ? 0u : code_bits(c, s, r, fast, off, lo, hi);
        word |= ((ASYM ? bits ^ 8u : bits) & 0xFu) << (4 * i);   // u - 8 == u ^ 8 as a nibble
      }
      uint8_t* dst = packed + slot * (GS / 2) + lane * (EPL / 2);
      if constexpr (EPL == 2) *dst = (uint8_t)word;
      else if constexpr (EPL == 4) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)word;
      else *reinterpret_cast<uint32_t*>(dst) = word;
    }
  }
}

template <typename T, bool ASYM>
int launch_ext_t(const T* x, long long rows, long long K, long long ldx, int gs, float clip, const T* smooth,
                 uint8_t* packed, float* scale, float* azp_adj, int sm_count, cudaStream_t st) {
  const int G = (int)(K / gs);
  const long long items = rows * G;
  I4TC_REQUIRE(items < (1ll << 31) - (1ll << 20), I4TC_EINVAL, "rows * groups too large");
  long long blocks = (items + 8 * kSlicesPerWarp - 1) / (8 * kSlicesPerWarp);
  const long long cap = (long long)sm_count * 8;
  if (blocks > cap) blocks = cap;
  const int epl = gs / 32;
  const bool vec_x = aligned_to(x, 2 * epl) && (ldx % epl == 0);
  const bool vec_s = smooth == nullptr || aligned_to(smooth, 2 * epl);
  switch (epl) {
    case 2: quant_ext_kernel<T, 2, ASYM><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, (unsigned)rows, (unsigned)G, ldx, clip, smooth, vec_x, vec_s, packed, scale, azp_adj); break;
    case 4: quant_ext_kernel<T, 4, ASYM><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, (unsigned)rows, (unsigned)G, ldx, clip, smooth, vec_x, vec_s, packed, scale, azp_adj); break;
    default: quant_ext_kernel<T, 8, ASYM><<<(unsigned)blocks, 256, 0, st>>>((const T*)x, (unsigned)rows, (unsigned)G, ldx, clip, smooth, vec_x, vec_s, packed, scale, azp_adj); break;
  }
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

template <bool ASYM>
int launch_ext(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, int64_t group_size, double clip_ratio,
               const void* smooth, uint8_t* packed, float* scale, float* azp_adj, int device, void* stream) {
  I4TC_REQUIRE(rows >= 0 && K >= 0, I4TC_EINVAL, "negative size");
  I4TC_REQUIRE(group_size == 64 || group_size == 128 || group_size == 256, I4TC_EUNSUPPORTED,
               "group_size must be 64, 128 or 256");
  I4TC_REQUIRE(K % group_size == 0, I4TC_EINVAL, "K must be divisible by group_size");
  I4TC_REQUIRE(clip_ratio > 0.0 && clip_ratio <= 1.0, I4TC_EINVAL, "clip_ratio must be in (0, 1]");
  I4TC_REQUIRE(rows < (1ll << 31) && K < (1ll << 31), I4TC_EINVAL, "sizes too large");
  if (rows == 0 || K == 0) return I4TC_OK;
  I4TC_REQUIRE(x && packed && scale && (!ASYM || azp_adj), I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(ldx >= K, I4TC_EINVAL, "row stride smaller than K");
  I4TC_REQUIRE(aligned_to(packed, 4), I4TC_EALIGN, "packed must be 4-byte aligned");
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // without a smoothing vector the 128-bit kernel does the same arithmetic at a fraction of the instructions
  if (smooth == nullptr && K % 32 == 0 && (dtype == I4TC_BF16 || dtype == I4TC_FP16) &&
      grouped_ext_fast_ok(x, ldx, packed))
    return launch_grouped_ext(ASYM, x, dtype, rows, K, ldx, (int)group_size, (float)clip_ratio, packed, scale, azp_adj,
                              st);
  if (dtype == I4TC_BF16)
    return launch_ext_t<__nv_bfloat16, ASYM>(static_cast<const __nv_bfloat16*>(x), rows, K, ldx, (int)group_size,
                                             (float)clip_ratio, static_cast<const __nv_bfloat16*>(smooth), packed,
                                             scale, azp_adj, info->sm_count, st);
  if (dtype == I4TC_FP16)
    return launch_ext_t<__half, ASYM>(static_cast<const __half*>(x), rows, K, ldx, (int)group_size, (float)clip_ratio,
                                      static_cast<const __half*>(smooth), packed, scale, azp_adj, info->sm_count, st);
  return fail(I4TC_EUNSUPPORTED, "input must be bf16 or fp16 (dtype %d)", dtype);
}

}  // namespace

namespace {

// out[r] = sum of the signed 4-bit codes of packed row r (`words` 32-bit words per row).
__global__ void __launch_bounds__(256) weight_group_sums_kernel(const uint32_t* __restrict__ packed, long long n_rows,
                                                                int words, float* __restrict__ out) {
  const long long r = (long long)blockIdx.x * 256 + threadIdx.x;
  if (r >= n_rows) return;
  const uint32_t* src = packed + r * words;
  int sum = 0;
  for (int i = 0; i < words; ++i) {
    // offset-binary trick: every nibble n becomes n ^ 8 = n + 8 (as unsigned), so the signed sum is the unsigned
    // nibble sum minus 8 per nibble
    const uint32_t w = __ldg(src + i) ^ 0x88888888u;
    const uint32_t pairs = (w & 0x0F0F0F0Fu) + ((w >> 4) & 0x0F0F0F0Fu);   // four byte lanes, each <= 30
    sum += (int)((pairs * 0x01010101u) >> 24) - 64;
  }
  out[r] = (float)sum;
}

}  // namespace

// Per-token symmetric int8: scale = max(absmax / 127, 1 / (127 * 512)); q = clamp(rint(x / (absmax / 127)), -128, 127)
// with IEEE division (the reproducible form of the reference's x * (127 / absmax)).  One block per row; the second pass
// over the row hits L1 / L2.
template <typename T>
__global__ void __launch_bounds__(256) quant_int8_rowwise_kernel(const T* __restrict__ x, int K, int64_t ldx,
                                                                 int8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float s_max[8];
  const int64_t r = blockIdx.x;
  const T* src = x + r * ldx;
  int8_t* dst = q + r * (int64_t)K;
  float m = 0.f;
  const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0) &&
                   sizeof(T) == 2;
  if (vec) {
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + k);
      const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(to_f32(e[i])));
    }
  } else {
    for (int k = threadIdx.x; k < K; k += 256) m = fmaxf(m, fabsf(to_f32(src[k])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = m;
  __syncthreads();
  m = s_max[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, s_max[i]);
  const float s = __fdiv_rn(m, 127.0f);
  if (threadIdx.x == 0) scale[r] = fmaxf(s, 1.0f / (127.0f * 512.0f));
  auto code = [&](float v) -> int {
    if (m == 0.f) return 0;
    const float t = fminf(fmaxf(rintf(__fdiv_rn(v, s)), -128.0f), 127.0f);
    return (int)t;
  };
  if (vec) {
    for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + k);
      const T* e = reinterpret_cast<const T*>(&u);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo |= ((uint32_t)code(to_f32(e[i])) & 0xFFu) << (8 * i);
        hi |= ((uint32_t)code(to_f32(e[i + 4])) & 0xFFu) << (8 * i);
      }
      *reinterpret_cast<uint2*>(dst + k) = make_uint2(lo, hi);
    }
  } else {
    for (int k = threadIdx.x; k < K; k += 256) dst[k] = (int8_t)code(to_f32(src[k]));
  }
}

}  // namespace i4tc

using namespace i4tc;

extern "C" int i4tc_quant_rowwise_int8(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, int8_t* q,
                                       float* scale, int device, void* stream) {
  I4TC_REQUIRE(rows >= 0 && K >= 0 && K < (1ll << 31) && rows < (1ll << 31), I4TC_EINVAL, "bad sizes");
  if (rows == 0 || K == 0) return I4TC_OK;
  I4TC_REQUIRE(x && q && scale, I4TC_EINVAL, "null pointer");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case I4TC_BF16:
      quant_int8_rowwise_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), (int)K, ldx, q, scale);
      break;
    case I4TC_FP16:
      quant_int8_rowwise_kernel<__half><<<(unsigned)rows, 256, 0, st>>>(static_cast<const __half*>(x), (int)K, ldx, q, scale);
      break;
    case I4TC_FP32:
      quant_int8_rowwise_kernel<float><<<(unsigned)rows, 256, 0, st>>>(static_cast<const float*>(x), (int)K, ldx, q, scale);
      break;
    default: return fail(I4TC_EUNSUPPORTED, "unsupported input dtype %d", dtype);
  }
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_quant_clipped_grouped(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                                          int64_t group_size, double clip_ratio, uint8_t* packed, float* scale,
                                          int device, void* stream) {
  return launch_ext<false>(x, dtype, rows, K, ldx, group_size, clip_ratio, nullptr, packed, scale, nullptr, device,
                           stream);
}

extern "C" int i4tc_quant_asymmetric_grouped(const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx,
                                             int64_t group_size, double clip_ratio, const void* smooth_scale,
                                             uint8_t* packed, float* scale, float* azp_adj, int device,
                                             void* stream) {
  return launch_ext<true>(x, dtype, rows, K, ldx, group_size, clip_ratio, smooth_scale, packed, scale, azp_adj,
                          device, stream);
}

extern "C" int i4tc_weight_group_sums(const uint8_t* b_packed, int64_t rows, int64_t group_size, float* out,
                                      int device, void* stream) {
  I4TC_REQUIRE(rows >= 0, I4TC_EINVAL, "negative size");
  I4TC_REQUIRE(group_size > 0 && group_size % 8 == 0, I4TC_EINVAL, "group_size must be a positive multiple of 8");
  if (rows == 0) return I4TC_OK;
  I4TC_REQUIRE(b_packed && out, I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(aligned_to(b_packed, 4), I4TC_EALIGN, "packed weights must be 4-byte aligned");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  const long long blocks = (rows + 255) / 256;
  I4TC_REQUIRE(blocks < (1ll << 31), I4TC_EINVAL, "too many rows");
  weight_group_sums_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(b_packed), rows, (int)(group_size / 8), out);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}
