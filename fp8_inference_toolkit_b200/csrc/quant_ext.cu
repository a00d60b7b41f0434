// Clipped, asymmetric and smoothed per-group activation quantisers, the per-group sums of weight codes, and
// the zero-point pass that finishes a per-group linear whose activations were quantised asymmetrically.
//
// Quantisers: one warp owns one (row, K-group) slice; a lane keeps its gs/32 consecutive elements in
// registers between the reductions (warp shuffles) and the quantise step, so the input is read once; a warp
// writes gs/2 contiguous bytes.  The reference launches one 256-thread block per slice and reads it two or
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

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// clamp(rint(v / s + off), lo, hi).  Fast path: one FMA with r ~ 1/s (rcp.approx, within 2^-23); for
// |y| < 64 it lies within 3e-5 of the two-rounding IEEE value, so unless y is within 1e-4 of a rounding
// boundary both round to the same integer.  Everything else takes the IEEE division.
__device__ __forceinline__ float code_of(float v, float s, float r, bool fast, float off, float lo, float hi) {
  float y = fmaf(v, r, off);
  float q = rintf(y);
  if (!fast || !(fabsf(y - q) < 0.4999f) || !(fabsf(y) < 64.0f)) q = rintf(__fadd_rn(__fdiv_rn(v, s), off));
  return fminf(fmaxf(q, lo), hi);
}

template <typename T, int EPL, bool ASYM>
__global__ void __launch_bounds__(256) quant_ext_kernel(const T* __restrict__ x, long long rows, int G, long long ldx,
                                                        float clip, const T* __restrict__ smooth, bool vec_x,
                                                        bool vec_s, uint8_t* __restrict__ packed,
                                                        float* __restrict__ scale, float* __restrict__ azp_adj) {
  constexpr int GS = EPL * 32;
  const int lane = threadIdx.x & 31;
  const long long items = rows * G;
  for (long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); w < items; w += (long long)gridDim.x * 8) {
    const long long row = w / G;
    const int g = (int)(w - row * G);
    float v[EPL];
    load_elems<T, EPL>(x + row * ldx + (long long)g * GS + lane * EPL, vec_x, v);
    if (smooth != nullptr) {
      float sm[EPL];
      load_elems<T, EPL>(smooth + (long long)g * GS + lane * EPL, vec_s, sm);
#pragma unroll
      for (int i = 0; i < EPL; ++i) v[i] = __fdiv_rn(v[i], sm[i]);
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = warp_max(amax);
    const float thr = __fmul_rn(amax, clip);

    float s, off, lo, hi, out_scale;
    bool zero = false;
    if (ASYM) {
      float mn = INFINITY, mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        v[i] = fminf(fmaxf(v[i], -thr), thr);
        mn = fminf(mn, v[i]);
        mx = fmaxf(mx, v[i]);
      }
      mn = warp_min(mn);
      mx = warp_max(mx);
      s = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), 15.0f), ext_min_scale());
      off = fminf(fmaxf(rintf(__fdiv_rn(-mn, s)), 0.0f), 15.0f);
      lo = 0.0f; hi = 15.0f;
      out_scale = s;
    } else {
      s = __fdiv_rn(thr, 7.0f);
      zero = !(s > 0.0f);
      off = 0.0f; lo = -8.0f; hi = 7.0f;
      out_scale = fmaxf(s, ext_min_scale());
      if (zero) s = 1.0f;
    }
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(s));
    const bool fast = (r > 1e-30f) && (r < 1e30f);
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const float q = zero ? 0.0f : code_of(v[i], s, r, fast, off, lo, hi);
      const uint32_t nib = ASYM ? ((uint32_t)(int)q ^ 8u) : ((uint32_t)(int)q & 0xFu);   // u - 8 == u ^ 8 as a nibble
      word |= (nib & 0xFu) << (4 * i);
    }
    uint8_t* dst = packed + ((long long)g * rows + row) * (GS / 2) + lane * (EPL / 2);
    if constexpr (EPL == 2) *dst = (uint8_t)word;
    else if constexpr (EPL == 4) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)word;
    else *reinterpret_cast<uint32_t*>(dst) = word;
    if (lane == 0) {
      scale[(long long)g * rows + row] = out_scale;
      if (ASYM) azp_adj[(long long)g * rows + row] = 8.0f - off;
    }
  }
}

template <typename T, bool ASYM>
int launch_ext_t(const T* x, long long rows, long long K, long long ldx, int gs, float clip, const T* smooth,
                 uint8_t* packed, float* scale, float* azp_adj, int sm_count, cudaStream_t st) {
  const int G = (int)(K / gs);
  const long long items = rows * G;
  long long blocks = (items + 7) / 8;
  const long long cap = (long long)sm_count * 8;
  if (blocks > cap) blocks = cap;
  const int epl = gs / 32;
  const bool vec_x = aligned_to(x, 2 * epl) && (ldx % epl == 0);
  const bool vec_s = smooth == nullptr || aligned_to(smooth, 2 * epl);
  switch (epl) {
    case 2: quant_ext_kernel<T, 2, ASYM><<<(unsigned)blocks, 256, 0, st>>>(x, rows, G, ldx, clip, smooth, vec_x, vec_s, packed, scale, azp_adj); break;
    case 4: quant_ext_kernel<T, 4, ASYM><<<(unsigned)blocks, 256, 0, st>>>(x, rows, G, ldx, clip, smooth, vec_x, vec_s, packed, scale, azp_adj); break;
    default: quant_ext_kernel<T, 8, ASYM><<<(unsigned)blocks, 256, 0, st>>>(x, rows, G, ldx, clip, smooth, vec_x, vec_s, packed, scale, azp_adj); break;
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

// out[m, n] = bf16( sum_s ws[s][m, n] + sum_g (sa[g, m] * adj[g, m]) * (sb[g, n] * wcs[g, n]) ), g ascending.
// A thread owns a 4 x 4 block of outputs: the row factors are warp-uniform loads, the column factors and the
// partial sums 16-byte loads (VEC: N % 4 == 0 and 16-byte aligned pointers).
template <bool VEC>
__global__ void __launch_bounds__(256) azp_finish_kernel(const float* __restrict__ ws, long long stride, int splits,
                                                         const float* __restrict__ sa, const float* __restrict__ sb,
                                                         const float* __restrict__ adj, const float* __restrict__ wcs,
                                                         int G, long long M, long long N,
                                                         __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long n0 = ((long long)blockIdx.x * 32 + lane) * 4;
  const long long m0 = ((long long)blockIdx.y * 8 + warp) * 4;
  if (n0 >= N || m0 >= M) return;
  float corr[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) corr[i][j] = 0.0f;
  for (int g = 0; g < G; ++g) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long m = m0 + i;
      a[i] = (m < M) ? __ldg(sa + (long long)g * M + m) * __ldg(adj + (long long)g * M + m) : 0.0f;
    }
    if (VEC) {
      const float4 s4 = __ldg(reinterpret_cast<const float4*>(sb + (long long)g * N + n0));
      const float4 c4 = __ldg(reinterpret_cast<const float4*>(wcs + (long long)g * N + n0));
      b[0] = s4.x * c4.x; b[1] = s4.y * c4.y; b[2] = s4.z * c4.z; b[3] = s4.w * c4.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long n = n0 + j;
        b[j] = (n < N) ? __ldg(sb + (long long)g * N + n) * __ldg(wcs + (long long)g * N + n) : 0.0f;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) corr[i][j] = fmaf(a[i], b[j], corr[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long m = m0 + i;
    if (m >= M) break;
    const long long idx = m * N + n0;
    if (VEC) {
      float4 acc = *reinterpret_cast<const float4*>(ws + idx);
      for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(ws + (long long)s * stride + idx);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      union { __nv_bfloat16 h[4]; uint2 u; } pk;
      pk.h[0] = __float2bfloat16_rn(acc.x + corr[i][0]);
      pk.h[1] = __float2bfloat16_rn(acc.y + corr[i][1]);
      pk.h[2] = __float2bfloat16_rn(acc.z + corr[i][2]);
      pk.h[3] = __float2bfloat16_rn(acc.w + corr[i][3]);
      *reinterpret_cast<uint2*>(out + idx) = pk.u;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (n0 + j >= N) break;
        float acc = ws[idx + j];
        for (int s = 1; s < splits; ++s) acc += ws[(long long)s * stride + idx + j];
        out[idx + j] = __float2bfloat16_rn(acc + corr[i][j]);
      }
    }
  }
}

}  // namespace

int launch_azp_finish(const float* ws, long long stride, int splits, const float* sa, const float* sb,
                      const float* adj, const float* wcs, int G, long long M, long long N, void* out,
                      cudaStream_t st) {
  const bool vec = (N % 4 == 0) && (stride % 4 == 0) && aligned_to(ws, 16) && aligned_to(sb, 16) &&
                   aligned_to(wcs, 16) && aligned_to(out, 8);
  const dim3 grid((unsigned)((N + 127) / 128), (unsigned)((M + 31) / 32));
  I4TC_REQUIRE(grid.y <= 65535u, I4TC_EINVAL, "M too large for the zero-point pass");
  if (vec)
    azp_finish_kernel<true><<<grid, 256, 0, st>>>(ws, stride, splits, sa, sb, adj, wcs, G, M, N,
                                                  static_cast<__nv_bfloat16*>(out));
  else
    azp_finish_kernel<false><<<grid, 256, 0, st>>>(ws, stride, splits, sa, sb, adj, wcs, G, M, N,
                                                   static_cast<__nv_bfloat16*>(out));
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

}  // namespace i4tc

using namespace i4tc;

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
