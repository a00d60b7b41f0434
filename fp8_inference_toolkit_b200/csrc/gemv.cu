// W4A4 linear for a handful of tokens (M <= 8): weight streaming on the CUDA cores.
//
// With so few tokens the tensor-core kernel is a chain of per-group handshakes and reaches a small
// fraction of HBM bandwidth.  Here every lane owns one weight row and streams it 64 bytes (one K group
// of 128 codes) at a time with four 16-byte loads; the tokens' codes sit in shared memory, already
// expanded to int8, and are read with broadcast loads.  The arithmetic is the same as in the tensor
// kernel: a nibble moved to the top of its byte is 16 x the code, dp4a sums products of such bytes, so
// every int32 group sum is exactly 256 x the true one and the factor leaves as 2^-8 on a scale.
//
// A thread block covers 32 weight rows; its warps split the K groups into contiguous ranges and their
// partial results are added in ascending range order through shared memory (int32 for per-channel
// scales: exact; fp32 for per-group scales: a fixed order, so the result is deterministic).
#include "gemm.cuh"
#include "ptx.cuh"

namespace i4tc {

namespace {

constexpr int kRows = 32;   // weight rows per thread block (one per lane)

__device__ __forceinline__ void expand8(const uint4& w, uint32_t (&lo)[4], uint32_t (&hi)[4]) {
  lo[0] = (w.x << 4) & 0xF0F0F0F0u; hi[0] = w.x & 0xF0F0F0F0u;
  lo[1] = (w.y << 4) & 0xF0F0F0F0u; hi[1] = w.y & 0xF0F0F0F0u;
  lo[2] = (w.z << 4) & 0xF0F0F0F0u; hi[2] = w.z & 0xF0F0F0F0u;
  lo[3] = (w.w << 4) & 0xF0F0F0F0u; hi[3] = w.w & 0xF0F0F0F0u;
}

struct GemvParams {
  const uint8_t* x;   // activations, packed
  const uint8_t* w;   // weights, packed
  const float* sx;    // per-group: [G, M]; per-channel: [M]
  const float* sw;    // per-group: [G, N]; per-channel: [N]
  void* out;          // [M, N]
  int M, N, G;
  long long x_row, x_grp;   // byte strides of the activations: token, K group
  long long w_row, w_grp;   // byte strides of the weights: row, K group
  int out_fp16;
};

// MT: tokens handled (M <= MT).  PER_GROUP: fp32 scaling after every K group, else one int32 sum per row.
template <int MT, bool PER_GROUP>
__global__ void __launch_bounds__(512) w4a4_gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  // layout: expanded activations [G][MT][128] | group scales of the tokens [G][MT] | partials [warps][MT][32]
  uint8_t* act = smem;
  float* sx_s = reinterpret_cast<float*>(smem + (size_t)p.G * MT * 128);
  float* part = sx_s + (PER_GROUP ? p.G * MT : 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int n = blockIdx.x * kRows + lane;
  const bool n_ok = n < p.N;
  // this warp's K groups
  const int gper = (p.G + nwarps - 1) / nwarps;
  const int g0 = min(p.G, warp * gper), g1 = min(p.G, g0 + gper);

  // the first weight group is requested before the activations are staged
  const uint8_t* wrow = p.w + (long long)(n_ok ? n : 0) * p.w_row;
  uint4 wv[4];
  if (g0 < g1) {
    const uint4* src = reinterpret_cast<const uint4*>(wrow + (long long)g0 * p.w_grp);
#pragma unroll
    for (int j = 0; j < 4; ++j) wv[j] = __ldg(src + j);
  }

  // ---- stage the tokens: packed 16-byte chunk -> 16 bytes of even codes, 16 bytes of odd codes ----
  for (int i = threadIdx.x; i < p.G * MT * 4; i += blockDim.x) {
    const int j = i & 3, m = (i >> 2) % MT, g = (i >> 2) / MT;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m < p.M) v = __ldg(reinterpret_cast<const uint4*>(p.x + (long long)m * p.x_row + (long long)g * p.x_grp) + j);
    uint32_t lo[4], hi[4];
    expand8(v, lo, hi);
    uint4* dst = reinterpret_cast<uint4*>(act + ((size_t)(g * MT + m) * 128 + j * 32));
    dst[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    dst[1] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  }
  if (PER_GROUP) {
    for (int i = threadIdx.x; i < p.G * MT; i += blockDim.x) {
      const int m = i % MT, g = i / MT;
      sx_s[i] = (m < p.M) ? __ldg(p.sx + (long long)g * p.M + m) * (1.0f / 256.0f) : 0.f;
    }
  }
  __syncthreads();

  float f[MT];
  int acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) { f[m] = 0.f; acc[m] = 0; }

  for (int g = g0; g < g1; ++g) {
    uint4 cur[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) cur[j] = wv[j];
    if (g + 1 < g1) {
      const uint4* src = reinterpret_cast<const uint4*>(wrow + (long long)(g + 1) * p.w_grp);
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = __ldg(src + j);
    }
    float swv = 0.f;
    if (PER_GROUP) {
      swv = n_ok ? __ldg(p.sw + (long long)g * p.N + n) : 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[m] = 0;
    }
    const uint8_t* ag = act + (size_t)g * MT * 128;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t lo[4], hi[4];
      expand8(cur[j], lo, hi);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4 al = *reinterpret_cast<const uint4*>(ag + m * 128 + j * 32);
        const uint4 ah = *reinterpret_cast<const uint4*>(ag + m * 128 + j * 32 + 16);
        int s = acc[m];
        s = __dp4a((int)lo[0], (int)al.x, s); s = __dp4a((int)lo[1], (int)al.y, s);
        s = __dp4a((int)lo[2], (int)al.z, s); s = __dp4a((int)lo[3], (int)al.w, s);
        s = __dp4a((int)hi[0], (int)ah.x, s); s = __dp4a((int)hi[1], (int)ah.y, s);
        s = __dp4a((int)hi[2], (int)ah.z, s); s = __dp4a((int)hi[3], (int)ah.w, s);
        acc[m] = s;
      }
    }
    if (PER_GROUP) {
      // reference order: (acc * scale_x[g, m]) * scale_w[g, n]; 2^-8 rides on the token scale (exact)
#pragma unroll
      for (int m = 0; m < MT; ++m) f[m] = fmaf(__int2float_rn(acc[m]) * sx_s[g * MT + m], swv, f[m]);
    }
  }

  // ---- add the warps' ranges in ascending order ----
  if (nwarps > 1) {
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (PER_GROUP) part[(warp * MT + m) * kRows + lane] = f[m];
      else reinterpret_cast<int*>(part)[(warp * MT + m) * kRows + lane] = acc[m];
    }
    __syncthreads();
  }
  // warp w finishes tokens w, w + nwarps, ...
  for (int m = warp; m < p.M; m += nwarps) {
    float v;
    if (PER_GROUP) {
      if (nwarps > 1) {
        v = part[m * kRows + lane];
        for (int w2 = 1; w2 < nwarps; ++w2) v += part[(w2 * MT + m) * kRows + lane];
      } else {
        v = 0.f;
#pragma unroll
        for (int mm = 0; mm < MT; ++mm) if (mm == m) v = f[mm];
      }
    } else {
      int s;
      if (nwarps > 1) {
        s = reinterpret_cast<int*>(part)[m * kRows + lane];
        for (int w2 = 1; w2 < nwarps; ++w2) s += reinterpret_cast<int*>(part)[(w2 * MT + m) * kRows + lane];
      } else {
        s = 0;
#pragma unroll
        for (int mm = 0; mm < MT; ++mm) if (mm == m) s = acc[mm];
      }
      // reference order: (acc * scale_b[n]) * scale_a[m]
      const float sb = n_ok ? __ldg(p.sw + n) : 0.f;
      v = (__int2float_rn(s) * (sb * (1.0f / 256.0f))) * __ldg(p.sx + m);
    }
    if (n_ok) {
      if (p.out_fp16) static_cast<__half*>(p.out)[(long long)m * p.N + n] = __float2half_rn(v);
      else static_cast<__nv_bfloat16*>(p.out)[(long long)m * p.N + n] = __float2bfloat16_rn(v);
    }
  }
}

template <int MT, bool PER_GROUP>
int launch_mt(const GemvParams& p, int warps, size_t smem, cudaStream_t st) {
  static bool configured[64] = {false};
  int dev = 0;
  I4TC_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    I4TC_CUDA(cudaFuncSetAttribute(w4a4_gemv_kernel<MT, PER_GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured[dev] = true;
  }
  const int grid = (p.N + kRows - 1) / kRows;
  w4a4_gemv_kernel<MT, PER_GROUP><<<grid, warps * 32, smem, st>>>(p);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

}  // namespace

bool gemv_applicable(long long M, long long N, long long K, int epi_mode) {
  // at 16 tokens the broadcast shared-memory loads of the tokens' codes bound this kernel and the
  // tensor-core kernel is faster again (measured), so the hand-over is at 8
  if (M < 1 || M > 8 || N < 1 || K % 128 != 0) return false;
  if (epi_mode != EPI_GROUP && epi_mode != EPI_CHANNEL) return false;
  const int mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  const size_t need = (size_t)(K / 128) * mt * (128 + 4) + 16 * mt * kRows * 4;
  return need <= 200 * 1024;
}

int launch_w4a4_gemv(const uint8_t* x, const uint8_t* w, const float* sx, const float* sw, void* out, int out_dtype,
                     long long M, long long N, int G, bool rowmajor, int epi_mode, int sm_count, cudaStream_t st) {
  GemvParams p;
  p.x = x; p.w = w; p.sx = sx; p.sw = sw; p.out = out;
  p.M = (int)M; p.N = (int)N; p.G = G;
  if (rowmajor) {
    p.x_row = p.w_row = (long long)G * 64; p.x_grp = p.w_grp = 64;
  } else {
    p.x_row = p.w_row = 64; p.x_grp = M * 64; p.w_grp = N * 64;
  }
  p.out_fp16 = out_dtype == I4TC_FP16;
  I4TC_REQUIRE(aligned_to(x, 16) && aligned_to(w, 16), I4TC_EALIGN, "packed operands must be 16-byte aligned");
  const int mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  // enough warps to keep the memory system busy: aim for >= 16 warps per SM over the whole grid
  const long long blocks = (N + kRows - 1) / kRows;
  int warps = (int)((16ll * sm_count + blocks - 1) / blocks);
  warps = warps < 2 ? 2 : warps > 16 ? 16 : warps;
  if (warps > G) warps = G;
  const bool pg = epi_mode == EPI_GROUP;
  const size_t smem = (size_t)G * mt * 128 + (pg ? (size_t)G * mt * 4 : 0) + (size_t)warps * mt * kRows * 4;
#define I4TC_GEMV_CASE(MT_)                                                        \
  case MT_:                                                                        \
    return pg ? launch_mt<MT_, true>(p, warps, smem, st) : launch_mt<MT_, false>(p, warps, smem, st);
  switch (mt) {
    I4TC_GEMV_CASE(1)
    I4TC_GEMV_CASE(2)
    I4TC_GEMV_CASE(4)
    I4TC_GEMV_CASE(8)
    I4TC_GEMV_CASE(16)
  }
#undef I4TC_GEMV_CASE
  return fail(I4TC_EINVAL, "unsupported token count");
}

}  // namespace i4tc
