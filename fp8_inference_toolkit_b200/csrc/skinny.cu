// W4A4 linear for 3 to 32 tokens: weight streaming through register-fed tensor-core instructions.
//
// At these sizes the op moves half a byte per 2 M operations, far below the machine balance, so the only thing that
// counts is how many weight bytes are in flight.  The tile kernel (TMA -> converter warps -> tcgen05 -> TMEM drain) is a
// chain of per-group handshakes with a handful of stages per SM; here a thread block asks for ALL of its bytes
// at once (cp.async.bulk, one mbarrier per warp and K group -- per warp for row-major operands, where a row's K range is
// one copy: the weight rows and, where they fit, the tokens' codes and the scales), several blocks share an SM, and nothing waits on another role: a warp expands the nibbles of its
// K groups in registers, multiplies them with mma.sync.m16n8k32 (int8, int32 accumulators in registers) and applies
// the group's scales in registers.
//
// A block covers ROWS = 16 or 32 weight rows and the whole K; its 8 or 16 warps split the K groups into contiguous ranges
// and the ranges are added in ascending order through shared memory (int32 for per-channel scales: exact; fp32 for
// per-group scales: a fixed order, so the result is deterministic).  No workspace and no second launch.
//
// Nibble arithmetic as in the other kernels: a nibble moved to the top of its byte is 16 x the code, so every int32
// sum is exactly 256 x the true one and the factor leaves as 2^-8 on a scale.  The k order inside an MMA is
// free as long as both operands agree: fragment register j of a lane holds the even (a0/a1/b0) or odd (a2/a3/b1)
// codes of 32-bit word 4 t + j of the 64-byte group row, for weights and tokens alike.
#include "gemm.cuh"
#include "ptx.cuh"

namespace i4tc {

namespace {

using namespace ptx;

// Warps per block: 16 halve the serial chain of a warp; 32-row tiles take 8 so that the registers of two blocks fit an SM.
__host__ __device__ constexpr int skinny_warps(int mtiles) { return mtiles == 2 ? 8 : 16; }
constexpr int kMaxGroupsPerWarp = 16;
constexpr uint64_t kSkinnyWaitNs = 2000000000ull;   // 2 s

struct SkinnyParams {
  const uint8_t* x;   // activations, packed
  const uint8_t* w;   // weights, packed
  const float* sx;    // per-group: [G, M]; per-channel: [M]
  const float* sw;    // per-group: [G, N]; per-channel: [N]
  void* out;          // [M, N]
  int M, N, G;
  int gper;           // K groups per warp
  int warps;          // warps per block
  long long x_row, x_grp;   // byte strides of the activations: token, K group
  long long w_row, w_grp;   // byte strides of the weights: row, K group
  int rowmajor;
  int rstride;        // row-major operands: bytes between rows in shared memory (a warp's K range plus padding)
  int out_fp16;
  unsigned int* status;     // bit 0 is set when a bounded wait expires
};

__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :: "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ void expand4(const uint4& w, uint32_t (&lo)[4], uint32_t (&hi)[4]) {
  lo[0] = (w.x << 4) & 0xF0F0F0F0u; hi[0] = w.x & 0xF0F0F0F0u;
  lo[1] = (w.y << 4) & 0xF0F0F0F0u; hi[1] = w.y & 0xF0F0F0F0u;
  lo[2] = (w.z << 4) & 0xF0F0F0F0u; hi[2] = w.z & 0xF0F0F0F0u;
  lo[3] = (w.w << 4) & 0xF0F0F0F0u; hi[3] = w.w & 0xF0F0F0F0u;
}

// Bounded wait for phase 0 of a barrier; on expiry bit 0 of the status word is set and false returned.
__device__ __forceinline__ bool wait_landed(uint32_t bar, unsigned int* status) {
  if (mbar_test_wait(bar, 0)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, 0)) return true;
    if ((++spins & 63u) == 0 && globaltimer_ns() - t0 > kSkinnyWaitNs) {
      atomicOr(status, 1u);
      return false;
    }
  }
}

// Bytes of shared memory per warp and K group: the block's weight rows, then (STAGE) the tokens' codes and the rows'
// scales of that group.
__host__ __device__ constexpr int skinny_item(int rows, int tok, bool stage) {
  return rows * 64 + (stage ? tok * 64 + rows * 4 : 0);
}

// MTILES: 16-row tiles per block (ROWS = 16 MTILES).  NT: 8-token tiles (M <= 8 NT).
// STAGE: the tokens' codes and both scale vectors of a warp's K groups are brought into shared memory up front as
// well (bulk copies on the weights' barriers, plain loads for the token scales), so that the loop over the groups
// touches no global memory; otherwise they are fetched into registers one group ahead (shapes whose tokens would
// leave room for only one block per SM).
template <int MTILES, int NT, bool PER_GROUP, bool STAGE>
__global__ void __launch_bounds__(skinny_warps(MTILES) * 32) w4a4_skinny_kernel(const SkinnyParams p) {
  constexpr int ROWS = 16 * MTILES;
  constexpr int TOK = 8 * NT;
  constexpr int CHUNK = ROWS * 64;   // bytes of one K group of the block's rows
  constexpr int ITEM = skinny_item(ROWS, TOK, STAGE);
  extern __shared__ __align__(128) uint8_t smem[];
  // layout: items [warp][group of the warp][ITEM] | token scales [warp][group][TOK] (STAGE) | barriers; the start is
  // later reused for the warps' partial sums
  constexpr int nwarps = skinny_warps(MTILES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * ROWS;
  const int g0 = min(p.G, warp * p.gper), g1 = min(p.G, g0 + p.gper), gw = g1 - g0;
  // Group-major operands: one item per K group ([ROWS][64] codes, then the staged tokens and scales).  Row-major operands
  // ([rows, K/2]): a warp's K range of one row is contiguous, so each row arrives as one copy of gw * 64 bytes and rows
  // lie `rstride` bytes apart (= 64 mod 128, so that eight rows x four 16-byte chunks hit distinct banks).
  const bool rm = p.rowmajor != 0;
  const int rs = rm ? p.rstride : 64;                  // bytes between rows of one K group
  const int gstep = rm ? 64 : ITEM;                    // bytes between K groups
  const int tok_off = rm ? ROWS * p.rstride : CHUNK;   // where the staged tokens' codes start
  const size_t region = rm ? (size_t)(ROWS + (STAGE ? TOK : 0)) * p.rstride : (size_t)p.gper * ITEM;
  const size_t item_bytes = (size_t)nwarps * region;
  const size_t sx_bytes = (STAGE && PER_GROUP) ? (size_t)nwarps * p.gper * TOK * 4 : 0;
  const size_t red_bytes = (size_t)nwarps * TOK * ROWS * 4;
  const size_t data_bytes = item_bytes + sx_bytes > red_bytes ? item_bytes + sx_bytes : red_bytes;
  uint8_t* wsm = smem + (size_t)warp * region;
  float* sx_s = reinterpret_cast<float*>(smem + item_bytes) + (size_t)warp * p.gper * TOK;
  const uint32_t bars = smem_u32(smem + data_bytes) + (uint32_t)warp * kMaxGroupsPerWarp * 8u;

  // ---- ask for every byte of this warp's K range ----
  if (lane < gw) mbar_init(bars + lane * 8u, 1);
  fence_mbar_init();
  __syncwarp();
  if (!rm) {
    const uint32_t tx = CHUNK + (STAGE ? (uint32_t)p.M * 64u + (PER_GROUP ? ROWS * 4u : 0u) : 0u);
    if (lane < gw) {
      const uint32_t bar = bars + lane * 8u, dst = smem_u32(wsm) + lane * ITEM;
      const int grp = g0 + lane;
      mbar_arrive_expect_tx(bar, tx);
      // the block's rows (and all tokens) of one group are contiguous
      bulk_load(dst, p.w + (long long)grp * p.w_grp + (long long)n0 * 64, CHUNK, bar);
      if (STAGE) {
        bulk_load(dst + CHUNK, p.x + (long long)grp * p.x_grp, (uint32_t)p.M * 64u, bar);
        if (PER_GROUP) bulk_load(dst + CHUNK + TOK * 64, p.sw + (long long)grp * p.N + n0, ROWS * 4, bar);
      }
    }
  } else if (gw > 0) {
    // everything of this warp on its first barrier: one copy per weight row (and per staged token)
    if (lane == 0) mbar_arrive_expect_tx(bars, (uint32_t)(ROWS + (STAGE ? p.M : 0)) * (uint32_t)gw * 64u);
    __syncwarp();
    for (int r = lane; r < ROWS; r += 32)
      bulk_load(smem_u32(wsm) + r * rs, p.w + (long long)(n0 + r) * p.w_row + (long long)g0 * 64, (uint32_t)gw * 64u, bars);
    if (STAGE) {
      for (int m = lane; m < p.M; m += 32)
        bulk_load(smem_u32(wsm) + tok_off + m * rs, p.x + (long long)m * p.x_row + (long long)g0 * 64, (uint32_t)gw * 64u, bars);
    }
  }
  if (STAGE) {
    // padding tokens: zero codes; token scales with the 2^-8 folded in
    const int pad = TOK - p.M;
    if (!rm) {
      for (int i = lane; i < gw * pad * 4; i += 32) {
        const int gi = i / (pad * 4), r = i - gi * (pad * 4);
        *reinterpret_cast<uint4*>(wsm + (size_t)gi * ITEM + CHUNK + (size_t)p.M * 64 + (size_t)r * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
    } else {
      for (int i = lane; i < pad * gw * 4; i += 32) {
        const int r = i / (gw * 4), c = i - r * (gw * 4);
        *reinterpret_cast<uint4*>(wsm + tok_off + (size_t)(p.M + r) * rs + (size_t)c * 16) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (PER_GROUP) {
      for (int i = lane; i < gw * TOK; i += 32) {
        const int gi = i / TOK, m = i - gi * TOK;
        sx_s[i] = m < p.M ? __ldg(p.sx + (long long)(g0 + gi) * p.M + m) * (1.0f / 256.0f) : 0.f;
      }
    }
    __syncwarp();
  }

  // ---- without staging: token codes and scales of the first group (registers) ----
  uint4 xb[NT];
  float sxs[NT][2], sws[MTILES][2];
  auto fetch = [&](int grp) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int tok = 8 * nt + g;
      xb[nt] = make_uint4(0u, 0u, 0u, 0u);
      if (tok < p.M) xb[nt] = __ldg(reinterpret_cast<const uint4*>(p.x + (long long)tok * p.x_row + (long long)grp * p.x_grp) + t);
      if (PER_GROUP) {
        const int t0 = 8 * nt + 2 * t;
        sxs[nt][0] = t0 < p.M ? __ldg(p.sx + (long long)grp * p.M + t0) * (1.0f / 256.0f) : 0.f;
        sxs[nt][1] = t0 + 1 < p.M ? __ldg(p.sx + (long long)grp * p.M + t0 + 1) * (1.0f / 256.0f) : 0.f;
      }
    }
    if (PER_GROUP) {
#pragma unroll
      for (int mt = 0; mt < MTILES; ++mt) {
        sws[mt][0] = __ldg(p.sw + (long long)grp * p.N + n0 + 16 * mt + g);
        sws[mt][1] = __ldg(p.sw + (long long)grp * p.N + n0 + 16 * mt + g + 8);
      }
    }
  };
  if (!STAGE && gw > 0) fetch(g0);

  float f[MTILES][NT][4];
  int c[MTILES][NT][4];
#pragma unroll
  for (int mt = 0; mt < MTILES; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) { f[mt][nt][i] = 0.f; c[mt][nt][i] = 0; }

  bool alive = true;
  for (int gi = 0; gi < gw && alive; ++gi) {
    uint32_t blo[NT][4], bhi[NT][4];
    float sx_c[NT][2], sw_c[MTILES][2];
    if (!STAGE) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        expand4(xb[nt], blo[nt], bhi[nt]);
        sx_c[nt][0] = sxs[nt][0]; sx_c[nt][1] = sxs[nt][1];
      }
#pragma unroll
      for (int mt = 0; mt < MTILES; ++mt) { sw_c[mt][0] = sws[mt][0]; sw_c[mt][1] = sws[mt][1]; }
      if (gi + 1 < gw) fetch(g0 + gi + 1);
    }
    alive = wait_landed(bars + (rm ? 0 : gi) * 8u, p.status);
    alive = __all_sync(0xffffffffu, alive);
    if (!alive) break;
    const uint32_t item = smem_u32(wsm) + gi * gstep;
    if (STAGE) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 xv = lds128(item + tok_off + (8 * nt + g) * rs + t * 16);
        expand4(xv, blo[nt], bhi[nt]);
        if (PER_GROUP) {
          const float2 s2 = *reinterpret_cast<const float2*>(sx_s + gi * TOK + 8 * nt + 2 * t);
          sx_c[nt][0] = s2.x; sx_c[nt][1] = s2.y;
        }
      }
      if (PER_GROUP) {
#pragma unroll
        for (int mt = 0; mt < MTILES; ++mt) {
          sw_c[mt][0] = lds_f32(item + CHUNK + TOK * 64 + (16 * mt + g) * 4);
          sw_c[mt][1] = lds_f32(item + CHUNK + TOK * 64 + (16 * mt + g + 8) * 4);
        }
      }
    }
    const uint32_t base = item + g * rs + t * 16;
#pragma unroll
    for (int mt = 0; mt < MTILES; ++mt) {
      const uint4 ra = lds128(base + mt * 16 * rs);
      const uint4 rb = lds128(base + mt * 16 * rs + 8 * rs);
      uint32_t alo[4], ahi[4], a8lo[4], a8hi[4];
      expand4(ra, alo, ahi);
      expand4(rb, a8lo, a8hi);
      if (PER_GROUP) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) c[mt][nt][i] = 0;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_s8(c[mt][nt], alo[j], a8lo[j], ahi[j], a8hi[j], blo[nt][j], bhi[nt][j]);
      if (PER_GROUP) {
        // reference order: (acc * scale_x[g, m]) * scale_w[g, n]; 2^-8 rides on the token scale (exact)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          f[mt][nt][0] = fmaf(__int2float_rn(c[mt][nt][0]) * sx_c[nt][0], sw_c[mt][0], f[mt][nt][0]);
          f[mt][nt][1] = fmaf(__int2float_rn(c[mt][nt][1]) * sx_c[nt][1], sw_c[mt][0], f[mt][nt][1]);
          f[mt][nt][2] = fmaf(__int2float_rn(c[mt][nt][2]) * sx_c[nt][0], sw_c[mt][1], f[mt][nt][2]);
          f[mt][nt][3] = fmaf(__int2float_rn(c[mt][nt][3]) * sx_c[nt][1], sw_c[mt][1], f[mt][nt][3]);
        }
      }
    }
  }

  // ---- add the warps' ranges in ascending order ----
  __syncthreads();   // every warp is done with its staged bytes: the region becomes [warp][token][row] partial sums
  {
    uint32_t* red = reinterpret_cast<uint32_t*>(smem) + (size_t)warp * TOK * ROWS;
#pragma unroll
    for (int mt = 0; mt < MTILES; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = 16 * mt + g + (i >> 1) * 8, tok = 8 * nt + 2 * t + (i & 1);
          red[tok * ROWS + row] = PER_GROUP ? __float_as_uint(f[mt][nt][i]) : (uint32_t)c[mt][nt][i];
        }
  }
  __syncthreads();
  for (int o = threadIdx.x; o < TOK * ROWS; o += nwarps * 32) {
    const int tok = o / ROWS, row = o - tok * ROWS;
    if (tok >= p.M) continue;
    const uint32_t* red = reinterpret_cast<const uint32_t*>(smem) + o;
    float v;
    if (PER_GROUP) {
      v = __uint_as_float(red[0]);
#pragma unroll
      for (int w2 = 1; w2 < nwarps; ++w2) v += __uint_as_float(red[(size_t)w2 * TOK * ROWS]);
    } else {
      int s = (int)red[0];
#pragma unroll
      for (int w2 = 1; w2 < nwarps; ++w2) s += (int)red[(size_t)w2 * TOK * ROWS];
      // reference order: (acc * scale_b[n]) * scale_a[m]
      v = (__int2float_rn(s) * (__ldg(p.sw + n0 + row) * (1.0f / 256.0f))) * __ldg(p.sx + tok);
    }
    const long long idx = (long long)tok * p.N + n0 + row;
    if (p.out_fp16) static_cast<__half*>(p.out)[idx] = __float2half_rn(v);
    else static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
  }
}

int skinny_rstride(int gper) { return gper * 64 + ((gper % 2 == 0) ? 64 : 0); }

size_t skinny_smem(int warps, int rows, int nt, int gper, bool per_group, bool stage, bool rowmajor) {
  const size_t region = rowmajor ? (size_t)(rows + (stage ? 8 * nt : 0)) * skinny_rstride(gper)
                                 : (size_t)gper * skinny_item(rows, 8 * nt, stage);
  const size_t item_bytes = (size_t)warps * region;
  const size_t sx_bytes = (stage && per_group) ? (size_t)warps * gper * 8 * nt * 4 : 0;
  const size_t red_bytes = (size_t)warps * (8 * nt) * rows * 4;
  return (item_bytes + sx_bytes > red_bytes ? item_bytes + sx_bytes : red_bytes) + (size_t)warps * kMaxGroupsPerWarp * 8;
}

template <int MTILES, int NT, bool PER_GROUP, bool STAGE>
int launch_one(const SkinnyParams& p, size_t smem, cudaStream_t st) {
  static bool configured[64] = {false};
  int dev = 0;
  I4TC_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    I4TC_CUDA(cudaFuncSetAttribute(w4a4_skinny_kernel<MTILES, NT, PER_GROUP, STAGE>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    configured[dev] = true;
  }
  w4a4_skinny_kernel<MTILES, NT, PER_GROUP, STAGE><<<p.N / (16 * MTILES), skinny_warps(MTILES) * 32, smem, st>>>(p);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

template <int MTILES, bool PER_GROUP, bool STAGE>
int launch_nt(const SkinnyParams& p, int nt, size_t smem, cudaStream_t st) {
  switch (nt) {
    case 1: return launch_one<MTILES, 1, PER_GROUP, STAGE>(p, smem, st);
    case 2: return launch_one<MTILES, 2, PER_GROUP, STAGE>(p, smem, st);
    default: break;
  }
  if constexpr (MTILES == 1) {   // 32-row tiles exist for up to 16 tokens only
    if (nt == 3) return launch_one<MTILES, 3, PER_GROUP, STAGE>(p, smem, st);
    if (nt == 4) return launch_one<MTILES, 4, PER_GROUP, STAGE>(p, smem, st);
  }
  return fail(I4TC_EINVAL, "unsupported token count");
}

struct SkinnyPlan {
  int rows = 0;        // 0: the shape does not fit
  int warps = 16;
  int gper = 0;
  bool stage = false;
  size_t smem = 0;
};

// Rows per block: 32 when that still gives every SM two blocks (and there are at most 16 tokens), else 16.  The tokens are staged in shared memory when
// at least two blocks still fit an SM.
SkinnyPlan skinny_plan(long long M, long long N, long long K, bool per_group, bool rowmajor, int sm_count) {
  SkinnyPlan pl;
  const int G = (int)(K / 128), nt = (int)((M + 7) / 8);
  for (int rows : {32, 16}) {
    if (N % rows != 0) continue;
    if (rows == 32 && (N / 32 < 2ll * sm_count || nt > 2)) continue;   // (two row tiles x four token tiles would spill)
    const int warps = skinny_warps(rows / 16);
    const int gper = (G + warps - 1) / warps;
    if (gper > kMaxGroupsPerWarp) continue;
    // (row-major operands with per-group scales: no call site; the scales would need a layout of their own)
    const size_t staged = (rowmajor && per_group) ? (size_t)-1 : skinny_smem(warps, rows, nt, gper, per_group, true, rowmajor);
    const size_t plain = skinny_smem(warps, rows, nt, gper, per_group, false, rowmajor);
    pl.warps = warps;
    pl.gper = gper;
    if (staged <= 110 * 1024) {
      pl.rows = rows; pl.stage = true; pl.smem = staged;
      return pl;
    }
    if (plain <= 220 * 1024) {
      pl.rows = rows; pl.stage = false; pl.smem = plain;
      return pl;
    }
  }
  return pl;
}

}  // namespace

bool skinny_applicable(long long M, long long N, long long K, int epi_mode, bool rowmajor, int sm_count) {
  if (M < 1 || M > 32 || N < 16 || K < 128 || K % 128 != 0 || K > 65536) return false;
  if (epi_mode != EPI_GROUP && epi_mode != EPI_CHANNEL) return false;
  // per-channel scales: the tile kernel has no per-group drain and is the faster one beyond 16 tokens (measured)
  if (epi_mode == EPI_CHANNEL && M > 16) return false;
  return skinny_plan(M, N, K, epi_mode == EPI_GROUP, rowmajor, sm_count).rows != 0;
}

int launch_w4a4_skinny(const uint8_t* x, const uint8_t* w, const float* sx, const float* sw, void* out, int out_dtype,
                       long long M, long long N, int G, bool rowmajor, int epi_mode, int sm_count, unsigned int* status,
                       cudaStream_t st) {
  SkinnyParams p;
  p.x = x; p.w = w; p.sx = sx; p.sw = sw; p.out = out;
  p.M = (int)M; p.N = (int)N; p.G = G;
  if (rowmajor) {
    p.x_row = p.w_row = (long long)G * 64; p.x_grp = p.w_grp = 64;
  } else {
    p.x_row = p.w_row = 64; p.x_grp = M * 64; p.w_grp = N * 64;
  }
  p.rowmajor = rowmajor ? 1 : 0;
  p.out_fp16 = out_dtype == I4TC_FP16;
  p.status = status;
  I4TC_REQUIRE(aligned_to(x, 16) && aligned_to(w, 16), I4TC_EALIGN, "packed operands must be 16-byte aligned");
  const bool pg = epi_mode == EPI_GROUP;
  SkinnyPlan pl = skinny_plan(M, N, (long long)G * 128, pg, rowmajor, sm_count);
  I4TC_REQUIRE(pl.rows != 0, I4TC_EINVAL, "shape not supported by the small-batch kernel");
  const int nt = (int)((M + 7) / 8);
  p.gper = pl.gper;
  p.rstride = skinny_rstride(pl.gper);
  p.warps = pl.warps;
  if (pl.stage && pg && !aligned_to(sw, 16)) {   // the bulk copy of the row scales needs 16-byte alignment
    pl.stage = false;
    pl.smem = skinny_smem(pl.warps, pl.rows, nt, pl.gper, pg, false, rowmajor);
  }
#define I4TC_SKINNY_CASE(MT_, PG_, ST_) \
  if (pl.rows == 16 * MT_ && pg == PG_ && pl.stage == ST_) return launch_nt<MT_, PG_, ST_>(p, nt, pl.smem, st);
  I4TC_SKINNY_CASE(1, true, true)
  I4TC_SKINNY_CASE(1, true, false)
  I4TC_SKINNY_CASE(1, false, true)
  I4TC_SKINNY_CASE(1, false, false)
  I4TC_SKINNY_CASE(2, true, true)
  I4TC_SKINNY_CASE(2, true, false)
  I4TC_SKINNY_CASE(2, false, true)
  I4TC_SKINNY_CASE(2, false, false)
#undef I4TC_SKINNY_CASE
  return fail(I4TC_EINVAL, "unsupported configuration");
}

}  // namespace i4tc
