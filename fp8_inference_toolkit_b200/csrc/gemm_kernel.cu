// Persistent warp-specialised W4A4 GEMM kernel for sm_100a (tcgen05 + TMEM + TMA).
//
// sm_100 tensor cores have no int4 MMA kind, so packed int4 tiles are staged by TMA, expanded
// to int8 by converter warps and multiplied with tcgen05.mma kind::i8 into int32 accumulators
// that live in tensor memory.  One K group of 128 codes is exactly one 128-byte swizzled row of
// int8, i.e. four K=32 MMAs.
//
// Expansion trick: a nibble moved to the top of its byte is the code times 16 as a signed int8
//   hi = w & 0xF0F0F0F0          (odd elements)      lo = (w << 4) & 0xF0F0F0F0   (even elements)
// so both operands carry 16*code, every product is 256*(a*b) and the int32 accumulator is exactly
// 256 times the true sum (|256 * 64 * K| < 2^31 for K <= 65536).  The factor is removed exactly
// in the epilogue (arithmetic shift, or a 2^-8 folded into a scale).  Even and odd elements of a
// 32-code chunk land in different 16-byte K slots; A and B use the same permutation, and integer
// sums do not depend on the order of k.
//
// Roles (512 or 768 threads):
//   warp 0      TMA producer: packed P (128 x 64 B) and Q (BN x 64 B) tiles, one K group per stage
//   warp 1      MMA issuer (one thread runs the whole loop) and owner of the TMEM allocation
//   warps 2-3   per-group mode: copy the row and column scales of each K group into a ring in shared memory
//   warps 4-7   converters: packed stage -> 128B-swizzled K-major int8 stage
//   warps 8-..  epilogue (8 or 16 warps): tcgen05.ld, int32 -> fp32, scales, fp32 accumulation across groups, store
// Two to four TMEM accumulators (BN columns each) let later groups be multiplied while one is drained.
// The MMA thread's loop is the serial path of the kernel (an MMA costs it ~50 cycles, a commit ~48, a barrier probe
// 150-200), so it does the least possible per K group: two overlapped probes (operands converted, accumulator free),
// four MMAs and ONE commit.  With a flush per group that commit's barrier tells the converters "stage free" and the
// epilogue "accumulator full" at once; in a CTA pair it arrives in both CTAs (tcgen05.commit multicast).  With
// per-group scales, where the epilogue warps are the busy ones, this thread also waits for the group's scale stage.
// CG = 2: two CTAs on neighbouring SMs share a 256 x 256 tile (tcgen05.mma.cta_group::2 issued by the first
// one); each stages and converts its own 128 rows of P and only half of the Q rows.
// Every wait is bounded: on expiry the kernel sets bit 0 of the status word, all roles leave
// their loops, TMEM is released and the kernel returns.
#include "gemm.cuh"
#include "ptx.cuh"

namespace i4tc {

using namespace ptx;

constexpr int kBM = 128;             // rows of the P tile == TMEM lanes
constexpr int kPackedRow = 64;       // bytes of one packed row of one group
constexpr int kI8Row = 128;          // bytes of one int8 row of one group (the swizzle width)
constexpr int kConvWarp0 = 4, kConvWarps = 4;
constexpr int kEpiWarp0 = 8;
constexpr int kNS = 4;               // scale stages (per-group epilogue)
constexpr int kScaleWarp0 = 2, kScaleWarps = 2;
// Register budgets per role (whole warpgroups), within what the launch allocates (threads x registers per thread):
//   8 epilogue warps, 512 threads x 128: 128*56 + 128*72 + 256*192 = 65536
//  16 epilogue warps, 768 threads x  80: 128*32 + 128*40 + 512*102 -> 104: 128*24 + 128*40 + 512*104 = 61440
template <int EW> struct Regs;
template <> struct Regs<8> { static constexpr int WG0 = 56, CONV = 64, EPI = 192; static constexpr bool PIPE = false; };
template <> struct Regs<16> { static constexpr int WG0 = 24, CONV = 40, EPI = 104; static constexpr bool PIPE = false; };
//  12 epilogue warps, 640 threads x 96: 128*56 + 128*64 + 384*120 = 61440 (192-column tiles: 64 running sums per thread)
template <> struct Regs<12> { static constexpr int WG0 = 56, CONV = 64, EPI = 120; static constexpr bool PIPE = false; };
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

// CG = 1: one CTA computes a 128 x BN tile.  CG = 2: a pair of CTAs (a cluster of two SMs) computes a
// 256 x BN tile with tcgen05.mma.cta_group::2; each CTA stages its own 128 P rows and only BN / 2 rows of
// the Q operand, so a third less is converted and moved through shared memory per unit of MMA work.
// EW = number of epilogue warps (8 or 16): a drain is a chain of TMEM round trips and dependent conversions, so
// four warps per scheduler hide what two cannot; 16 warps hold BN / 4 columns of running sums each.
template <int BN, int CG = 1, int EW = 8>
struct Cfg {
  static_assert(EW == 8 || EW == 12 || EW == 16, "8, 12 or 16 epilogue warps");
  static_assert(BN % (EW / 4) == 0 && (BN / (EW / 4)) % 32 == 0, "every epilogue warp drains whole 32-column chunks");
  static_assert(BN / (EW / 4) >= 32, "an epilogue warp drains at least one 32-column chunk");
  static constexpr int EPI_WARPS = EW;
  static constexpr int THREADS = (kEpiWarp0 + EW) * 32;
  static constexpr int QR = BN / CG;                                   // Q rows staged by this CTA
  static constexpr int NP = (CG == 2) ? 4 : ((BN >= 128) ? 5 : 6);     // packed stages
  static constexpr int NI = (CG == 2) ? 4 : (BN >= 192 ? 2 : 4);       // int8 stages
  // TMEM accumulators: as many as fit in the 512 columns (at most 4), so that narrow tiles -- whose K loop is a
  // chain of short handshakes -- find a free accumulator and a converted stage without waiting
  static constexpr int NT = (BN >= 192) ? 2 : 4;
  // With a flush per group the epilogue waits on the barrier ring of the int8 stages.  Group j + NI can only be
  // multiplied after group j + NI - NT was drained, so with NI >= NT a barrier never completes a second phase
  // before the epilogue has seen the first.
  static_assert(NI >= NT, "the int8 stage ring must be at least as deep as the accumulator ring");
  static constexpr int PK_P = kBM * kPackedRow;                        // 8 KB
  static constexpr int PK_Q = QR * kPackedRow;
  static constexpr int I8_P = kBM * kI8Row;                            // 16 KB
  static constexpr int I8_Q = QR * kI8Row;
  static constexpr int COLS_PER_WARP = BN / (EW / 4);                  // epilogue columns per warp
  static constexpr int TMEM_COLS = (NT * BN > 256) ? 512 : 256;        // allocation: a power of two >= 32
  // shared memory layout (offsets from a 1024-byte aligned base)
  static constexpr int OFF_I8 = 0;
  static constexpr int OFF_PK = OFF_I8 + NI * (I8_P + I8_Q);
  // scale stages of the per-group epilogue: kBM row scales then BN column scales of one K group;
  // the one-flush epilogues use the start of the same region for their per-warp column scales
  static constexpr int OFF_SQ = OFF_PK + NP * (PK_P + PK_Q);
  static constexpr int SCALE_STAGE = (kBM + BN) * 4;                  // bytes
  static constexpr int SQ_BYTES = (kNS * SCALE_STAGE > EW * COLS_PER_WARP * 4) ? kNS * SCALE_STAGE : EW * COLS_PER_WARP * 4;
  static constexpr int OFF_BAR = OFF_SQ + SQ_BYTES;
  static constexpr int NUM_BARS = 2 * NP + 2 * NI + 2 * NT + 3 * kNS;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;              // tmem ptr, abort flag
  static constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;              // + alignment slack
};

struct TileInfo {
  int p0, q0;        // first row of the P / Q tile
  int p_lim, q_lim;  // exclusive row limits for output
  int zq;            // slab offset of the Q operand (MoE: expert * G)
  long long sq_off;  // float offset into sq (MoE: expert * sq_estride)
  int g0, g1;        // K groups [g0, g1) of this work item (all of them unless split-K)
  int split;
};

// Static persistent schedule: CTA b takes tiles b, b + grid, ...  P tiles vary fastest so that
// CTAs running together share Q (weight) tiles in L2.
// With CG = 2 a work item is a 256-row P tile of a CTA pair; rank r of the pair owns rows 128 r .. 128 r + 127
// of it (p.num_p_tiles then counts 256-row tiles).
template <int CG = 1>
struct SchedT {
  int tile;
  int e;
  int tile_base;
  int rank;
  __device__ SchedT() : tile(blockIdx.x / CG), e(0), tile_base(0), rank(CG == 2 ? (int)cluster_ctarank() : 0) {}
  template <int BN>
  __device__ bool next(const GemmParams& p, TileInfo& ti) {
    if (p.expert_offsets == nullptr) {
      const int per_split = p.num_p_tiles * p.num_q_tiles;
      if (tile >= per_split * p.splits) return false;
      const int sp = tile / per_split, local = tile - sp * per_split;
      const int pt = local % p.num_p_tiles, qt = local / p.num_p_tiles;
      ti.p0 = pt * (kBM * CG) + rank * kBM; ti.q0 = qt * BN; ti.p_lim = p.P_rows; ti.q_lim = p.Q_rows; ti.zq = 0; ti.sq_off = 0;
      ti.split = sp; ti.g0 = sp * p.groups_per_split;
      ti.g1 = min(p.G, ti.g0 + p.groups_per_split);
    } else {
      for (;;) {
        if (e >= p.num_experts) return false;
        const int r0 = __ldg(p.expert_offsets + e), r1 = __ldg(p.expert_offsets + e + 1);
        const int npt = (r1 - r0 + kBM - 1) / kBM;
        const int nt = npt * p.num_q_tiles;
        if (tile < tile_base + nt) {
          const int local = tile - tile_base;
          const int pt = local % npt, qt = local / npt;
          ti.p0 = r0 + pt * kBM; ti.p_lim = r1; ti.q0 = qt * BN; ti.q_lim = p.Q_rows;
          ti.zq = e * p.G; ti.sq_off = (long long)e * p.sq_estride;
          ti.split = 0; ti.g0 = 0; ti.g1 = p.G;
          break;
        }
        tile_base += nt; ++e;
      }
    }
    tile += gridDim.x / CG;
    return true;
  }
};
using Sched = SchedT<1>;

// Bounded mbarrier wait, uniform across the warp.  Returns false (and raises the abort flag)
// when the limit expires or another role has already aborted.  The common case -- the phase has
// already completed -- is one non-blocking probe; everything else is the rare path.
__device__ __forceinline__ bool wait_bar_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  bool ok = mbar_try_wait(bar, parity);
  if (!ok) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
      ok = mbar_try_wait(bar, parity);
      if (ok) break;
      if ((++spins & 63u) == 0) {
        if (*abort_flag) break;
        if (globaltimer_ns() - t0 > kWaitLimitNs) break;
      }
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) *abort_flag = 1;
  return ok;
}
// The same wait for a role that runs as a single thread (no warp vote).
__device__ __forceinline__ bool wait_bar_thread(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;
  bool ok = mbar_try_wait(bar, parity);
  if (!ok) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
      ok = mbar_try_wait(bar, parity);
      if (ok) break;
      if ((++spins & 63u) == 0) {
        if (*abort_flag) break;
        if (globaltimer_ns() - t0 > kWaitLimitNs) break;
      }
    }
  }
  if (!ok) *abort_flag = 1;
  return ok;
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (__all_sync(0xffffffffu, mbar_test_wait(bar, parity))) return true;
  return wait_bar_slow(bar, parity, abort_flag);
}

// Arrival on a barrier that, for CG = 2, may live in the peer CTA (`bar` is then a shared::cluster address).
template <int CG>
__device__ __forceinline__ void arrive_bar(uint32_t bar) {
  if (CG == 2) mbar_arrive_cluster(bar);
  else mbar_arrive(bar);
}

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  // K-major, 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart (SBO), LBO unused (1),
  // descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int BN, int CG>
__device__ __forceinline__ constexpr uint32_t make_idesc() {
  // D = S32 (2 << 4), A = B = signed int8 (1 << 7, 1 << 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((kBM * CG) >> 4) << 24);
}

// Row order of a converted Q tile.  After tcgen05.ld.16x256b a lane (lr, lq) holds, of every 32-column chunk, the column
// pairs 8 kk + 2 lq + {0, 1}, kk = 0..3.  The converters therefore store Q row n of a 32-row block at row
// qperm(n) = 8 * ((n >> 1) & 3) + 2 * (n >> 3) + (n & 1): accumulator column 8 kk + 2 lq + e is then output column
// 8 lq + 2 kk + e, a lane's four pairs are eight CONSECUTIVE output columns, and a chunk row leaves as one 16-byte store
// per lane with no exchange between lanes (a 4 x 4 transpose in the quad costs 4 shuffles and 16 selects per chunk row).
// The map is its own inverse.  Tiles that reach shared memory without the converters (int8 operands) keep the
// natural order (QP = false below).
__host__ __device__ constexpr int qperm(int n) {
  return (n & ~31) | (((n >> 1) & 3) << 3) | (((n >> 3) & 3) << 1) | (n & 1);
}
// first of the two output columns (inside a 32-column chunk) of a lane's pair kk
template <bool QP>
__device__ __forceinline__ constexpr int pair_col(int kk, int lq) { return QP ? lq * 8 + kk * 2 : kk * 8 + lq * 2; }

// Expand the packed P tile (ROWS_P x 64 B, dense) and Q tile (ROWS_Q x 64 B) of one stage into swizzled int8 tiles
// (rows x 128 B).  16-byte packed chunk j of a row becomes int8 chunks 2j (even codes) and 2j+1 (odd codes).
// The two tiles are walked as one list of chunks, up to six loads in flight per thread, so that a narrow stage
// (64 or 128 Q rows) is one round trip to shared memory instead of one per tile.
template <int ROWS_P, int ROWS_Q>
__device__ __forceinline__ void convert_stage(uint32_t pkP, uint32_t i8P, uint32_t pkQ, uint32_t i8Q, int tid) {
  constexpr int NT = kConvWarps * 32;
  static_assert((ROWS_P * 4) % NT == 0 && (ROWS_Q * 4) % NT == 0, "tile rows must be a multiple of 32");
  constexpr int TP = ROWS_P * 4 / NT, TQ = ROWS_Q * 4 / NT, T = TP + TQ;
  constexpr int BATCH = 6;
#pragma unroll
  for (int i0 = 0; i0 < T; i0 += BATCH) {
    uint4 w[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int c = i0 + i;
      if (c < T) w[i] = lds128((c < TP ? pkP : pkQ) + (uint32_t)(tid + (c < TP ? c : c - TP) * NT) * 16u);
    }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int c = i0 + i;
      if (c < T) {
        const int q = tid + (c < TP ? c : c - TP) * NT;
        const int row = (c < TP) ? (q >> 2) : qperm(q >> 2), j = q & 3;   // Q rows in the order the epilogue wants
        uint4 lo, hi;
        lo.x = (w[i].x << 4) & 0xF0F0F0F0u; hi.x = w[i].x & 0xF0F0F0F0u;
        lo.y = (w[i].y << 4) & 0xF0F0F0F0u; hi.y = w[i].y & 0xF0F0F0F0u;
        lo.z = (w[i].z << 4) & 0xF0F0F0F0u; hi.z = w[i].z & 0xF0F0F0F0u;
        lo.w = (w[i].w << 4) & 0xF0F0F0F0u; hi.w = w[i].w & 0xF0F0F0F0u;
        const uint32_t c0 = (uint32_t)((2 * j) ^ (row & 7));
        const uint32_t base = (c < TP ? i8P : i8Q) + (uint32_t)row * kI8Row;
        sts128(base + c0 * 16u, lo);
        sts128(base + (c0 ^ 1u) * 16u, hi);
      }
    }
  }
}

template <typename OutT>
__device__ __forceinline__ OutT cast_out(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }

// Stores 32 consecutive int32 values of one tile row (normal) or of one tile column spread over 32 rows
// (swap); the accumulators are 256 x the integer sums.
__device__ __forceinline__ void store_chunk_i(const GemmParams& p, int32_t* out, const uint32_t (&r)[32], int prow,
                                              int qcol0, const TileInfo& ti) {
  if (prow >= ti.p_lim) return;
  if (!p.swap) {
    int32_t* dst = out + (long long)prow * p.ldc + qcol0;
    const bool vec = (qcol0 + 32 <= ti.q_lim) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
    // accumulator column i of the chunk is output column qperm(i); output columns n .. n + 3 are r[qperm(n .. n + 3)]
    if (vec) {
#pragma unroll
      for (int n = 0; n < 32; n += 4) {
        int4 o = make_int4(((int32_t)r[qperm(n)]) >> 8, ((int32_t)r[qperm(n + 1)]) >> 8, ((int32_t)r[qperm(n + 2)]) >> 8,
                           ((int32_t)r[qperm(n + 3)]) >> 8);
        *reinterpret_cast<int4*>(dst + n) = o;
      }
    } else {
#pragma unroll
      for (int n = 0; n < 32; ++n)
        if (qcol0 + n < ti.q_lim) dst[n] = ((int32_t)r[qperm(n)]) >> 8;
    }
  } else {
#pragma unroll
    for (int n = 0; n < 32; ++n)
      if (qcol0 + n < ti.q_lim) out[(long long)(qcol0 + n) * p.ldc + prow] = ((int32_t)r[qperm(n)]) >> 8;
  }
}

// 4 x 4 transpose inside a quad of lanes (two butterfly exchanges).  On entry lane lq of the quad holds
// x[kk], kk = 0..3; on return it holds { x of lane 0, 1, 2, 3 }[kk = lq].  With x[kk] = the packed pair of
// columns 8 kk + 2 lq + {0, 1} this gives every lane 8 consecutive 16-bit columns (8 lq .. 8 lq + 7).
__device__ __forceinline__ uint4 quad_transpose(const uint32_t (&x)[4], int lq) {
  const bool odd = (lq & 1) != 0, hi = (lq & 2) != 0;
  // exchange with lane ^ 1: keep the pairs whose kk has my low bit, receive the partner's
  const uint32_t r0 = __shfl_xor_sync(0xffffffffu, odd ? x[0] : x[1], 1);
  const uint32_t r1 = __shfl_xor_sync(0xffffffffu, odd ? x[2] : x[3], 1);
  const uint32_t own0 = odd ? x[1] : x[0], own1 = odd ? x[3] : x[2];
  const uint32_t u00 = odd ? r0 : own0, u01 = odd ? own0 : r0;   // kk = (lq & 1), from the even / odd lane
  const uint32_t u10 = odd ? r1 : own1, u11 = odd ? own1 : r1;   // kk = (lq & 1) + 2
  // exchange with lane ^ 2: keep kk's high bit == (lq >> 1)
  const uint32_t t0 = __shfl_xor_sync(0xffffffffu, hi ? u00 : u10, 2);
  const uint32_t t1 = __shfl_xor_sync(0xffffffffu, hi ? u01 : u11, 2);
  const uint32_t k0 = hi ? u10 : u00, k1 = hi ? u11 : u01;
  uint4 y;
  y.x = hi ? t0 : k0; y.y = hi ? t1 : k1; y.z = hi ? k0 : t0; y.w = hi ? k1 : t1;
  return y;
}

template <typename OutT>
__device__ __forceinline__ uint32_t pack_pair(float2 v) {
  union { OutT h[2]; uint32_t u; } pk;
  pk.h[0] = cast_out<OutT>(v.x); pk.h[1] = cast_out<OutT>(v.y);
  return pk.u;
}

// Writes the column pair (q, q + 1) of tile row prow without any alignment assumption beyond what
// `pair_ok` promises (even ldc, 4-byte aligned base): 16-bit output, normal or swapped orientation.
template <typename OutT, bool SWAP>
__device__ __forceinline__ void store_pair(OutT* out, long long ldc, int prow, int q, int q_lim, float2 v, bool pair_ok) {
  if (!SWAP) {
    OutT* dst = out + (long long)prow * ldc + q;
    if (q + 1 < q_lim && pair_ok) {
      *reinterpret_cast<uint32_t*>(dst) = pack_pair<OutT>(v);
    } else {
      if (q < q_lim) dst[0] = cast_out<OutT>(v.x);
      if (q + 1 < q_lim) dst[1] = cast_out<OutT>(v.y);
    }
  } else {
    if (q < q_lim) out[(long long)q * ldc + prow] = cast_out<OutT>(v.x);
    if (q + 1 < q_lim) out[(long long)(q + 1) * ldc + prow] = cast_out<OutT>(v.y);
  }
}

// ------------------------------------------------------------------------------------------
// Epilogue bodies
// ------------------------------------------------------------------------------------------
// Per-group accumulate: a flush per K group, fp32 running sums in registers.
//
// Register layout.  A warp owns 32 TMEM lanes (tile rows) and COLS_PER_WARP columns.  It drains them in
// "slabs" of 16 rows x 32 columns with tcgen05.ld.16x256b.x4: lane (lr = lane / 4, lq = lane % 4) then holds
// rows {lr, lr + 8} of the slab and column pairs 8 * kk + 2 * lq + {0, 1}, kk = 0..3.  Over the two slabs of
// a 32-column chunk a thread therefore owns 4 rows (8 * a + lr, a = 0..3) and, per row, adjacent column
// pairs: the pair is the unit of the packed f32x2 arithmetic and of the scale reads (one 8-byte shared
// load per pair, the same address in the 8 lanes that share lq).
//
// Scales.  Two otherwise idle warps copy the kBM row scales and BN column scales of each K group from
// global to shared memory (4-byte cp.async, kNS stages ahead, completion signalled on an mbarrier), so the
// epilogue warps spend no instructions or registers on global addresses.
// AZP: the zero-point term of asymmetric activations, acc_g + zp[p] * zq[q] before the scales (one more packed
// multiply-add per pair; an exact integer below 2^24 like acc_g itself).  The two extra vectors of a group travel
// with its scales: the ring then holds two stages of double size instead of four.
template <int BN, typename OutT, bool SWAP, int CG, int EW, bool AZP>
__device__ __forceinline__ void epilogue_group(const GemmParams& p, uint8_t* smem, uint32_t tmem_base,
                                               uint32_t bar_done, uint32_t bar_tm_empty, uint32_t bar_sc_full,
                                               uint32_t bar_sc_empty, volatile int* abort_flag) {
  using C = Cfg<BN, CG, EW>;
  constexpr int CW = C::COLS_PER_WARP;
  constexpr int NCH = CW / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ew = warp - kEpiWarp0;
  const int quad = warp & 3;         // TMEM lane quarter this warp may access
  const int part = ew >> 2;          // which CW-wide part of the BN columns
  const int col_base = part * CW;
  const int lq = lane & 3, lr = lane >> 2;
  const float* sc = reinterpret_cast<const float*>(smem + C::OFF_SQ);
  // order of the two multiplies: normal (p = m): (acc * sp) * sq ; swapped (p = n): (acc * sq) * sp.
  // The accumulators are 256 x the integer sums; 2^-8 rides on the row-side scale (exact in both orders).
  constexpr bool pq_order = !SWAP;
  const float kInv256 = p.acc_unit;   // 2^-8 for packed int4 operands (both carry 16 x code)
  constexpr uint32_t NS = AZP ? kNS / 2 : kNS;                       // scale stages in the ring
  constexpr int STAGE_F = (AZP ? 2 : 1) * (C::SCALE_STAGE / 4);      // floats per stage

  SchedT<CG> sched;
  TileInfo ti;
  uint32_t flush = 0;
  while (sched.template next<BN>(p, ti)) {
    float2 f[CW / 2];   // [a][c][kk]: row 8a + lr, columns c * 32 + kk * 8 + 2 lq + {0, 1}
#pragma unroll
    for (int i = 0; i < CW / 2; ++i) f[i] = make_float2(0.f, 0.f);
    bool ok = true;
    // Software pipeline over the slabs: the load of slab u + 1 is in flight while slab u is folded in, and the first
    // slab of the next group is requested under the last slab of this one (when its accumulator and scales are
    // already there), so a warp's drain is not a chain of TMEM round trips.  rb[u & 1] holds slab u; a group has
    // an even number of slabs, so every group starts in rb[0].
    constexpr int S = 2 * NCH;
    constexpr bool PIPE = Regs<EW>::PIPE;   // the second slab buffer needs 16 more registers
    uint32_t rb[PIPE ? 2 : 1][16];
    bool pre = false;      // the first slab of group `flush` was requested under the previous group's last slab
    for (int g = ti.g0; g < ti.g1; ++g) {
      // group number `flush` is done when the commit behind its MMAs arrives on the barrier of its int8 stage
      // (the one the converters wait for before they reuse the stage); its scales have their own ring
      const uint32_t ss = flush % NS;
      const uint32_t buf = flush % C::NT;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + col_base;
      if (!pre) {
        // (the MMA thread waited for this group's scale stage before it issued the group)
        ok = wait_bar(bar_done + (flush % C::NI) * 8, (flush / C::NI) & 1u, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        if (PIPE) tmem_ld_16x256b_x4(taddr, rb[0]);
      }
      const float* st_p = sc + ss * STAGE_F + quad * 32;         // this warp's 32 row scales
      const float* st_q = sc + ss * STAGE_F + kBM + col_base;    // this warp's CW column scales
      float2 sp2[4], zp2[AZP ? 4 : 1];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float v = st_p[8 * a + lr] * kInv256;
        sp2[a] = make_float2(v, v);
        if (AZP) {
          // the accumulators are 256 x the integer sums, so the zero-point term is scaled alike (exact)
          const float z = st_p[(kBM + BN) + 8 * a + lr] * 256.0f;
          zp2[a] = make_float2(z, z);
        }
      }
#pragma unroll
      for (int u = 0; u < S; ++u) {
        const int c = u >> 1, sl = u & 1;
        if (!PIPE) tmem_ld_16x256b_x4(taddr + ((uint32_t)(sl * 16) << 16) + c * 32, rb[0]);
        tmem_ld_wait();   // slab u has arrived in rb[u & 1]
        if (u + 1 < S) {
          if (PIPE) tmem_ld_16x256b_x4(taddr + ((uint32_t)(((u + 1) & 1) * 16) << 16) + ((u + 1) >> 1) * 32, rb[(u + 1) & 1]);
        } else {
          // all of this warp's part of the buffer is in registers: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) arrive_bar<CG>(bar_tm_empty + buf * 8);
          pre = false;
          if (g + 1 < ti.g1) {
            const uint32_t nf = flush + 1;
            const bool ready = mbar_test_wait(bar_done + (nf % C::NI) * 8, (nf / C::NI) & 1u);
            if (__all_sync(0xffffffffu, ready)) {
              tc_fence_after_sync();
              if (PIPE) tmem_ld_16x256b_x4(tmem_base + ((uint32_t)(quad * 32) << 16) + (nf % C::NT) * BN + col_base, rb[0]);
              pre = true;
            }
          }
        }
        const uint32_t (&r)[16] = rb[PIPE ? (u & 1) : 0];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const float2 sq = *reinterpret_cast<const float2*>(st_q + c * 32 + pair_col<true>(kk, lq));
          float2 zq = make_float2(0.f, 0.f);
          if (AZP) zq = *reinterpret_cast<const float2*>(st_q + (kBM + BN) + c * 32 + pair_col<true>(kk, lq));
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int a = sl * 2 + h;
            float2 d = make_float2(__int2float_rn((int32_t)r[4 * kk + 2 * h]),
                                   __int2float_rn((int32_t)r[4 * kk + 2 * h + 1]));
            if (AZP) d = __ffma2_rn(zp2[a], zq, d);
            float2& acc = f[(a * NCH + c) * 4 + kk];
            if (pq_order) acc = __ffma2_rn(__fmul2_rn(d, sp2[a]), sq, acc);
            else acc = __ffma2_rn(__fmul2_rn(d, sq), sp2[a], acc);
          }
        }
      }
      __syncwarp();   // every lane has read its scales of this stage
      if (lane == 0) mbar_arrive(bar_sc_empty + ss * 8);
      ++flush;
    }
    if (PIPE && pre) tmem_ld_wait();   // never taken: a request is only made when another group of this tile follows
    if (!ok) break;
    // ---- write the tile: thread owns rows 8a + lr, column pairs c * 32 + kk * 8 + 2 lq ----
    OutT* out = static_cast<OutT*>(p.out);
    float* ws = (p.split_ws != nullptr) ? p.split_ws + (long long)ti.split * p.ws_stride : nullptr;
    // row addresses from a table (rows of another GPU's buffer, for instance) instead of out + row * ldc
    const unsigned long long* orows = SWAP ? nullptr : p.out_rows;
    const bool vec_ok = !SWAP && ws == nullptr && ((p.ldc & 7) == 0) &&
                        (orows != nullptr || (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (ti.q0 + col_base + CW <= ti.q_lim);
    if (vec_ok) {
      // per row and 32-column chunk the quad holds four column pairs per lane; after the quad transpose
      // each lane writes 8 consecutive columns with one 16-byte store (64 contiguous bytes per quad)
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int prow = ti.p0 + quad * 32 + 8 * a + lr;
        OutT* rowp = nullptr;
        if (prow < ti.p_lim)
          rowp = (orows != nullptr) ? reinterpret_cast<OutT*>(orows[prow]) : out + (long long)prow * p.ldc;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          // a lane's four pairs of a chunk are eight consecutive output columns (see qperm)
          const uint4 y = make_uint4(pack_pair<OutT>(f[(a * NCH + c) * 4 + 0]), pack_pair<OutT>(f[(a * NCH + c) * 4 + 1]),
                                     pack_pair<OutT>(f[(a * NCH + c) * 4 + 2]), pack_pair<OutT>(f[(a * NCH + c) * 4 + 3]));
          if (prow < ti.p_lim) *reinterpret_cast<uint4*>(rowp + ti.q0 + col_base + c * 32 + lq * 8) = y;
        }
      }
    } else {
      const bool pair_ok = ((p.ldc & 1) == 0) && (orows != nullptr || (reinterpret_cast<uintptr_t>(p.out) & 3) == 0);
      // split-K partial sums, unswapped: a lane's four pairs of a chunk are eight consecutive floats of a row
      const bool ws_vec = !SWAP && ws != nullptr && ((p.ldc & 3) == 0) && (ti.q0 + col_base + CW <= ti.q_lim);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int prow = ti.p0 + quad * 32 + 8 * a + lr;
        if (prow >= ti.p_lim) continue;
        // (with a row table: the row's own base and row index 0)
        OutT* obase = (orows != nullptr) ? reinterpret_cast<OutT*>(orows[prow]) : out;
        const int orow = (orows != nullptr) ? 0 : prow;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          if (ws_vec) {
            float4* dst = reinterpret_cast<float4*>(ws + (long long)prow * p.ldc + ti.q0 + col_base + c * 32 + lq * 8);
            const float2 v0 = f[(a * NCH + c) * 4 + 0], v1 = f[(a * NCH + c) * 4 + 1];
            const float2 v2 = f[(a * NCH + c) * 4 + 2], v3 = f[(a * NCH + c) * 4 + 3];
            dst[0] = make_float4(v0.x, v0.y, v1.x, v1.y);
            dst[1] = make_float4(v2.x, v2.y, v3.x, v3.y);
            continue;
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const float2 v = f[(a * NCH + c) * 4 + kk];
            const int q = ti.q0 + col_base + c * 32 + pair_col<true>(kk, lq);
            if (ws != nullptr) {
              // split-K: fp32 partial sums of this K range, element (m, n) at ws[split][m * ldc + n]
              if (!SWAP) {
                float* dst = ws + (long long)prow * p.ldc + q;
                if (q + 1 < ti.q_lim && (p.ldc & 1) == 0) *reinterpret_cast<float2*>(dst) = v;
                else { if (q < ti.q_lim) dst[0] = v.x; if (q + 1 < ti.q_lim) dst[1] = v.y; }
              } else {
                if (q < ti.q_lim) ws[(long long)q * p.ldc + prow] = v.x;
                if (q + 1 < ti.q_lim) ws[(long long)(q + 1) * p.ldc + prow] = v.y;
              }
            } else {
              store_pair<OutT, SWAP>(obase, p.ldc, orow, q, ti.q_lim, v, pair_ok);
            }
          }
        }
      }
    }
  }
}

// One flush per tile with per-channel scales: out = cast((acc * scale_b[n]) * scale_a[m]), the
// reference's order.  Same slab register layout and quad-transposed stores as the per-group epilogue.
template <int BN, typename OutT, bool SWAP, int CG, int EW, bool QP>
__device__ __forceinline__ void epilogue_channel(const GemmParams& p, uint8_t* smem, uint32_t tmem_base,
                                                 uint32_t bar_tm_full, uint32_t bar_tm_empty,
                                                 volatile int* abort_flag) {
  using C = Cfg<BN, CG, EW>;
  constexpr int CW = C::COLS_PER_WARP;
  constexpr int NCH = CW / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ew = warp - kEpiWarp0;
  const int quad = warp & 3;
  const int part = ew >> 2;
  const int col_base = part * CW;
  const int lq = lane & 3, lr = lane >> 2;
  float* sq_s = reinterpret_cast<float*>(smem + C::OFF_SQ) + ew * CW;
  const float kInv256 = p.acc_unit;   // 2^-8 for packed int4 operands, 1 for int8 operands
  // normal: columns are n, so the column scale (scale_b) multiplies first; swapped: rows are n.
  // The first multiplier also carries the 2^-8 that undoes the x16 operand scaling (exact).
  constexpr bool q_first = !SWAP;
  OutT* out = static_cast<OutT*>(p.out);

  SchedT<CG> sched;
  TileInfo ti;
  uint32_t flush = 0;
  bool ok = true;
  while (ok && sched.template next<BN>(p, ti)) {
    __syncwarp();  // the previous tile's reads of sq_s are done
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int q = ti.q0 + col_base + c * 32 + lane;
      const float sv = (q < ti.q_lim) ? __ldg(p.sq + ti.sq_off + q) : 0.f;
      sq_s[c * 32 + lane] = q_first ? sv * kInv256 : sv;
    }
    float spv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int prow = ti.p0 + quad * 32 + 8 * a + lr;
      const float sv = (prow < ti.p_lim) ? __ldg(p.sp + prow) : 0.f;
      spv[a] = q_first ? sv : sv * kInv256;
    }
    __syncwarp();
    const bool vec_ok = !SWAP && ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) &&
                        (ti.q0 + col_base + CW <= ti.q_lim);
    const bool pair_ok = ((p.ldc & 1) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 3) == 0);
    const uint32_t buf = flush % C::NT;
    ok = wait_bar(bar_tm_full + buf * 8, (flush / C::NT) & 1u, abort_flag);
    if (!ok) break;
    tc_fence_after_sync();
    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + col_base;
#pragma unroll
    for (int u = 0; u < 2 * NCH; ++u) {
      const int c = u >> 1, sl = u & 1;
      uint32_t r[16];
      tmem_ld_16x256b_x4(taddr + ((uint32_t)(sl * 16) << 16) + c * 32, r);
      tmem_ld_wait();
      if (u == 2 * NCH - 1) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) arrive_bar<CG>(bar_tm_empty + buf * 8);
      }
      if (p.split_ws != nullptr) {
        // split-K: this work item covers a range of K groups; its integer sums go out as fp32 (exact: below
        // 2^24), element (m, n) at ws[split][m * ldc + n], and a second kernel adds the ranges and scales
        float* ws = p.split_ws + (long long)ti.split * p.ws_stride;
        // unswapped, converted tiles: a lane's four pairs of a chunk are eight consecutive floats of a row
        const bool ws_vec = QP && !SWAP && ((p.ldc & 3) == 0) && (ti.q0 + col_base + CW <= ti.q_lim);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int prow = ti.p0 + quad * 32 + 8 * (sl * 2 + h) + lr;
          if (prow >= ti.p_lim) continue;
          if (ws_vec) {
            float4* dst = reinterpret_cast<float4*>(ws + (long long)prow * p.ldc + ti.q0 + col_base + c * 32 + lq * 8);
            dst[0] = make_float4(__int2float_rn((int32_t)r[2 * h]) * kInv256, __int2float_rn((int32_t)r[2 * h + 1]) * kInv256,
                                 __int2float_rn((int32_t)r[4 + 2 * h]) * kInv256, __int2float_rn((int32_t)r[4 + 2 * h + 1]) * kInv256);
            dst[1] = make_float4(__int2float_rn((int32_t)r[8 + 2 * h]) * kInv256, __int2float_rn((int32_t)r[8 + 2 * h + 1]) * kInv256,
                                 __int2float_rn((int32_t)r[12 + 2 * h]) * kInv256, __int2float_rn((int32_t)r[12 + 2 * h + 1]) * kInv256);
            continue;
          }
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const int q = ti.q0 + col_base + c * 32 + pair_col<QP>(kk, lq);
            const float d0 = __int2float_rn((int32_t)r[4 * kk + 2 * h]) * kInv256;
            const float d1 = __int2float_rn((int32_t)r[4 * kk + 2 * h + 1]) * kInv256;
            if (!SWAP) {
              if (q < ti.q_lim) ws[(long long)prow * p.ldc + q] = d0;
              if (q + 1 < ti.q_lim) ws[(long long)prow * p.ldc + q + 1] = d1;
            } else {
              if (q < ti.q_lim) ws[(long long)q * p.ldc + prow] = d0;
              if (q + 1 < ti.q_lim) ws[(long long)(q + 1) * p.ldc + prow] = d1;
            }
          }
        }
        continue;
      }
      float2 v[2][4];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float2 sq = *reinterpret_cast<const float2*>(sq_s + c * 32 + pair_col<QP>(kk, lq));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float sp = spv[sl * 2 + h];
          const float d0 = __int2float_rn((int32_t)r[4 * kk + 2 * h]);
          const float d1 = __int2float_rn((int32_t)r[4 * kk + 2 * h + 1]);
          v[h][kk] = q_first ? make_float2((d0 * sq.x) * sp, (d1 * sq.y) * sp)
                             : make_float2((d0 * sp) * sq.x, (d1 * sp) * sq.y);
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int prow = ti.p0 + quad * 32 + 8 * (sl * 2 + h) + lr;
        if (vec_ok) {
          uint32_t x[4];
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) x[kk] = pack_pair<OutT>(v[h][kk]);
          // converted tiles: the four pairs are eight consecutive columns already (see qperm)
          const uint4 y = QP ? make_uint4(x[0], x[1], x[2], x[3]) : quad_transpose(x, lq);
          if (prow < ti.p_lim)
            *reinterpret_cast<uint4*>(out + (long long)prow * p.ldc + ti.q0 + col_base + c * 32 + lq * 8) = y;
        } else if (prow < ti.p_lim) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            store_pair<OutT, SWAP>(out, p.ldc, prow, ti.q0 + col_base + c * 32 + pair_col<QP>(kk, lq), ti.q_lim,
                                   v[h][kk], pair_ok);
        }
      }
    }
    ++flush;
  }
}

// One flush per tile (EPI_INT32) or raw per-group dumps (EPI_GROUP_INT32): int32 out = acc >> 8.
// Thread = tile row here (32x32b loads): these are the verification paths, not the fast ones.
template <int BN, int EW>
__device__ __forceinline__ void epilogue_int32(const GemmParams& p, uint32_t tmem_base,
                                               uint32_t bar_tm_full, uint32_t bar_done, uint32_t bar_tm_empty,
                                               volatile int* abort_flag) {
  using C = Cfg<BN, 1, EW>;
  constexpr int NCH = C::COLS_PER_WARP / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ew = warp - kEpiWarp0;
  const int quad = warp & 3;
  const int part = ew >> 2;
  const int col_base = part * C::COLS_PER_WARP;
  const bool per_group = p.epi_mode == EPI_GROUP_INT32;

  Sched sched;
  TileInfo ti;
  uint32_t flush = 0;
  bool ok = true;
  while (ok && sched.template next<BN>(p, ti)) {
    const int prow = ti.p0 + quad * 32 + lane;
    const int nflush = per_group ? (ti.g1 - ti.g0) : 1;
    for (int fl = 0; fl < nflush; ++fl) {
      const uint32_t buf = flush % C::NT;
      // a flush per group: the group's commit arrives on the barrier of its int8 stage (see epilogue_group)
      ok = per_group ? wait_bar(bar_done + (flush % C::NI) * 8, (flush / C::NI) & 1u, abort_flag)
                     : wait_bar(bar_tm_full + buf * 8, (flush / C::NT) & 1u, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * BN + col_base;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (c == NCH - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tm_empty + buf * 8);
        }
        int32_t* out = static_cast<int32_t*>(p.out) + (per_group ? (long long)(ti.g0 + fl) * p.out_gstride : 0ll);
        store_chunk_i(p, out, r, prow, ti.q0 + col_base + c * 32, ti);
      }
      ++flush;
    }
  }
}

// ------------------------------------------------------------------------------------------
// The kernel
// ------------------------------------------------------------------------------------------
template <int BN, int CG, int EW>
__global__ void __launch_bounds__((kEpiWarp0 + EW) * 32, 1)
w4a4_gemm_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap tmP,
                 const __grid_constant__ CUtensorMap tmQ) {
  using C = Cfg<BN, CG, EW>;
  using R = Regs<EW>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTA pair: rank 0 (the leader) issues the MMAs for both CTAs and owns the barriers both CTAs arrive on
  const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;

  const uint32_t bar0 = sbase + C::OFF_BAR;
  const uint32_t bar_pk_full = bar0;
  const uint32_t bar_pk_empty = bar_pk_full + C::NP * 8;
  const uint32_t bar_i8_full = bar_pk_empty + C::NP * 8;
  const uint32_t bar_i8_empty = bar_i8_full + C::NI * 8;
  const uint32_t bar_tm_full = bar_i8_empty + C::NI * 8;
  const uint32_t bar_tm_empty = bar_tm_full + C::NT * 8;
  const uint32_t bar_sc_full = bar_tm_empty + C::NT * 8;
  const uint32_t bar_sc_empty = bar_sc_full + kNS * 8;
  const uint32_t bar_sc_peer = bar_sc_empty + kNS * 8;   // leader only: the second CTA's scale stage has landed
  // where converters and epilogue warps arrive: the leader's barriers (shared::cluster addresses for CG = 2)
  const uint32_t arr_i8_full = (CG == 2) ? mapa_shared(bar_i8_full, 0) : bar_i8_full;
  const uint32_t arr_tm_empty = (CG == 2) ? mapa_shared(bar_tm_empty, 0) : bar_tm_empty;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 8);

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::NP; ++i) { mbar_init(bar_pk_full + i * 8, 1); mbar_init(bar_pk_empty + i * 8, kConvWarps); }
    for (int i = 0; i < C::NI; ++i) { mbar_init(bar_i8_full + i * 8, kConvWarps * CG); mbar_init(bar_i8_empty + i * 8, 1); }
    for (int i = 0; i < C::NT; ++i) { mbar_init(bar_tm_full + i * 8, 1); mbar_init(bar_tm_empty + i * 8, EW * CG); }
    for (int i = 0; i < kNS; ++i) {
      mbar_init(bar_sc_full + i * 8, 32); mbar_init(bar_sc_empty + i * 8, EW); mbar_init(bar_sc_peer + i * 8, 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmP);
    prefetch_tensormap(&tmQ);
  }
  if (warp == 1) {
    if (CG == 2) { tmem_alloc_cg2(smem_u32(tmem_slot), C::TMEM_COLS); tmem_relinquish_cg2(); }
    else { tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS); tmem_relinquish(); }
  }
  tc_fence_before_sync();
  if (CG == 2) cluster_sync();   // the peer's barriers are initialised before anything arrives on them
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Rebalance registers between the roles (whole warpgroups): the epilogue keeps BN / 2 (8 warps) or BN / 4
  // (16 warps) fp32 running sums per thread.  The setmaxnreg of each role sits at the top of that role's branch.

  const bool per_group_flush = (p.epi_mode == EPI_GROUP) || (p.epi_mode == EPI_GROUP_INT32);

  if (warp < 4) {
  setmaxnreg_dec<R::WG0>();
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    SchedT<CG> sched;
    TileInfo ti;
    uint32_t it = 0;
    bool ok = true;
    if (p.i8_operands) {
      // int8 operands: the tiles land in the swizzled int8 stages themselves (the tensor maps swizzle); the stage is
      // free again when the MMAs that read it have completed
      while (ok && sched.template next<BN>(p, ti)) {
        for (int g = ti.g0; g < ti.g1; ++g, ++it) {
          const uint32_t s = it % C::NI, ph = (it / C::NI) & 1u;
          ok = wait_bar(bar_i8_empty + s * 8, ph ^ 1u, abort_flag);
          if (!ok) break;
          if (lane == 0) {
            const uint32_t full = bar_pk_full + s * 8;
            const uint32_t dstP = sbase + C::OFF_I8 + s * (C::I8_P + C::I8_Q);
            const uint32_t dstQ = dstP + C::I8_P;
            mbar_arrive_expect_tx(full, C::I8_P + C::I8_Q);
            tma_load_2d(dstP, &tmP, full, g * kI8Row, ti.p0);
            tma_load_2d(dstQ, &tmQ, full, g * kI8Row, ti.q0 + (int)rank * C::QR);
          }
          __syncwarp();
        }
      }
    } else {
    while (ok && sched.template next<BN>(p, ti)) {
      for (int g = ti.g0; g < ti.g1; ++g, ++it) {
        const uint32_t s = it % C::NP, ph = (it / C::NP) & 1u;
        ok = wait_bar(bar_pk_empty + s * 8, ph ^ 1u, abort_flag);
        if (!ok) break;
        if (lane == 0) {
          const uint32_t full = bar_pk_full + s * 8;
          const uint32_t dstP = sbase + C::OFF_PK + s * (C::PK_P + C::PK_Q);
          const uint32_t dstQ = dstP + C::PK_P;
          mbar_arrive_expect_tx(full, C::PK_P + C::PK_Q);
          if (p.p_rowmajor) tma_load_2d(dstP, &tmP, full, g * kPackedRow, ti.p0);
          else tma_load_3d(dstP, &tmP, full, 0, ti.p0, g);
          const int qrow = ti.q0 + (int)rank * C::QR;   // CG = 2: this CTA stages half of the Q tile
          if (p.q_rowmajor) tma_load_2d(dstQ, &tmQ, full, g * kPackedRow, qrow);
          else tma_load_3d(dstQ, &tmQ, full, 0, qrow, ti.zq + g);
        }
        __syncwarp();
      }
    }
    }
    if (!ok) {
      // aborting: wait (bounded) for copies that may still be in flight into this CTA's shared memory
      const uint32_t depth = p.i8_operands ? (uint32_t)C::NI : (uint32_t)C::NP;
      const uint32_t n = it < depth ? it : depth;
      for (uint32_t j = it - n; j < it; ++j) {
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(bar_pk_full + (j % depth) * 8, (j / depth) & 1u)) {
          if (globaltimer_ns() - t0 > 100000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (CG = 2: the leader CTA only) ----------------
    // One thread runs the whole loop: the loop is the serial path of every small tile, and a warp-wide version
    // pays a vote and a reconvergence (~250 cycles) per K group for nothing.
    if (leader && lane == 0) {
    constexpr uint32_t idesc = make_idesc<BN, CG>();
    const uint32_t sc_ring = (p.zp != nullptr) ? kNS / 2 : kNS;   // scale stages in the ring (see epilogue_group)
    SchedT<CG> sched;
    TileInfo ti;
    uint32_t it = 0, flush = 0;
    bool ok = true;
    while (ok && sched.template next<BN>(p, ti)) {
      for (int g = ti.g0; g < ti.g1; ++g, ++it) {
        const bool first = per_group_flush || g == ti.g0;
        const bool last = per_group_flush || g == ti.g1 - 1;
        const uint32_t buf = flush % C::NT;
        const uint32_t s = it % C::NI, ph = (it / C::NI) & 1u;
        const uint32_t b_tm = bar_tm_empty + buf * 8, p_tm = ((flush / C::NT) & 1u) ^ 1u;
        // Per-group scales: this thread also waits for the group's scale stage (in a CTA pair: both CTAs' stages), so
        // that "group done" vouches for the scales and the epilogue warps -- the busy ones in that mode -- wait once.
        const bool need_sc = p.epi_mode == EPI_GROUP;
        const uint32_t sc_slot = flush % sc_ring, p_sc = (flush / sc_ring) & 1u;
        const uint32_t b_sc = bar_sc_full + sc_slot * 8, b_pe = bar_sc_peer + sc_slot * 8;
        // all probes back to back -- their latencies overlap -- and the one-at-a-time waits only if something is missing
        bool ready = mbar_test_wait(bar_i8_full + s * 8, ph);
        if (first) ready &= mbar_test_wait(b_tm, p_tm);
        if (need_sc) ready &= mbar_test_wait(b_sc, p_sc);
        if (need_sc && CG == 2) ready &= mbar_test_wait(b_pe, p_sc);
        if (!ready) {
          if (first) {
            ok = wait_bar_thread(b_tm, p_tm, abort_flag);
            if (!ok) break;
          }
          ok = wait_bar_thread(bar_i8_full + s * 8, ph, abort_flag);
          if (!ok) break;
          if (need_sc) {
            ok = wait_bar_thread(b_sc, p_sc, abort_flag);
            if (!ok) break;
            if (CG == 2) {
              ok = wait_bar_thread(b_pe, p_sc, abort_flag);
              if (!ok) break;
            }
          }
        }
        tc_fence_after_sync();
        {
          const uint32_t aP = sbase + C::OFF_I8 + s * (C::I8_P + C::I8_Q);
          const uint32_t aQ = aP + C::I8_P;
          const uint64_t dP = make_desc(aP), dQ = make_desc(aQ);
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 32 bytes of K per MMA: advance the start-address field by 32 >> 4
            if (CG == 2) mma_i8_cg2(d_tmem, dP + (uint64_t)(2 * k), dQ + (uint64_t)(2 * k), idesc, (first && k == 0) ? 0u : 1u);
            else mma_i8(d_tmem, dP + (uint64_t)(2 * k), dQ + (uint64_t)(2 * k), idesc, (first && k == 0) ? 0u : 1u);
          }
          // "stage free" for the converters; with a flush per group the same arrival is the epilogue's "accumulator
          // full".  In a CTA pair one commit arrives on the barrier at this offset in both CTAs.
          if (CG == 2) {
            tc_commit_cg2_both(bar_i8_empty + s * 8, (uint16_t)3);
            if (last && !per_group_flush) tc_commit_cg2_both(bar_tm_full + buf * 8, (uint16_t)3);
          } else {
            tc_commit(bar_i8_empty + s * 8);
            if (last && !per_group_flush) tc_commit(bar_tm_full + buf * 8);
          }
        }
        if (last) ++flush;
      }
    }
    } else if (!leader && CG == 2 && p.epi_mode == EPI_GROUP) {
      // second CTA of a pair: this warp has no MMAs to issue; it tells the leader when a scale stage of this
      // CTA has landed, so that the leader's "group done" vouches for both CTAs' scales
      const uint32_t arr_sc_peer = mapa_shared(bar_sc_peer, 0);
      const uint32_t sc_ring = (p.zp != nullptr) ? kNS / 2 : kNS;
      SchedT<CG> sched;
      TileInfo ti;
      uint32_t it = 0;
      bool ok = true;
      while (ok && sched.template next<BN>(p, ti)) {
        for (int g = ti.g0; g < ti.g1; ++g, ++it) {
          ok = wait_bar(bar_sc_full + (it % sc_ring) * 8, (it / sc_ring) & 1u, abort_flag);
          if (!ok) break;
          if (lane == 0) mbar_arrive_cluster(arr_sc_peer + (it % sc_ring) * 8);
          __syncwarp();
        }
      }
    }
    __syncwarp();   // the issuing thread rejoins its warp before the block-wide teardown
  } else if (p.epi_mode == EPI_GROUP) {
    // ---------------- scale loaders (warps 2 and 3 take alternate K groups) ----------------
    const uint32_t w = (uint32_t)(warp - kScaleWarp0);
    const bool azp = p.zp != nullptr;
    const uint32_t ns = azp ? kNS / 2 : kNS;                        // with zero-point vectors: two stages of double size
    const uint32_t stage_bytes = (azp ? 2u : 1u) * C::SCALE_STAGE;
    SchedT<CG> sched;
    TileInfo ti;
    uint32_t it = 0;
    bool ok = true;
    while (ok && sched.template next<BN>(p, ti)) {
      for (int g = ti.g0; g < ti.g1; ++g, ++it) {
        if ((it % kScaleWarps) != w) continue;
        const uint32_t ss = it % ns;
        ok = wait_bar(bar_sc_empty + ss * 8, ((it / ns) & 1u) ^ 1u, abort_flag);
        if (!ok) break;
        const uint32_t dst = sbase + C::OFF_SQ + ss * stage_bytes;
        const float* src_p = p.sp + (long long)g * p.sp_gstride;
        const float* src_zp = azp ? p.zp + (long long)g * p.sp_gstride : nullptr;
#pragma unroll
        for (int j = 0; j < kBM / 32; ++j) {
          const int row = ti.p0 + j * 32 + lane;
          const bool v = row < ti.p_lim;
          cp_async_4_zfill(dst + (uint32_t)(j * 32 + lane) * 4u, v ? src_p + row : p.sp, v);
          if (azp) cp_async_4_zfill(dst + (uint32_t)(kBM + BN + j * 32 + lane) * 4u, v ? src_zp + row : p.sp, v);
        }
        const float* src_q = p.sq + ti.sq_off + (long long)g * p.sq_gstride;
        const float* src_zq = azp ? p.zq + (long long)g * p.sq_gstride : nullptr;
#pragma unroll
        for (int j = 0; j < BN / 32; ++j) {
          const int q = ti.q0 + j * 32 + lane;
          const bool v = q < ti.q_lim;
          cp_async_4_zfill(dst + (uint32_t)(kBM + j * 32 + lane) * 4u, v ? src_q + q : p.sq, v);
          if (azp) cp_async_4_zfill(dst + (uint32_t)(2 * kBM + BN + j * 32 + lane) * 4u, v ? src_zq + q : p.sq, v);
        }
        cp_async_mbar_arrive_noinc(bar_sc_full + ss * 8);   // fires when this lane's copies have landed
      }
    }
    cp_async_wait_all();   // nothing of this warp is in flight into shared memory at teardown
  }
  } else if (warp < kConvWarp0 + kConvWarps) {
    // ---------------- converters ----------------
    setmaxnreg_dec<R::CONV>();
    const int tid = threadIdx.x - kConvWarp0 * 32;
    SchedT<CG> sched;
    TileInfo ti;
    uint32_t it = 0;
    bool ok = true;
    if (p.i8_operands) {
      // nothing to convert: these warps only pass "tile landed" on to the MMA thread (in a CTA pair: the leader's)
      while (ok && sched.template next<BN>(p, ti)) {
        for (int g = ti.g0; g < ti.g1; ++g, ++it) {
          const uint32_t si = it % C::NI, phi = (it / C::NI) & 1u;
          ok = wait_bar(bar_pk_full + si * 8, phi, abort_flag);
          if (!ok) break;
          if (lane == 0) arrive_bar<CG>(arr_i8_full + si * 8);
        }
      }
    } else
    while (ok && sched.template next<BN>(p, ti)) {
      for (int g = ti.g0; g < ti.g1; ++g, ++it) {
        const uint32_t sp_ = it % C::NP, php = (it / C::NP) & 1u;
        const uint32_t si = it % C::NI, phi = (it / C::NI) & 1u;
        // both probes in flight together (their latencies overlap); one-at-a-time waits only if something is missing
        const bool ready = mbar_test_wait(bar_pk_full + sp_ * 8, php) & mbar_test_wait(bar_i8_empty + si * 8, phi ^ 1u);
        if (!__all_sync(0xffffffffu, ready)) {
          ok = wait_bar(bar_pk_full + sp_ * 8, php, abort_flag);
          if (!ok) break;
          ok = wait_bar(bar_i8_empty + si * 8, phi ^ 1u, abort_flag);
          if (!ok) break;
        }
        const uint32_t pkP = sbase + C::OFF_PK + sp_ * (C::PK_P + C::PK_Q);
        const uint32_t i8P = sbase + C::OFF_I8 + si * (C::I8_P + C::I8_Q);
        convert_stage<kBM, C::QR>(pkP, i8P, pkP + C::PK_P, i8P + C::I8_P, tid);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          arrive_bar<CG>(arr_i8_full + si * 8);
          mbar_arrive(bar_pk_empty + sp_ * 8);
        }
      }
    }
  } else {
    // ---------------- epilogue ----------------
    setmaxnreg_inc<R::EPI>();
    if (p.epi_mode == EPI_GROUP) {
      if (p.zp != nullptr) {
        if (p.swap) epilogue_group<BN, __nv_bfloat16, true, CG, EW, true>(p, smem, tmem_base, bar_i8_empty, arr_tm_empty, bar_sc_full, bar_sc_empty, abort_flag);
        else epilogue_group<BN, __nv_bfloat16, false, CG, EW, true>(p, smem, tmem_base, bar_i8_empty, arr_tm_empty, bar_sc_full, bar_sc_empty, abort_flag);
      } else {
        if (p.swap) epilogue_group<BN, __nv_bfloat16, true, CG, EW, false>(p, smem, tmem_base, bar_i8_empty, arr_tm_empty, bar_sc_full, bar_sc_empty, abort_flag);
        else epilogue_group<BN, __nv_bfloat16, false, CG, EW, false>(p, smem, tmem_base, bar_i8_empty, arr_tm_empty, bar_sc_full, bar_sc_empty, abort_flag);
      }
    } else if (p.epi_mode == EPI_CHANNEL) {
      if (p.out_dtype == I4TC_FP16) {
        if (p.i8_operands) {
          if (p.swap) epilogue_channel<BN, __half, true, CG, EW, false>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
          else epilogue_channel<BN, __half, false, CG, EW, false>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
        } else {
          if (p.swap) epilogue_channel<BN, __half, true, CG, EW, true>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
          else epilogue_channel<BN, __half, false, CG, EW, true>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
        }
      } else {
        if (p.i8_operands) {
          if (p.swap) epilogue_channel<BN, __nv_bfloat16, true, CG, EW, false>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
          else epilogue_channel<BN, __nv_bfloat16, false, CG, EW, false>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
        } else {
          if (p.swap) epilogue_channel<BN, __nv_bfloat16, true, CG, EW, true>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
          else epilogue_channel<BN, __nv_bfloat16, false, CG, EW, true>(p, smem, tmem_base, bar_tm_full, arr_tm_empty, abort_flag);
        }
      }
    } else {
      epilogue_int32<BN, EW>(p, tmem_base, bar_tm_full, bar_i8_empty, bar_tm_empty, abort_flag);   // CG = 1 only
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  if (CG == 2) cluster_sync();   // neither CTA leaves while the other may still read its shared memory or arrive on its barriers
  else __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) {
    if (CG == 2) tmem_dealloc_cg2(tmem_base, C::TMEM_COLS);
    else tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.status, 1u);
}

template <int BN, int CG, int EW>
static int launch_bn(const GemmParams& p, const CUtensorMap& tmP, const CUtensorMap& tmQ, int grid, cudaStream_t st) {
  using C = Cfg<BN, CG, EW>;
  static_assert(C::SMEM_BYTES <= 232448, "shared memory layout exceeds the 227 KB a CTA may use");
  static bool configured[64] = {false};
  int dev = 0;
  I4TC_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    I4TC_CUDA(cudaFuncSetAttribute(w4a4_gemm_kernel<BN, CG, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    configured[dev] = true;
  }
  if (CG == 1) {
    w4a4_gemm_kernel<BN, CG, EW><<<grid, C::THREADS, C::SMEM_BYTES, st>>>(p, tmP, tmQ);
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(C::THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    I4TC_CUDA(cudaLaunchKernelEx(&cfg, w4a4_gemm_kernel<BN, CG, EW>, p, tmP, tmQ));
  }
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

__global__ void __launch_bounds__(256) split_reduce_kernel(const float* __restrict__ ws, long long stride, int splits,
                                                          long long n, __nv_bfloat16* __restrict__ out) {
  const long long i = ((long long)blockIdx.x * 256 + threadIdx.x) * 4;
  // 16-byte loads need every range to start on a 16-byte boundary, the 8-byte store an 8-byte aligned output
  const bool vec = ((stride & 3) == 0) && ((reinterpret_cast<uintptr_t>(ws) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(out) & 7) == 0);
  if (vec && i + 3 < n) {
    float4 acc = *reinterpret_cast<const float4*>(ws + i);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(ws + (long long)s * stride + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    union { __nv_bfloat16 h[4]; uint2 u; } pk;
    pk.h[0] = __float2bfloat16_rn(acc.x); pk.h[1] = __float2bfloat16_rn(acc.y);
    pk.h[2] = __float2bfloat16_rn(acc.z); pk.h[3] = __float2bfloat16_rn(acc.w);
    *reinterpret_cast<uint2*>(out + i) = pk.u;
  } else {
    for (long long j = i; j < n && j < i + 4; ++j) {
      float acc = ws[j];
      for (int s = 1; s < splits; ++s) acc += ws[(long long)s * stride + j];
      out[j] = __float2bfloat16_rn(acc);
    }
  }
}

// Per-channel variant: the ranges hold exact integer sums; out[m, n] = cast((sum * scale_b[n]) * scale_a[m]).
template <typename OutT>
__global__ void __launch_bounds__(256) split_reduce_scaled_kernel(const float* __restrict__ ws, long long stride, int splits,
                                                                 long long M, long long N, const float* __restrict__ sa,
                                                                 const float* __restrict__ sb, OutT* __restrict__ out) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= M * N) return;
  float acc = ws[i];
  for (int s = 1; s < splits; ++s) acc += ws[(long long)s * stride + i];
  const long long m = i / N, n = i - m * N;
  out[i] = cast_out<OutT>((acc * __ldg(sb + n)) * __ldg(sa + m));
}

int launch_split_reduce_scaled(const float* ws, long long stride, int splits, long long M, long long N, const float* sa,
                               const float* sb, void* out, int out_dtype, cudaStream_t st) {
  const long long blocks = (M * N + 255) / 256;
  if (out_dtype == I4TC_FP16)
    split_reduce_scaled_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(ws, stride, splits, M, N, sa, sb, static_cast<__half*>(out));
  else
    split_reduce_scaled_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(ws, stride, splits, M, N, sa, sb,
                                                                                static_cast<__nv_bfloat16*>(out));
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

int launch_split_reduce(const float* ws, long long stride, int splits, long long n, void* out, cudaStream_t st) {
  const long long blocks = (n + 1023) / 1024;
  split_reduce_kernel<<<(unsigned)blocks, 256, 0, st>>>(ws, stride, splits, n, static_cast<__nv_bfloat16*>(out));
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

int launch_w4a4_gemm(const GemmParams& p, const CUtensorMap& tmP, const CUtensorMap& tmQ, int bn, int grid,
                     bool cta_pair, int epi_warps, cudaStream_t st) {
  const bool wide = epi_warps == 16 && bn >= 128;   // 64-column tiles have only 8 x 32 columns to hand out
  if (cta_pair) {
    I4TC_REQUIRE((bn == 256 || bn == 192) && (grid % 2) == 0 && p.expert_offsets == nullptr && !p.swap && p.splits == 1 &&
                     (p.epi_mode == EPI_CHANNEL || p.epi_mode == EPI_GROUP),
                 I4TC_EINVAL, "CTA-pair launch needs a dense, unswapped 192- or 256-wide problem and an even grid");
    // 192-column tiles: three epilogue warps per scheduler, 64 running sums per thread
    if (bn == 192) return launch_bn<192, 2, 12>(p, tmP, tmQ, grid, st);
    return wide ? launch_bn<256, 2, 16>(p, tmP, tmQ, grid, st) : launch_bn<256, 2, 8>(p, tmP, tmQ, grid, st);
  }
  switch (bn) {
    case 64: return launch_bn<64, 1, 8>(p, tmP, tmQ, grid, st);
    case 128: return wide ? launch_bn<128, 1, 16>(p, tmP, tmQ, grid, st) : launch_bn<128, 1, 8>(p, tmP, tmQ, grid, st);
    case 256: return wide ? launch_bn<256, 1, 16>(p, tmP, tmQ, grid, st) : launch_bn<256, 1, 8>(p, tmP, tmQ, grid, st);
    default: return fail(I4TC_EINVAL, "unsupported tile width %d", bn);
  }
}

}  // namespace i4tc
