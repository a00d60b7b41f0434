// MoE support kernels: device-side stable counting sort of (token, slot) pairs by expert, and the
// weighted combine of expert outputs.  The reference has no MoE path; these feed the grouped-tile
// W4A4 GEMM, which walks the sorted rows expert by expert.
//
// Up to one chunk per SM the three steps below run as ONE cooperative launch (a grid-wide barrier between counting
// and placing: every block is resident by construction of a cooperative launch); larger inputs use three launches:
//   1. per-chunk histogram                    -> scratch counts [chunks, E]
//   2. scan over chunks and experts           -> scratch bases  [chunks, E], expert_offsets [E+1]
//   3. stable rank inside the chunk + scatter -> sorted_pairs, inv_pairs
// The scratch ([chunks, E] int32) is caller-provided global memory.
#include "common.cuh"
#include <cooperative_groups.h>
#include <mutex>

namespace i4tc {

constexpr int kSortChunk = 1024;
constexpr int kMaxExperts = 256;

// Stable rank of every element of a 1024-pair chunk among equal expert ids.
// On return: rank (this thread's rank inside the chunk among its expert), and s_cnt[32][E] holds, per
// warp, the exclusive prefix over earlier warps; total[e] (threads < E) is the chunk's count for e.
__device__ __forceinline__ void chunk_rank(int e, bool valid, int E, int (*s_cnt)[kMaxExperts], int& rank,
                                           int& total_for_thread_expert) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * kMaxExperts; i += kSortChunk) (&s_cnt[0][0])[i] = 0;
  __syncthreads();
  const int key = valid ? e : -1 - lane;  // invalid lanes match nobody
  const unsigned mask = __match_any_sync(0xffffffffu, key);
  const int rank_w = __popc(mask & ((1u << lane) - 1u));
  if (valid && rank_w == 0) s_cnt[warp][e] = __popc(mask);
  __syncthreads();
  total_for_thread_expert = 0;
  if ((int)threadIdx.x < E) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = s_cnt[w][threadIdx.x];
      s_cnt[w][threadIdx.x] = run;
      run += c;
    }
    total_for_thread_expert = run;
  }
  __syncthreads();
  rank = valid ? s_cnt[warp][e] + rank_w : 0;
}

__global__ void __launch_bounds__(kSortChunk) moe_hist_kernel(const int32_t* __restrict__ ids, int P, int E,
                                                             int32_t* __restrict__ counts) {
  __shared__ int s_cnt[32][kMaxExperts];
  const int i = blockIdx.x * kSortChunk + threadIdx.x;
  const bool in = i < P;
  const int e = in ? ids[i] : 0;
  const bool valid = in && e >= 0 && e < E;
  int rank, total;
  chunk_rank(e, valid, E, s_cnt, rank, total);
  if ((int)threadIdx.x < E) counts[(long long)blockIdx.x * E + threadIdx.x] = total;
}

// One block of kMaxExperts threads, thread e = expert e.  Two passes over the [chunks, E] histogram, each with eight
// independent loads in flight (a load-add-store chain per chunk would pay a trip to L2 per chunk): totals per
// expert, an exclusive scan of the totals across experts (warp shuffles), then the running bases of every chunk.
// Pairs whose id lies outside [0, E) are left out of the sort; the tail of sorted_pairs that they would have
// filled is set to -1 here, so that no later kernel reads an uninitialised pair index.
__global__ void __launch_bounds__(kMaxExperts) moe_scan_kernel(int32_t* __restrict__ counts, int chunks, int E,
                                                              int32_t* __restrict__ expert_offsets,
                                                              int32_t* __restrict__ sorted_pairs, int P) {
  __shared__ int s_warp[kMaxExperts / 32];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  const bool ok = e < E;
  int total = 0;
  if (ok) {
    for (int c0 = 0; c0 < chunks; c0 += 8) {
      int v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (c0 + j < chunks) ? counts[(long long)(c0 + j) * E + e] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) total += v[j];
    }
  }
  // exclusive scan of `total` over the experts
  int incl = total;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int warp_base = 0;
#pragma unroll
  for (int w = 0; w < kMaxExperts / 32; ++w) warp_base += (w < warp) ? s_warp[w] : 0;
  const int off = warp_base + incl - total;
  if (ok) {
    expert_offsets[e] = off;
    if (e == E - 1) {
      expert_offsets[E] = off + total;
      s_warp[0] = off + total;   // read below, after the barrier (s_warp is no longer needed for the scan)
    }
    int run = off;
    for (int c0 = 0; c0 < chunks; c0 += 8) {
      int v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (c0 + j < chunks) ? counts[(long long)(c0 + j) * E + e] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (c0 + j < chunks) counts[(long long)(c0 + j) * E + e] = run;
        run += v[j];
      }
    }
  }
  __syncthreads();
  for (int i = s_warp[0] + threadIdx.x; i < P; i += kMaxExperts) sorted_pairs[i] = -1;
}

__global__ void __launch_bounds__(kSortChunk) moe_scatter_kernel(const int32_t* __restrict__ ids, int P, int E,
                                                                const int32_t* __restrict__ bases,
                                                                int32_t* __restrict__ sorted_pairs,
                                                                int32_t* __restrict__ inv_pairs) {
  __shared__ int s_cnt[32][kMaxExperts];
  const int i = blockIdx.x * kSortChunk + threadIdx.x;
  const bool in = i < P;
  const int e = in ? ids[i] : 0;
  const bool valid = in && e >= 0 && e < E;
  int rank, total;
  chunk_rank(e, valid, E, s_cnt, rank, total);
  if (valid) {
    const int pos = bases[(long long)blockIdx.x * E + e] + rank;
    sorted_pairs[pos] = i;
    if (inv_pairs) inv_pairs[i] = pos;
  } else if (in && inv_pairs) {
    inv_pairs[i] = -1;
  }
}

// The whole sort in one cooperative launch (chunks <= co-resident blocks): count, grid barrier, then every block forms
// the expert offsets and its own bases from the [chunks, E] histogram and places its pairs.  Same outputs as the
// three-launch form, including the -1 tail of sorted_pairs.
__global__ void __launch_bounds__(kSortChunk) moe_sort_fused_kernel(const int32_t* __restrict__ ids, int P, int E,
                                                                   int32_t* __restrict__ counts,
                                                                   int32_t* __restrict__ expert_offsets,
                                                                   int32_t* __restrict__ sorted_pairs,
                                                                   int32_t* __restrict__ inv_pairs) {
  __shared__ int s_cnt[32][kMaxExperts];
  __shared__ int s_base[kMaxExperts];
  __shared__ int s_warp[kMaxExperts / 32];
  __shared__ int s_total;
  const int chunks = gridDim.x;
  const int i = blockIdx.x * kSortChunk + threadIdx.x;
  const bool in = i < P;
  const int e = in ? ids[i] : 0;
  const bool valid = in && e >= 0 && e < E;
  int rank, total;
  chunk_rank(e, valid, E, s_cnt, rank, total);
  if ((int)threadIdx.x < E) counts[(long long)blockIdx.x * E + threadIdx.x] = total;
  __threadfence();
  cooperative_groups::this_grid().sync();
  const int t = threadIdx.x;
  if (t < kMaxExperts) {
    int tot = 0, before = 0;
    if (t < E) {
      for (int c0 = 0; c0 < chunks; c0 += 8) {
        int v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (c0 + j < chunks) ? __ldcg(counts + (long long)(c0 + j) * E + t) : 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          tot += v[j];
          if (c0 + j < (int)blockIdx.x) before += v[j];
        }
      }
    }
    const int lane = t & 31, warp = t >> 5;
    int incl = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += u;
    }
    if (lane == 31) s_warp[warp] = incl;
    // the first kMaxExperts threads are whole warps, so the block barrier below is reached by everyone
    s_base[t] = incl - tot + before;   // completed after the barrier with the totals of the earlier warps
  }
  __syncthreads();
  if (t < kMaxExperts) {
    const int warp = t >> 5;
    int warp_base = 0;
#pragma unroll
    for (int w = 0; w < kMaxExperts / 32; ++w) warp_base += (w < warp) ? s_warp[w] : 0;
    const int off = s_base[t] - 0 + warp_base;   // expert offset + rows of earlier chunks
    s_base[t] = off;
    if (blockIdx.x == 0 && t < E) {
      expert_offsets[t] = off;   // block 0 has no earlier chunks: its bases are the offsets themselves
    }
    if (t == kMaxExperts - 1) {
      int all = 0;
#pragma unroll
      for (int w = 0; w < kMaxExperts / 32; ++w) all += s_warp[w];
      s_total = all;
      if (blockIdx.x == 0) expert_offsets[E] = all;
    }
  }
  __syncthreads();
  if (valid) {
    const int pos = s_base[e] + rank;
    sorted_pairs[pos] = i;
    if (inv_pairs) inv_pairs[i] = pos;
  } else if (in && inv_pairs) {
    inv_pairs[i] = -1;
  }
  // the tail that left-out pairs would have filled
  for (int j = s_total + blockIdx.x * kSortChunk + threadIdx.x; j < P; j += chunks * kSortChunk) sorted_pairs[j] = -1;
}

// out[t, :] = bf16( sum_j w[t, j] * y[inv[t*k + j], :] ), fp32 accumulation in ascending j, one fused multiply-add
// per term.
__global__ void __launch_bounds__(256) moe_combine_kernel(const __nv_bfloat16* __restrict__ y,
                                                         const int32_t* __restrict__ inv,
                                                         const float* __restrict__ w, int top_k, int H,
                                                         __nv_bfloat16* __restrict__ out) {
  const long long t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += 256 * 8) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const int row = __ldg(inv + t * top_k + j);
      if (row < 0) continue;
      const float wj = __ldg(w + t * top_k + j);
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(y + (long long)row * H + c));
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] = __fmaf_rn(wj, __uint_as_float(ww[i] << 16), acc[2 * i]);
        acc[2 * i + 1] = __fmaf_rn(wj, __uint_as_float(ww[i] & 0xFFFF0000u), acc[2 * i + 1]);
      }
    }
    union { __nv_bfloat16 h[8]; uint4 u; } pk;
#pragma unroll
    for (int i = 0; i < 8; ++i) pk.h[i] = __float2bfloat16_rn(acc[i]);
    *reinterpret_cast<uint4*>(out + t * H + c) = pk.u;
  }
}

// ------------------------------------------------------------------------------------------
// Expert parallelism with fixed-capacity exchange buffers (no host synchronisation).
//
// A rank sorts its (token, slot) pairs by global expert id; sorted by expert is sorted by owner rank.  For every
// destination rank d it fills a block of the send buffer: one header row, then up to `cap` quantised token rows
// (G x 64 bytes of codes followed by G fp32 group scales) in sorted order.  Header (int32): [0] rows in the block,
// [1] sorted position of the block's first row at the source, [2 .. 2 + e_loc) rows per local expert of d.
// Blocks have a fixed size, so the all-to-all needs no split sizes from the device.  A destination that would get
// more than `cap` rows raises the overflow flag (the counts are clipped so that every index stays in range); the
// caller then repeats the step with exact split sizes.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_ep_plan_kernel(const int32_t* __restrict__ expert_offsets,
                                                         const int32_t* __restrict__ sorted_pairs, int P, int world,
                                                         int e_loc, int cap, long long row_bytes,
                                                         uint8_t* __restrict__ send_buf, int32_t* __restrict__ slot,
                                                         int32_t* __restrict__ ret_row, unsigned int* overflow,
                                                         const unsigned long long* __restrict__ peer_bases, int my_rank) {
  if (blockIdx.x == 0) {
    // headers: thread (d, e) pairs in a strided loop; with peer destinations the header of destination d is written
    // straight into block `my_rank` of d's receive buffer
    for (int i = threadIdx.x; i < world * (e_loc + 2); i += blockDim.x) {
      const int d = i / (e_loc + 2), f = i - d * (e_loc + 2);
      const int start = expert_offsets[d * e_loc];
      int32_t* hdr = (peer_bases != nullptr)
                         ? reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(peer_bases[d]) +
                                                      (long long)my_rank * (1 + cap) * row_bytes)
                         : reinterpret_cast<int32_t*>(send_buf + (long long)d * (1 + cap) * row_bytes);
      if (f == 0) {
        const int n = expert_offsets[(d + 1) * e_loc] - start;
        hdr[0] = min(n, cap);
        if (n > cap) atomicOr(overflow, 1u);
      } else if (f == 1) {
        hdr[1] = start;
      } else {
        const int e = d * e_loc + (f - 2);
        const int a = min(expert_offsets[e] - start, cap), b = min(expert_offsets[e + 1] - start, cap);
        hdr[f] = b - a;
      }
    }
  }
  const int total = expert_offsets[world * e_loc];
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < P; p += gridDim.x * blockDim.x) {
    int s = -1;
    if (p < total) {
      int d = 0;
      while (d + 1 < world && p >= expert_offsets[(d + 1) * e_loc]) ++d;
      const int j = p - expert_offsets[d * e_loc];
      if (j < cap) {
        s = d * (1 + cap) + 1 + j;
        ret_row[sorted_pairs[p]] = d * cap + j;
      }
    }
    slot[p] = s;
  }
}

// Receiver, step 1 (one block): read the `world` headers, build the local expert offsets and, per (source, expert),
// where that run of rows starts in expert-sorted order and where it starts inside the source's block.
// meta layout (int32): tot[world] | base[world][e_loc] | cum[world][e_loc + 1] | start[world] (sorted position, at the
// source, of the first row of its block).
__global__ void __launch_bounds__(256) moe_ep_offsets_kernel(const uint8_t* __restrict__ recv_buf, int world, int e_loc,
                                                            int cap, long long row_bytes,
                                                            int32_t* __restrict__ expert_offsets_loc,
                                                            int32_t* __restrict__ meta, int32_t* __restrict__ rows_dev) {
  __shared__ int s_off[kMaxExperts + 1];
  int32_t* tot = meta;
  int32_t* base = meta + world;
  int32_t* cum = base + world * e_loc;
  const int e = threadIdx.x;
  int mine = 0;
  if (e < e_loc)
    for (int s = 0; s < world; ++s)
      mine += reinterpret_cast<const int32_t*>(recv_buf + (long long)s * (1 + cap) * row_bytes)[2 + e];
  if (e < kMaxExperts) s_off[e + 1] = (e < e_loc) ? mine : 0;
  if (e == 0) s_off[0] = 0;
  __syncthreads();
  if (e == 0) {
    for (int i = 1; i <= e_loc; ++i) s_off[i] += s_off[i - 1];
    *rows_dev = s_off[e_loc];
  }
  __syncthreads();
  if (e <= e_loc) expert_offsets_loc[e] = s_off[e];
  if (e < e_loc) {
    int run = s_off[e];
    for (int s = 0; s < world; ++s) {
      base[s * e_loc + e] = run;
      run += reinterpret_cast<const int32_t*>(recv_buf + (long long)s * (1 + cap) * row_bytes)[2 + e];
    }
  }
  if (e < world) {
    const int32_t* hdr = reinterpret_cast<const int32_t*>(recv_buf + (long long)e * (1 + cap) * row_bytes);
    int run = 0;
    for (int i = 0; i < e_loc; ++i) {
      cum[e * (e_loc + 1) + i] = run;
      run += hdr[2 + i];
    }
    cum[e * (e_loc + 1) + e_loc] = run;
    tot[e] = min(min(hdr[0], run), cap);
    cum[world * (e_loc + 1) + e] = hdr[1];   // start[e]
  }
}

// Receiver, step 2: one warp per received row (source s, index j): find its local expert, hence its position in
// expert-sorted order, and move codes and scales into the group-major layout the grouped GEMM reads.
__global__ void __launch_bounds__(256) moe_ep_scatter_kernel(const uint8_t* __restrict__ recv_buf, int world, int e_loc,
                                                            int cap, long long row_bytes, int G, long long r_max,
                                                            const int32_t* __restrict__ meta,
                                                            uint8_t* __restrict__ ap, float* __restrict__ asc,
                                                            int32_t* __restrict__ pos_of) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + warp;
  if (row >= (long long)world * cap) return;
  const int s = (int)(row / cap), j = (int)(row - (long long)s * cap);
  const int32_t* tot = meta;
  const int32_t* base = meta + world;
  const int32_t* cum = base + world * e_loc + s * (e_loc + 1);
  if (j >= tot[s]) {
    if (lane == 0) pos_of[row] = -1;
    return;
  }
  int lo = 0, hi = e_loc - 1;   // last expert whose run starts at or before j
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cum[mid] <= j) lo = mid; else hi = mid - 1;
  }
  const long long pos = base[s * e_loc + lo] + (j - cum[lo]);
  const uint8_t* src = recv_buf + ((long long)s * (1 + cap) + 1 + j) * row_bytes;
  for (int c = lane; c < G * 4; c += 32) {     // 16-byte chunks of the codes: group c / 4, quarter c % 4
    const uint4 v = *reinterpret_cast<const uint4*>(src + (long long)c * 16);
    *reinterpret_cast<uint4*>(ap + ((long long)(c >> 2) * r_max + pos) * 64 + (c & 3) * 16) = v;
  }
  const float* ssrc = reinterpret_cast<const float*>(src + (long long)G * 64);
  for (int g = lane; g < G; g += 32) asc[(long long)g * r_max + pos] = ssrc[g];
  if (lane == 0) pos_of[row] = (int32_t)pos;
}

// Expert outputs back into the order each source sent its rows in: ret_send[s][j] = y[pos_of[s][j]].  With peer
// destinations row (s, j) goes straight to row start[s] + j of source s's return buffer (its own sorted order).
__global__ void __launch_bounds__(256) moe_ep_pack_return_kernel(const __nv_bfloat16* __restrict__ y,
                                                                const int32_t* __restrict__ pos_of, long long rows,
                                                                int H, __nv_bfloat16* __restrict__ ret_send,
                                                                const unsigned long long* __restrict__ peer_bases,
                                                                const int32_t* __restrict__ start, int cap, int world,
                                                                int rot) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long row = (long long)blockIdx.x * 8 + warp;
  if (row >= rows) return;
  if (peer_bases != nullptr) {
    // Neighbouring warps write to different ranks, and rank r starts its round with rank r + 1: otherwise every rank
    // would send its block for rank 0 first, then the one for rank 1, ... and one receiver at a time would take all
    // the senders' traffic while the other links sit idle.
    const int s = (int)((row + rot) % world);
    row = (long long)s * cap + row / world;
  }
  const int pos = pos_of[row];
  if (pos < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(y + (long long)pos * H);
  uint4* dst = reinterpret_cast<uint4*>(ret_send + row * H);
  if (peer_bases != nullptr) {
    const int s = (int)(row / cap), j = (int)(row - (long long)s * cap);
    dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_bases[s]) + ((long long)start[s] + j) * H);
  }
  // four 16-byte loads in flight per lane before the (possibly remote) stores
  const int n = H / 8;
  for (int c0 = 0; c0 < n; c0 += 128) {
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = c0 + i * 32 + lane;
      if (c < n) v[i] = __ldg(src + c);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = c0 + i * 32 + lane;
      if (c < n) dst[c] = v[i];
    }
  }
}

// Where the expert output of every expert-sorted row has to go when it is written straight into the sources' return
// buffers: out_rows[pos_of[s][j]] = address of row start[s] + j of source s's buffer (H 16-bit values per row).
__global__ void moe_ep_return_rows_kernel(const int32_t* __restrict__ pos_of, long long rows, int H,
                                          const unsigned long long* __restrict__ peer_bases,
                                          const int32_t* __restrict__ start, int cap,
                                          unsigned long long* __restrict__ out_rows) {
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  const int pos = pos_of[row];
  if (pos < 0) return;
  const int s = (int)(row / cap), j = (int)(row - (long long)s * cap);
  out_rows[pos] = peer_bases[s] + ((unsigned long long)(start[s] + j)) * (unsigned long long)H * 2ull;
}

// Rows that were quantised once per token, copied to where each (token, slot) pair needs them.  One warp per output
// row r: source token = pairs[r] / top_k (nothing is copied for a negative or out-of-range pair index, or beyond
// *rows_dev).  Source layout: group-major [G, T, 64] codes and [G, T] scales.  Destination: group-major [G, R, 64] / [G, R]
// (row_map == nullptr), or rows of G x 64 code bytes followed by G scales (row_bytes = 68 G) at row row_map[r] of a
// block buffer -- a local one, or with peer_bases the block `my_block` of the buffer of the rank that owns block
// row_map[r] / block_rows (plain stores over NVLink).
__global__ void __launch_bounds__(256) moe_gather_packed_kernel(const uint8_t* __restrict__ src_codes,
                                                               const float* __restrict__ src_scale, long long T, int G,
                                                               const int32_t* __restrict__ pairs, int top_k, long long R,
                                                               uint8_t* __restrict__ dst_codes, float* __restrict__ dst_scale,
                                                               const int32_t* __restrict__ row_map, long long row_bytes,
                                                               const unsigned long long* __restrict__ peer_bases,
                                                               int block_rows, int my_block) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long r = (long long)blockIdx.x * 8 + warp;
  if (peer_bases != nullptr) {
    // rows are sorted by destination rank: walk eight evenly spaced stretches of them at once (warp w of a block takes
    // stretch w, first stretch rotated by the rank), so that a rank writes to all its peers at the same time instead
    // of every rank flooding rank 0 first
    const long long per = (R + 7) / 8;
    const long long i = r / 8;
    r = (long long)((warp + my_block) & 7) * per + i;
    if (i >= per) return;
  }
  if (r >= R) return;
  const int pair = pairs[r];
  if (pair < 0) return;
  const long long t = pair / top_k;
  if (t >= T) return;
  if (row_map == nullptr) {
    for (int c = lane; c < G * 4; c += 32) {
      const int g = c >> 2, q = c & 3;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(src_codes + ((long long)g * T + t) * 64 + q * 16));
      *reinterpret_cast<uint4*>(dst_codes + ((long long)g * R + r) * 64 + q * 16) = v;
    }
    for (int g = lane; g < G; g += 32) dst_scale[(long long)g * R + r] = __ldg(src_scale + (long long)g * T + t);
    return;
  }
  const long long m = row_map[r];
  if (m < 0) return;
  uint8_t* row;
  if (peer_bases != nullptr) {
    const long long blk = m / block_rows;
    row = reinterpret_cast<uint8_t*>(peer_bases[blk]) + ((long long)my_block * block_rows + (m - blk * block_rows)) * row_bytes;
  } else {
    row = dst_codes + m * row_bytes;
  }
  for (int c = lane; c < G * 4; c += 32) {
    const int g = c >> 2, q = c & 3;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(src_codes + ((long long)g * T + t) * 64 + q * 16));
    *reinterpret_cast<uint4*>(row + (long long)c * 16) = v;
  }
  float* srow = reinterpret_cast<float*>(row + (long long)G * 64);
  for (int g = lane; g < G; g += 32) srow[g] = __ldg(src_scale + (long long)g * T + t);
}

// Cross-GPU completion flags.  A rank that has finished writing into its peers' buffers (all earlier work of its
// stream) stores a growing epoch number into its slot of every peer's flag array; a rank that is about to read its
// own buffer waits until every slot has reached the epoch.  The wait is bounded: after two seconds it sets bit 1 of
// the status word and lets the stream go on.
// `counter` (optional): the epoch lives in device memory, so that a captured graph of a layer advances it on every
// replay.  The dispatch signal of a layer bumps it; everything else in the layer reads it.
__global__ void peer_signal_kernel(const unsigned long long* __restrict__ flag_addrs, int world, unsigned int epoch,
                                   unsigned int* counter, int bump) {
  __shared__ unsigned int s_epoch;
  if (threadIdx.x == 0) {
    unsigned int e = epoch;
    if (counter != nullptr) {
      e = *counter + (bump ? 1u : 0u);
      if (bump) *counter = e;
    }
    s_epoch = e;
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world) {
    volatile unsigned int* f = reinterpret_cast<volatile unsigned int*>(flag_addrs[threadIdx.x]);
    *f = s_epoch;
  }
  __threadfence_system();
}

__global__ void peer_wait_kernel(const unsigned int* __restrict__ flags, int world, unsigned int epoch,
                                 const unsigned int* counter, unsigned int* status) {
  if (counter != nullptr) epoch = *counter;
  if ((int)threadIdx.x < world) {
    const volatile unsigned int* f = flags + threadIdx.x;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    unsigned int spins = 0;
    while ((int)(*f - epoch) < 0) {
      if ((++spins & 255u) == 0) {
        unsigned long long t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) {
          atomicOr(status, 2u);
          break;
        }
      }
    }
  }
  __threadfence_system();
}

int moe_sort_launch(const int32_t* ids, int64_t P, int64_t E, int32_t* sorted_pairs, int32_t* inv_pairs,
                    int32_t* expert_offsets, int32_t* scratch, cudaStream_t st) {
  const int chunks = (int)((P + kSortChunk - 1) / kSortChunk);
  int dev = 0, sms = 0, coop = 0;
  I4TC_CUDA(cudaGetDevice(&dev));
  I4TC_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  I4TC_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
  if (coop && chunks <= sms) {
    int Pi = (int)P, Ei = (int)E;
    void* args[] = {(void*)&ids, (void*)&Pi, (void*)&Ei, (void*)&scratch, (void*)&expert_offsets, (void*)&sorted_pairs,
                    (void*)&inv_pairs};
    const cudaError_t e = cudaLaunchCooperativeKernel((const void*)moe_sort_fused_kernel, dim3(chunks), dim3(kSortChunk), args,
                                                      0, st);
    if (e == cudaSuccess) return I4TC_OK;
    cudaGetLastError();   // not launchable as one cooperative grid here (a partitioned GPU, for instance): three launches
  }
  moe_hist_kernel<<<chunks, kSortChunk, 0, st>>>(ids, (int)P, (int)E, scratch);
  moe_scan_kernel<<<1, kMaxExperts, 0, st>>>(scratch, chunks, (int)E, expert_offsets, sorted_pairs, (int)P);
  moe_scatter_kernel<<<chunks, kSortChunk, 0, st>>>(ids, (int)P, (int)E, scratch, sorted_pairs, inv_pairs);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

}  // namespace i4tc

using namespace i4tc;

extern "C" int64_t i4tc_moe_sort_scratch_bytes(int64_t num_pairs, int64_t num_experts) {
  if (num_pairs < 0 || num_experts <= 0) return 0;
  const int64_t chunks = (num_pairs + kSortChunk - 1) / kSortChunk;
  return (chunks > 0 ? chunks : 1) * num_experts * (int64_t)sizeof(int32_t);
}

extern "C" int i4tc_moe_sort(const int32_t* expert_ids, int64_t num_pairs, int64_t num_experts,
                             int32_t* sorted_pairs, int32_t* inv_pairs, int32_t* expert_offsets, void* scratch,
                             int64_t scratch_bytes, int device, void* stream) {
  I4TC_REQUIRE(num_pairs >= 0 && num_pairs < (1ll << 31), I4TC_EINVAL, "num_pairs out of range");
  I4TC_REQUIRE(num_experts > 0 && num_experts <= kMaxExperts, I4TC_EINVAL, "num_experts must be in [1, %d]",
               kMaxExperts);
  I4TC_REQUIRE(expert_offsets != nullptr, I4TC_EINVAL, "null expert_offsets");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (num_pairs == 0) {
    I4TC_CUDA(cudaMemsetAsync(expert_offsets, 0, (num_experts + 1) * sizeof(int32_t), st));
    return I4TC_OK;
  }
  I4TC_REQUIRE(expert_ids && sorted_pairs && scratch, I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(scratch_bytes >= i4tc_moe_sort_scratch_bytes(num_pairs, num_experts), I4TC_EINVAL,
               "scratch too small: need %lld bytes", (long long)i4tc_moe_sort_scratch_bytes(num_pairs, num_experts));
  return moe_sort_launch(expert_ids, num_pairs, num_experts, sorted_pairs, inv_pairs, expert_offsets,
                         static_cast<int32_t*>(scratch), st);
}

// ------------------------------------------------------------------------------------------
// Sort variant that allocates nothing.
//
// Some callers cannot obtain device memory at call time: a serving engine that handed every free
// byte of HBM to its own cache pool at start-up (a later cudaMalloc fails), or a latency-critical
// loop that must not pay for cudaMalloc / cudaFree, which synchronise the whole device.  For them
// the per-chunk histogram scratch of the sort lives in this fixed array instead of a caller buffer.
// Every GPU that loads the library holds the 64 KiB until the process exits.
//
// In host code `g_sort_scratch` is only a host-side stand-in for the symbol, never a device
// address: the address is resolved once per device with cudaGetSymbolAddress (below) and that
// pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------
constexpr int kNoAllocScratchInts = 16384;  // ceil(num_pairs / 1024) * num_experts must not exceed this
static __device__ __align__(256) int32_t g_sort_scratch[kNoAllocScratchInts];

static int32_t* g_sort_scratch_ptr[64] = {nullptr};
static std::mutex g_sort_scratch_mutex;

// Resolves the device address of g_sort_scratch for `device` (which must be current).  The first
// resolution on a device also makes the CUDA runtime load this module there (with lazy module loading
// that is when the driver sets aside the array and the kernels' code), which is why callers that will
// have no free device memory later do it at start-up through i4tc_moe_sort_noalloc_prepare.
static int sort_scratch_for(int device, int32_t** out) {
  I4TC_REQUIRE(device >= 0 && device < 64, I4TC_EINVAL, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_sort_scratch_mutex);
  if (g_sort_scratch_ptr[device] == nullptr) {
    int32_t* ptr = nullptr;
    I4TC_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_sort_scratch));
    I4TC_REQUIRE(ptr != nullptr, I4TC_EDEVICE, "could not resolve the device address of the sort scratch");
    g_sort_scratch_ptr[device] = ptr;
  }
  *out = g_sort_scratch_ptr[device];
  return I4TC_OK;
}

extern "C" int64_t i4tc_moe_sort_noalloc_max_scratch_ints(void) { return kNoAllocScratchInts; }

extern "C" int i4tc_moe_sort_noalloc_prepare(int device) {
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  int32_t* scratch = nullptr;
  if (int rc = sort_scratch_for(device, &scratch)) return rc;
  // ask for the kernels' attributes so that their code is resident too (nothing is launched)
  cudaFuncAttributes attr;
  I4TC_CUDA(cudaFuncGetAttributes(&attr, moe_hist_kernel));
  I4TC_CUDA(cudaFuncGetAttributes(&attr, moe_scan_kernel));
  I4TC_CUDA(cudaFuncGetAttributes(&attr, moe_scatter_kernel));
  I4TC_CUDA(cudaFuncGetAttributes(&attr, moe_sort_fused_kernel));
  return I4TC_OK;
}

extern "C" int i4tc_moe_sort_noalloc(const int32_t* expert_ids, int64_t num_pairs, int64_t num_experts,
                                     int32_t* sorted_pairs, int32_t* inv_pairs, int32_t* expert_offsets,
                                     int device, void* stream) {
  I4TC_REQUIRE(num_pairs >= 0 && num_pairs < (1ll << 31), I4TC_EINVAL, "num_pairs out of range");
  I4TC_REQUIRE(num_experts > 0 && num_experts <= kMaxExperts, I4TC_EINVAL, "num_experts must be in [1, %d]",
               kMaxExperts);
  const int64_t chunks = (num_pairs + kSortChunk - 1) / kSortChunk;
  I4TC_REQUIRE(chunks * num_experts <= kNoAllocScratchInts, I4TC_EINVAL,
               "i4tc_moe_sort_noalloc: ceil(num_pairs/1024) * num_experts = %lld exceeds the built-in scratch of "
               "%d entries; use i4tc_moe_sort with a caller-provided scratch buffer",
               (long long)(chunks * num_experts), kNoAllocScratchInts);
  I4TC_REQUIRE(expert_offsets != nullptr, I4TC_EINVAL, "null expert_offsets");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t* scratch = nullptr;
  if (int rc = sort_scratch_for(device, &scratch)) return rc;   // also on an empty call, so that one can serve as a warm-up
  if (num_pairs == 0) {
    I4TC_CUDA(cudaMemsetAsync(expert_offsets, 0, (num_experts + 1) * sizeof(int32_t), st));
    return I4TC_OK;
  }
  I4TC_REQUIRE(expert_ids && sorted_pairs, I4TC_EINVAL, "null pointer");
  // Nothing in the scratch has to start at zero: the histogram pass writes every entry that the
  // scan and scatter passes of this call read, so the previous call's contents are never seen.
  return moe_sort_launch(expert_ids, num_pairs, num_experts, sorted_pairs, inv_pairs, expert_offsets, scratch, st);
}

extern "C" int i4tc_moe_gather_packed(const uint8_t* tok_packed, const float* tok_scale, int64_t num_tokens,
                                      int64_t num_groups, const int32_t* pairs, int64_t num_pairs, int64_t top_k,
                                      uint8_t* packed, float* scale, const int32_t* row_map, int64_t row_bytes,
                                      const uint64_t* peer_bases, int64_t cap, int64_t my_rank, int device,
                                      void* stream) {
  I4TC_REQUIRE(num_tokens >= 0 && num_pairs >= 0 && num_groups > 0 && top_k > 0 && top_k < (1 << 20), I4TC_EINVAL, "bad sizes");
  if (num_pairs == 0 || num_tokens == 0) return I4TC_OK;
  I4TC_REQUIRE(tok_packed && tok_scale && pairs, I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(aligned_to(tok_packed, 16), I4TC_EALIGN, "packed rows must be 16-byte aligned");
  if (row_map == nullptr) {
    I4TC_REQUIRE(packed && scale && aligned_to(packed, 16), I4TC_EINVAL, "group-major destination missing or misaligned");
  } else {
    I4TC_REQUIRE(row_bytes == num_groups * 68, I4TC_EINVAL, "a buffer row is 64 bytes of codes and one fp32 scale per group");
    I4TC_REQUIRE((packed && aligned_to(packed, 16)) || peer_bases, I4TC_EINVAL, "buffer destination missing or misaligned");
    I4TC_REQUIRE(peer_bases == nullptr || (cap > 0 && my_rank >= 0), I4TC_EINVAL, "peer destinations need cap and the rank");
  }
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  // (with peer destinations a block's eight warps take one row of each of eight stretches of ceil(num_pairs / 8) rows)
  const long long launch_rows = peer_bases ? ((num_pairs + 7) / 8) * 8 : num_pairs;
  moe_gather_packed_kernel<<<(unsigned)((launch_rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      tok_packed, tok_scale, num_tokens, (int)num_groups, pairs, (int)top_k, num_pairs, packed, scale, row_map, row_bytes,
      reinterpret_cast<const unsigned long long*>(peer_bases), (int)(1 + cap), (int)my_rank);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_moe_ep_plan(const int32_t* expert_offsets, const int32_t* sorted_pairs, int64_t num_pairs,
                                int64_t num_experts, int64_t world, int64_t cap, int64_t row_bytes, void* send_buf,
                                int32_t* slot, int32_t* ret_row, unsigned int* overflow, const uint64_t* peer_bases,
                                int64_t my_rank, int device, void* stream) {
  I4TC_REQUIRE(world > 0 && num_experts > 0 && num_experts % world == 0 && num_experts <= kMaxExperts, I4TC_EINVAL,
               "experts must divide evenly across ranks (at most %d experts)", kMaxExperts);
  I4TC_REQUIRE(cap > 0 && cap < (1 << 24) && num_pairs >= 0 && num_pairs < (1ll << 31), I4TC_EINVAL, "bad capacity or size");
  const int64_t e_loc = num_experts / world;
  I4TC_REQUIRE(row_bytes % 16 == 0 && row_bytes >= 4 * (2 + e_loc), I4TC_EINVAL,
               "a buffer row must be a multiple of 16 bytes and hold the %lld header integers", (long long)(2 + e_loc));
  I4TC_REQUIRE(expert_offsets && (send_buf || peer_bases) && slot && ret_row && overflow &&
                   (sorted_pairs || num_pairs == 0), I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(my_rank >= 0 && my_rank < world, I4TC_EINVAL, "rank out of range");
  I4TC_REQUIRE(aligned_to(send_buf, 16), I4TC_EALIGN, "send buffer must be 16-byte aligned");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // pairs the sort left out (ids outside [0, E)) and pairs beyond the capacity have no row on the way back
  if (num_pairs > 0) I4TC_CUDA(cudaMemsetAsync(ret_row, 0xFF, num_pairs * sizeof(int32_t), st));
  int64_t blocks = (num_pairs + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 1024) blocks = 1024;
  moe_ep_plan_kernel<<<(unsigned)blocks, 256, 0, st>>>(expert_offsets, sorted_pairs, (int)num_pairs, (int)world, (int)e_loc,
                                                       (int)cap, row_bytes, static_cast<uint8_t*>(send_buf), slot, ret_row,
                                                       overflow, reinterpret_cast<const unsigned long long*>(peer_bases),
                                                       (int)my_rank);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int64_t i4tc_moe_ep_meta_ints(int64_t world, int64_t e_loc) {
  return world + world * e_loc + world * (e_loc + 1) + world;
}

extern "C" int i4tc_moe_ep_unpack(const void* recv_buf, int64_t world, int64_t e_loc, int64_t cap, int64_t row_bytes,
                                  int64_t num_groups, uint8_t* a_packed, float* a_scale, int32_t* expert_offsets_loc,
                                  int32_t* pos_of, int32_t* meta, int32_t* rows_dev, int device, void* stream) {
  I4TC_REQUIRE(world > 0 && world <= 256 && e_loc > 0 && e_loc <= kMaxExperts && cap > 0 && num_groups > 0, I4TC_EINVAL, "bad sizes");
  I4TC_REQUIRE(row_bytes == num_groups * 68, I4TC_EINVAL, "a row is 64 bytes of codes and one fp32 scale per group");
  I4TC_REQUIRE(recv_buf && a_packed && a_scale && expert_offsets_loc && pos_of && meta && rows_dev, I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(aligned_to(recv_buf, 16) && aligned_to(a_packed, 16), I4TC_EALIGN, "buffers must be 16-byte aligned");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* rb = static_cast<const uint8_t*>(recv_buf);
  moe_ep_offsets_kernel<<<1, 256, 0, st>>>(rb, (int)world, (int)e_loc, (int)cap, row_bytes, expert_offsets_loc, meta, rows_dev);
  const long long rows = world * cap;
  moe_ep_scatter_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(rb, (int)world, (int)e_loc, (int)cap, row_bytes,
                                                                  (int)num_groups, rows, meta, a_packed, a_scale, pos_of);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_moe_ep_pack_return(const void* y, const int32_t* pos_of, int64_t rows, int64_t H, void* ret_send,
                                       const uint64_t* peer_bases, const int32_t* meta, int64_t world, int64_t e_loc,
                                       int64_t cap, int device, void* stream) {
  I4TC_REQUIRE(rows >= 0 && H > 0 && H % 8 == 0, I4TC_EINVAL, "H must be a positive multiple of 8");
  if (rows == 0) return I4TC_OK;
  I4TC_REQUIRE(y && pos_of && (ret_send || peer_bases), I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(aligned_to(y, 16) && aligned_to(ret_send, 16), I4TC_EALIGN, "buffers must be 16-byte aligned");
  I4TC_REQUIRE(peer_bases == nullptr || (meta && world > 0 && e_loc > 0 && cap > 0 && rows == world * cap), I4TC_EINVAL,
               "peer destinations need the unpack scratch and the block geometry");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  const int32_t* start = peer_bases ? meta + world + world * e_loc + world * (e_loc + 1) : nullptr;
  moe_ep_pack_return_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), pos_of, rows, (int)H, static_cast<__nv_bfloat16*>(ret_send),
      reinterpret_cast<const unsigned long long*>(peer_bases), start, (int)(cap > 0 ? cap : 1),
      (int)(world > 0 ? world : 1), peer_bases ? device + 1 : 0);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_moe_ep_return_rows(const int32_t* pos_of, int64_t rows, int64_t H, const uint64_t* peer_bases,
                                       const int32_t* meta, int64_t world, int64_t e_loc, int64_t cap,
                                       uint64_t* out_rows, int device, void* stream) {
  I4TC_REQUIRE(rows >= 0 && H > 0 && H % 8 == 0, I4TC_EINVAL, "H must be a positive multiple of 8");
  if (rows == 0) return I4TC_OK;
  I4TC_REQUIRE(pos_of && peer_bases && meta && out_rows, I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(world > 0 && e_loc > 0 && cap > 0 && rows == world * cap, I4TC_EINVAL, "rows must be world * cap");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  const int32_t* start = meta + world + world * e_loc + world * (e_loc + 1);
  moe_ep_return_rows_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pos_of, rows, (int)H, reinterpret_cast<const unsigned long long*>(peer_bases), start, (int)cap,
      reinterpret_cast<unsigned long long*>(out_rows));
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_peer_signal(const uint64_t* flag_addrs, int64_t world, uint32_t epoch, int device, void* stream) {
  I4TC_REQUIRE(flag_addrs && world > 0 && world <= 256, I4TC_EINVAL, "bad arguments");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  peer_signal_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const unsigned long long*>(flag_addrs), (int)world, epoch, nullptr, 0);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_peer_signal_counter(const uint64_t* flag_addrs, int64_t world, uint32_t* counter, int bump,
                                        int device, void* stream) {
  I4TC_REQUIRE(flag_addrs && counter && world > 0 && world <= 256, I4TC_EINVAL, "bad arguments");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  peer_signal_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const unsigned long long*>(flag_addrs), (int)world, 0u, counter, bump);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_peer_wait_counter(const uint32_t* flags, int64_t world, const uint32_t* counter, int device,
                                      void* stream) {
  I4TC_REQUIRE(flags && counter && world > 0 && world <= 256, I4TC_EINVAL, "bad arguments");
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  peer_wait_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(flags, (int)world, 0u, counter, info->status);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_peer_wait(const uint32_t* flags, int64_t world, uint32_t epoch, int device, void* stream) {
  I4TC_REQUIRE(flags && world > 0 && world <= 256, I4TC_EINVAL, "bad arguments");
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  peer_wait_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(flags, (int)world, epoch, nullptr, info->status);
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}

extern "C" int i4tc_moe_combine(const void* y, const int32_t* inv_pairs, const float* w, int64_t T, int64_t top_k,
                                int64_t H, void* out, int device, void* stream) {
  I4TC_REQUIRE(T >= 0 && top_k > 0 && H >= 0, I4TC_EINVAL, "bad sizes");
  I4TC_REQUIRE(H % 8 == 0, I4TC_EINVAL, "H must be a multiple of 8");
  I4TC_REQUIRE(T < (1ll << 31), I4TC_EINVAL, "too many tokens");
  if (T == 0 || H == 0) return I4TC_OK;
  I4TC_REQUIRE(y && inv_pairs && w && out, I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(aligned_to(y, 16) && aligned_to(out, 16), I4TC_EALIGN, "y and out must be 16-byte aligned");
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  moe_combine_kernel<<<(unsigned)T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), inv_pairs, w, (int)top_k, (int)H, static_cast<__nv_bfloat16*>(out));
  I4TC_CUDA(cudaGetLastError());
  return I4TC_OK;
}
