// MoE support kernels: device-side stable counting sort of (token, slot) pairs by expert, and the
// weighted combine of expert outputs.  The reference has no MoE path; these feed the grouped-tile
// W4A4 GEMM, which walks the sorted rows expert by expert.
//
// Sort = three small launches over chunks of 1024 pairs:
//   1. per-chunk histogram                    -> scratch counts [chunks, E]
//   2. scan over chunks and experts           -> scratch bases  [chunks, E], expert_offsets [E+1]
//   3. stable rank inside the chunk + scatter -> sorted_pairs, inv_pairs
// The scratch ([chunks, E] int32) is caller-provided global memory.
#include "common.cuh"
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

int moe_sort_launch(const int32_t* ids, int64_t P, int64_t E, int32_t* sorted_pairs, int32_t* inv_pairs,
                    int32_t* expert_offsets, int32_t* scratch, cudaStream_t st) {
  const int chunks = (int)((P + kSortChunk - 1) / kSortChunk);
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
