// Host side of the dense and MoE W4A4 GEMM entry points: argument checks, tensor maps,
// tile-shape choice and launch.
#include "gemm.cuh"
#include <stdlib.h>
#include <atomic>

namespace i4tc {

// Process-wide tuning hooks.  Atomics: a host thread may change one while another thread launches (each launch
// reads every hook once, at its start).
static std::atomic<int> g_force_bn{0};      // 0 = choose automatically
static std::atomic<int> g_force_swap{-1};   // -1 = choose automatically
static std::atomic<int> g_small_m_path{0};  // 0 = automatic, 1 = CUDA-core kernel only, 2 = register-fed tensor-core kernel whenever it applies, 3 = tile kernel only
static std::atomic<int> g_force_splits{0};  // 0 = choose automatically, 1 = never split, n = n K ranges
static std::atomic<int> g_cta_pairs{-1};    // -1 = choose automatically, 0 = never, 1 = whenever the problem allows it
static std::atomic<bool> g_pairs_launchable{true};   // cleared when an automatic cluster launch was refused
static std::atomic<int> g_epi_warps{0};     // 0 = choose automatically, 8 or 16

static int epi_warps_for(int epi_mode) {
  if (const int w = g_epi_warps.load()) return w;
  (void)epi_mode;
  return 8;
}

struct Shape {
  int bn;
  bool swap;
  bool pair;   // 256-row tiles on pairs of SMs (bn 256 or 192)
};

// Picks the tile width, the operand orientation and whether pairs of SMs share 256-row tiles.  Up to 64 tokens the
// weights go on the 128-row side of the MMA (so that no tensor-core rows are wasted on padding and more CTAs stream
// weights); otherwise the candidate with the fewest cost-weighted waves wins.  Weights = measured time per output
// column relative to 256-wide pair tiles at M = 8192 (per-group | per-channel epilogue): 192-wide pair tiles 1.10 | 1.30,
// 256-wide single tiles 1.05 | 1.20, 128-wide single tiles 1.25 | 1.45.
static Shape choose_shape(long long M, long long N, int sms, bool allow_swap, bool group_mode, bool pairs_allowed) {
  Shape s;
  s.pair = false;
  s.swap = allow_swap && M <= 64;
  if (const int fs = g_force_swap.load(); fs >= 0 && allow_swap) s.swap = fs != 0;
  const int force_pairs = g_cta_pairs.load();
  if (const int fb = g_force_bn.load()) {
    s.bn = fb;
    // a forced width keeps the old rule for pairs: at least 512 rows and pair tiles that fill the machine about as
    // well as single tiles would
    if (!s.swap && pairs_allowed && (fb == 256 || fb == 192)) {
      const long long t1 = ((M + 127) / 128) * ((N + fb - 1) / fb), t2 = ((M + 255) / 256) * ((N + fb - 1) / fb);
      const int pairs = sms / 2;
      const double eff1 = (double)t1 / (double)(((t1 + sms - 1) / sms) * sms);
      const double eff2 = pairs > 0 ? (double)t2 / (double)(((t2 + pairs - 1) / pairs) * pairs) : 0.0;
      s.pair = (M >= 512 && eff2 >= 0.9 * eff1 && force_pairs != 0) || force_pairs == 1 || fb == 192;
    }
    return s;
  }
  if (s.swap) {
    s.bn = M <= 64 ? 64 : 128;
    return s;
  }
  if (M <= 128) {
    // one row of tiles and K split into ranges: measured, 128-wide tiles win for the 4096..6144-row weight
    // matrices (more work items), 256-wide ones for the 24576-row one (fewer MMA issues per weight byte)
    s.bn = N >= 16384 ? 256 : 128;
    return s;
  }
  struct Cand { int bn; bool pair; double w_group, w_channel; };
  const Cand cands[4] = {{256, true, 1.00, 1.00}, {192, true, 1.10, 1.30}, {256, false, 1.05, 1.20}, {128, false, 1.25, 1.45}};
  double best = 1e30;
  s.bn = 256;
  for (const Cand& c : cands) {
    if (c.pair && (!pairs_allowed || M < 512 || sms < 2 || force_pairs == 0)) continue;
    if (!c.pair && force_pairs == 1 && pairs_allowed) continue;
    const long long rows = c.pair ? (M + 255) / 256 : (M + 127) / 128;
    const long long units = c.pair ? sms / 2 : sms;
    const long long tiles = rows * ((N + c.bn - 1) / c.bn);
    const long long waves = (tiles + units - 1) / units;
    const double cost = (double)waves * c.bn * (group_mode ? c.w_group : c.w_channel);
    if (cost < best) {
      best = cost;
      s.bn = c.bn;
      s.pair = c.pair;
    }
  }
  return s;
}

struct DenseArgs {
  const uint8_t* a;
  const uint8_t* b;
  const float* sa;
  const float* sb;
  void* out;
  int out_dtype;
  long long M, N;
  int G;
  bool rowmajor;    // operands are [rows, K/2] (else group-major [G, rows, 64])
  long long K;      // only for rowmajor
  int epi_mode;
  // zero-point term (per-group mode only): group g adds azp_adj[g, m] * w_col_sum[g, n] to its integer sum
  const float* azp_adj = nullptr;
  const float* w_col_sum = nullptr;
  bool i8_operands = false;   // a and b are int8 [rows, K] (W4A8): no conversion, accumulator unit 1
};

static int run_dense(const DenseArgs& d, int device, void* stream) {
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  I4TC_REQUIRE(info->cc_major == 10, I4TC_EDEVICE, "device %d is sm_%d%d; this library needs sm_100", device,
               info->cc_major, info->cc_minor);
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  I4TC_REQUIRE(d.M < (1ll << 31) - 256 && d.N < (1ll << 31) - 256, I4TC_EINVAL, "M or N too large");

  // a few dozen tokens: stream the weights (unless a test pins the tile shape)
  if (g_force_bn == 0 && g_force_swap < 0 && g_force_splits == 0 && d.azp_adj == nullptr && !d.i8_operands &&
      (!d.rowmajor || d.K == (long long)d.G * 128)) {
    const int path = g_small_m_path.load();
    const long long K = (long long)d.G * 128;
    const bool gemv_ok = path != 3 && path != 2 && gemv_applicable(d.M, d.N, K, d.epi_mode);
    const bool skinny_ok = path != 3 && path != 1 && skinny_applicable(d.M, d.N, K, d.epi_mode, d.rowmajor, info->sm_count);
    // one or two tokens: dp4a on the CUDA cores does not waste tensor-core columns; from three on the tensor cores win
    if (skinny_ok && (path == 2 || !gemv_ok || d.M > 2))
      return launch_w4a4_skinny(d.a, d.b, d.sa, d.sb, d.out, d.out_dtype, d.M, d.N, d.G, d.rowmajor, d.epi_mode,
                                info->sm_count, info->status, static_cast<cudaStream_t>(stream));
    if (gemv_ok)
      return launch_w4a4_gemv(d.a, d.b, d.sa, d.sb, d.out, d.out_dtype, d.M, d.N, d.G, d.rowmajor, d.epi_mode,
                              info->sm_count, static_cast<cudaStream_t>(stream));
  }

  const bool group_mode = d.epi_mode == EPI_GROUP || d.epi_mode == EPI_GROUP_INT32;
  const bool pairs_allowed = (d.epi_mode == EPI_CHANNEL || d.epi_mode == EPI_GROUP) && g_pairs_launchable.load();
  Shape sh = choose_shape(d.M, d.N, info->sm_count, true, group_mode, pairs_allowed);
  I4TC_REQUIRE(sh.bn != 192 || sh.pair, I4TC_EINVAL, "192-wide tiles need a dense problem with scaled outputs (SM pairs)");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.G = d.G;
  p.swap = sh.swap ? 1 : 0;
  p.i8_operands = d.i8_operands ? 1 : 0;
  p.acc_unit = d.i8_operands ? 1.0f : 1.0f / 256.0f;
  p.epi_mode = d.epi_mode;
  p.out_dtype = d.out_dtype;
  p.out = d.out;
  p.ldc = d.N;
  p.out_gstride = d.M * d.N;
  p.status = info->status;
  p.p_rowmajor = p.q_rowmajor = d.rowmajor ? 1 : 0;
  const bool per_group_scales = d.epi_mode == EPI_GROUP;
  const uint8_t *pbase, *qbase;
  long long prow, qrow;
  if (!sh.swap) {
    pbase = d.a; qbase = d.b; prow = d.M; qrow = d.N;
    p.sp = d.sa; p.sq = d.sb;
    p.zp = d.azp_adj; p.zq = d.w_col_sum;
    p.sp_gstride = per_group_scales ? d.M : 0;
    p.sq_gstride = per_group_scales ? d.N : 0;
  } else {
    pbase = d.b; qbase = d.a; prow = d.N; qrow = d.M;
    p.sp = d.sb; p.sq = d.sa;
    p.zp = d.w_col_sum; p.zq = d.azp_adj;
    p.sp_gstride = per_group_scales ? d.N : 0;
    p.sq_gstride = per_group_scales ? d.M : 0;
  }
  p.P_rows = (int)prow;
  p.Q_rows = (int)qrow;
  p.num_p_tiles = (int)((prow + 127) / 128);
  p.num_q_tiles = (int)((qrow + sh.bn - 1) / sh.bn);
  const long long tiles = (long long)p.num_p_tiles * p.num_q_tiles;
  I4TC_REQUIRE(tiles < (1ll << 31), I4TC_EINVAL, "too many tiles");
  // Split-K for the weight-streaming case (small M, scaled outputs): a tile's K loop is a serial
  // chain of per-group handshakes, so when there are fewer tiles than SMs -- or an awkward number
  // of waves -- the groups are cut into ranges handled by different CTAs and the partial sums are
  // added afterwards in a fixed order: fp32 for per-group scales (deterministic), exact integers held
  // in fp32 for per-channel scales (bit-identical to the unsplit result).
  p.splits = 1;
  p.groups_per_split = d.G;
  // (int8 operands: sums of a K range can exceed 2^24, so they are never parked in fp32)
  if ((d.epi_mode == EPI_GROUP || d.epi_mode == EPI_CHANNEL) && d.M <= 128 && g_force_splits != 1 && !d.i8_operands) {
    // cost in microseconds: waves x groups per range x ~0.65 us per group handshake, plus writing and
    // reading the fp32 partial sums at ~6 TB/s and one more launch
    int best_s = 1;
    double best_cost = (double)((tiles + info->sm_count - 1) / info->sm_count) * d.G * 0.65;
    for (int s = 2; s <= 8 && s <= d.G; ++s) {
      const long long gps = (d.G + s - 1) / s;
      const double traffic_us = 2.0 * s * (double)d.M * (double)d.N * 4.0 / 6.0e6;
      const double cost = (double)((tiles * s + info->sm_count - 1) / info->sm_count) * gps * 0.65 + traffic_us + 3.0;
      if (cost < best_cost) { best_cost = cost; best_s = s; }
    }
    if (const int fs = g_force_splits.load(); fs > 1) best_s = fs <= d.G ? fs : d.G;
    if (best_s > 1) {
      p.splits = best_s;
      p.groups_per_split = (d.G + best_s - 1) / best_s;
      p.splits = (d.G + p.groups_per_split - 1) / p.groups_per_split;  // no empty range
      p.ws_stride = (d.M * d.N + 3) & ~3ll;   // every range starts on a 16-byte boundary
      float* ws = nullptr;
      if (int rc = split_workspace(device, static_cast<cudaStream_t>(stream), (size_t)p.splits * p.ws_stride * sizeof(float), &ws)) return rc;
      p.split_ws = ws;
    }
  }

  // CTA pairs (256-row tiles on two SMs): each SM converts and stages a third less per unit of MMA work
  // (measured at M = 8192: +18-21 % with the one-flush per-channel epilogue, +4-5 % with the per-group one).
  bool pair = sh.pair && !sh.swap && p.splits == 1 && info->sm_count >= 2;
  const int clusters_max = info->sm_count / 2;
  const long long pair_tiles = ((prow + 255) / 256) * p.num_q_tiles;
  CUtensorMap tmP, tmQ;
  const long long extent = d.rowmajor ? d.K / 2 : (long long)d.G;
  auto operand_map = [&](const uint8_t* base, long long rows, int box_rows, CUtensorMap* out) -> int {
    if (d.i8_operands) return get_tensor_map_i8(device, base, rows, d.K, box_rows, out);
    return get_tensor_map(device, base, d.rowmajor, rows, extent, box_rows, out);
  };
  if (int rc = operand_map(pbase, prow, 128, &tmP)) return rc;
  if (pair) {
    if (int rc = operand_map(qbase, qrow, sh.bn / 2, &tmQ)) return rc;   // each CTA of a pair stages half of the Q tile
    GemmParams pp = p;
    pp.num_p_tiles = (int)((prow + 255) / 256);
    const int grid = 2 * (int)(pair_tiles < clusters_max ? pair_tiles : clusters_max);
    const int rc = launch_w4a4_gemm(pp, tmP, tmQ, sh.bn, grid, true, epi_warps_for(d.epi_mode), static_cast<cudaStream_t>(stream));
    if (rc == I4TC_OK) return I4TC_OK;
    if (g_cta_pairs == 1) return rc;   // the caller asked for pairs: report why they cannot run
    // an environment that cannot launch clusters of two (a restricted SM partition, for instance): the launch
    // was refused before anything ran; remember it and use single thread blocks from now on
    cudaGetLastError();
    g_pairs_launchable = false;
    if (sh.bn == 192) {   // that width exists on pairs only: fall back to 256-wide single tiles
      sh.bn = 256;
      p.num_q_tiles = (int)((qrow + sh.bn - 1) / sh.bn);
    }
  }
  if (int rc = operand_map(qbase, qrow, sh.bn, &tmQ)) return rc;
  const long long items = (long long)p.num_p_tiles * p.num_q_tiles * p.splits;
  const int grid = (int)(items < info->sm_count ? items : info->sm_count);
  if (int rc = launch_w4a4_gemm(p, tmP, tmQ, sh.bn, grid, false, epi_warps_for(d.epi_mode), static_cast<cudaStream_t>(stream))) return rc;
  if (p.splits > 1) {
    if (d.epi_mode == EPI_CHANNEL)
      return launch_split_reduce_scaled(p.split_ws, p.ws_stride, p.splits, d.M, d.N, d.sa, d.sb, d.out, d.out_dtype,
                                        static_cast<cudaStream_t>(stream));
    return launch_split_reduce(p.split_ws, p.ws_stride, p.splits, d.M * d.N, d.out, static_cast<cudaStream_t>(stream));
  }
  return I4TC_OK;
}

static int check_dense_common(const void* a, const void* b, const void* out, long long M, long long N) {
  I4TC_REQUIRE(M >= 0 && N >= 0, I4TC_EINVAL, "negative size");
  if (M == 0 || N == 0) return 1;  // nothing to do
  I4TC_REQUIRE(a && b && out, I4TC_EINVAL, "null pointer");
  return I4TC_OK;
}

}  // namespace i4tc

using namespace i4tc;

extern "C" int i4tc_set_tuning(int tile_n, int swap) {
  I4TC_REQUIRE(tile_n == 0 || tile_n == 64 || tile_n == 128 || tile_n == 192 || tile_n == 256, I4TC_EINVAL,
               "tile_n must be 0 (automatic), 64, 128, 192 (SM pairs only) or 256");
  I4TC_REQUIRE(swap >= -1 && swap <= 1, I4TC_EINVAL, "swap must be -1 (automatic), 0 or 1");
  g_force_bn = tile_n;
  g_force_swap = swap;
  return I4TC_OK;
}

extern "C" int i4tc_set_split_k(int splits) {
  I4TC_REQUIRE(splits >= 0 && splits <= 8, I4TC_EINVAL, "splits must be 0 (automatic) or 1..8");
  g_force_splits = splits;
  return I4TC_OK;
}

extern "C" int i4tc_set_cta_pairs(int mode) {
  I4TC_REQUIRE(mode >= -1 && mode <= 1, I4TC_EINVAL, "mode must be -1 (automatic), 0 or 1");
  g_cta_pairs = mode;
  return I4TC_OK;
}

extern "C" int i4tc_set_small_m_path(int path) {
  I4TC_REQUIRE(path >= 0 && path <= 3, I4TC_EINVAL, "path must be 0 (automatic), 1, 2 or 3");
  g_small_m_path = path;
  return I4TC_OK;
}

extern "C" int i4tc_set_epilogue_warps(int warps) {
  I4TC_REQUIRE(warps == 0 || warps == 8 || warps == 16, I4TC_EINVAL, "warps must be 0 (automatic), 8 or 16");
  g_epi_warps = warps;
  return I4TC_OK;
}

extern "C" int i4tc_gemm_int32(const uint8_t* a, const uint8_t* b, int32_t* c, int64_t M, int64_t N, int64_t K,
                               int device, void* stream) {
  I4TC_REQUIRE(K > 0 && K % 64 == 0, I4TC_EINVAL, "K must be a positive multiple of 64");
  I4TC_REQUIRE(K <= 65536, I4TC_EINVAL, "K must not exceed 65536");
  int rc = check_dense_common(a, b, c, M, N);
  if (rc) return rc < 0 ? rc : I4TC_OK;
  DenseArgs d{a, b, nullptr, nullptr, c, I4TC_INT32, M, N, (int)((K + 127) / 128), true, K, EPI_INT32};
  return run_dense(d, device, stream);
}

extern "C" int i4tc_gemm_scaled(const uint8_t* a, const uint8_t* b, const float* scale_a, const float* scale_b,
                                void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int device,
                                void* stream) {
  I4TC_REQUIRE(K > 0 && K % 64 == 0, I4TC_EINVAL, "K must be a positive multiple of 64");
  I4TC_REQUIRE(K <= 65536, I4TC_EINVAL, "K must not exceed 65536");
  I4TC_REQUIRE(out_dtype == I4TC_BF16 || out_dtype == I4TC_FP16, I4TC_EUNSUPPORTED, "out must be bf16 or fp16");
  int rc = check_dense_common(a, b, out, M, N);
  if (rc) return rc < 0 ? rc : I4TC_OK;
  I4TC_REQUIRE(scale_a && scale_b, I4TC_EINVAL, "null scale pointer");
  DenseArgs d{a, b, scale_a, scale_b, out, out_dtype, M, N, (int)((K + 127) / 128), true, K, EPI_CHANNEL};
  return run_dense(d, device, stream);
}

extern "C" int i4tc_gemm_w4a8_scaled(const int8_t* a, const int8_t* b, const float* scale_a, const float* scale_b,
                                     void* out, int out_dtype, int64_t M, int64_t N, int64_t K, int device,
                                     void* stream) {
  I4TC_REQUIRE(K > 0 && K % 32 == 0, I4TC_EINVAL, "K must be multiple of 32 for INT8 alignment");
  I4TC_REQUIRE(K <= 65536, I4TC_EINVAL, "K must not exceed 65536");
  I4TC_REQUIRE(out_dtype == I4TC_BF16 || out_dtype == I4TC_FP16, I4TC_EUNSUPPORTED, "out must be bf16 or fp16");
  int rc = check_dense_common(a, b, out, M, N);
  if (rc) return rc < 0 ? rc : I4TC_OK;
  I4TC_REQUIRE(scale_a && scale_b, I4TC_EINVAL, "null scale pointer");
  DenseArgs d{reinterpret_cast<const uint8_t*>(a), reinterpret_cast<const uint8_t*>(b), scale_a, scale_b, out, out_dtype,
              M, N, (int)((K + 127) / 128), true, K, EPI_CHANNEL};
  d.i8_operands = true;
  return run_dense(d, device, stream);
}

extern "C" int i4tc_gemm_grouped(const uint8_t* a, const uint8_t* b, const float* scale_a, const float* scale_b,
                                 void* out, int64_t M, int64_t N, int64_t group_size, int64_t num_groups,
                                 int device, void* stream) {
  I4TC_REQUIRE(group_size == 128, I4TC_EUNSUPPORTED, "fused grouped GEMM only supports group_size=128");
  I4TC_REQUIRE(num_groups > 0 && num_groups <= 512, I4TC_EINVAL, "num_groups must be in [1, 512]");
  int rc = check_dense_common(a, b, out, M, N);
  if (rc) return rc < 0 ? rc : I4TC_OK;
  I4TC_REQUIRE(scale_a && scale_b, I4TC_EINVAL, "null scale pointer");
  DenseArgs d{a, b, scale_a, scale_b, out, I4TC_BF16, M, N, (int)num_groups, false, 0, EPI_GROUP};
  return run_dense(d, device, stream);
}

extern "C" int i4tc_gemm_grouped_azp(const uint8_t* a, const uint8_t* b, const float* scale_a, const float* scale_b,
                                     const float* azp_adj, const float* w_col_sum, void* out, int64_t M, int64_t N,
                                     int64_t group_size, int64_t num_groups, int device, void* stream) {
  I4TC_REQUIRE(group_size == 128, I4TC_EUNSUPPORTED, "fused grouped GEMM only supports group_size=128");
  I4TC_REQUIRE(num_groups > 0 && num_groups <= 512, I4TC_EINVAL, "num_groups must be in [1, 512]");
  int rc = check_dense_common(a, b, out, M, N);
  if (rc) return rc < 0 ? rc : I4TC_OK;
  I4TC_REQUIRE(scale_a && scale_b && azp_adj && w_col_sum, I4TC_EINVAL, "null scale, azp_adj or w_col_sum pointer");
  DenseArgs d{a, b, scale_a, scale_b, out, I4TC_BF16, M, N, (int)num_groups, false, 0, EPI_GROUP};
  d.azp_adj = azp_adj;
  d.w_col_sum = w_col_sum;
  return run_dense(d, device, stream);
}

extern "C" int i4tc_gemm_grouped_int32(const uint8_t* a, const uint8_t* b, int32_t* out, int64_t M, int64_t N,
                                       int64_t num_groups, int device, void* stream) {
  I4TC_REQUIRE(num_groups > 0 && num_groups <= 512, I4TC_EINVAL, "num_groups must be in [1, 512]");
  int rc = check_dense_common(a, b, out, M, N);
  if (rc) return rc < 0 ? rc : I4TC_OK;
  DenseArgs d{a, b, nullptr, nullptr, out, I4TC_INT32, M, N, (int)num_groups, false, 0, EPI_GROUP_INT32};
  return run_dense(d, device, stream);
}

static int moe_grouped_gemm_impl(const uint8_t* a, const float* scale_a, const uint8_t* b, const float* scale_b,
                                 const int32_t* expert_offsets, void* out, const uint64_t* out_rows, int64_t num_pairs,
                                 int64_t N, int64_t num_groups, int64_t num_experts, int device, void* stream);

extern "C" int i4tc_moe_grouped_gemm(const uint8_t* a, const float* scale_a, const uint8_t* b,
                                     const float* scale_b, const int32_t* expert_offsets, void* out,
                                     int64_t num_pairs, int64_t N, int64_t num_groups, int64_t num_experts,
                                     int device, void* stream) {
  I4TC_REQUIRE(out != nullptr || num_pairs == 0 || N == 0, I4TC_EINVAL, "null pointer");
  return moe_grouped_gemm_impl(a, scale_a, b, scale_b, expert_offsets, out, nullptr, num_pairs, N, num_groups, num_experts,
                               device, stream);
}

extern "C" int i4tc_moe_grouped_gemm_rows(const uint8_t* a, const float* scale_a, const uint8_t* b,
                                          const float* scale_b, const int32_t* expert_offsets,
                                          const uint64_t* out_rows, int64_t num_pairs, int64_t N, int64_t num_groups,
                                          int64_t num_experts, int device, void* stream) {
  I4TC_REQUIRE(out_rows != nullptr || num_pairs == 0 || N == 0, I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(N % 8 == 0, I4TC_EINVAL, "N must be a multiple of 8 when rows are addressed through a table");
  return moe_grouped_gemm_impl(a, scale_a, b, scale_b, expert_offsets, nullptr, out_rows, num_pairs, N, num_groups,
                               num_experts, device, stream);
}

static int moe_grouped_gemm_impl(const uint8_t* a, const float* scale_a, const uint8_t* b, const float* scale_b,
                                 const int32_t* expert_offsets, void* out, const uint64_t* out_rows, int64_t num_pairs,
                                 int64_t N, int64_t num_groups, int64_t num_experts, int device, void* stream) {
  I4TC_REQUIRE(num_pairs >= 0 && N >= 0, I4TC_EINVAL, "negative size");
  I4TC_REQUIRE(num_groups > 0 && num_groups <= 512, I4TC_EINVAL, "num_groups must be in [1, 512]");
  I4TC_REQUIRE(num_experts > 0 && num_experts <= 65536, I4TC_EINVAL, "num_experts out of range");
  if (num_pairs == 0 || N == 0) return I4TC_OK;
  I4TC_REQUIRE(a && b && scale_a && scale_b && expert_offsets && (out || out_rows), I4TC_EINVAL, "null pointer");
  I4TC_REQUIRE(num_pairs < (1ll << 31) - 256 && N * num_experts < (1ll << 31), I4TC_EINVAL, "sizes too large");
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  I4TC_REQUIRE(info->cc_major == 10, I4TC_EDEVICE, "device %d is sm_%d%d; this library needs sm_100", device,
               info->cc_major, info->cc_minor);
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);

  // 256-column tiles amortise the conversion of the activation tile better; narrow outputs fall
  // back to 128 columns.
  const int forced_bn = g_force_bn.load();
  int bn = forced_bn ? forced_bn : ((N % 256 == 0) ? 256 : 128);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.P_rows = (int)num_pairs;
  p.Q_rows = (int)N;
  p.G = (int)num_groups;
  p.epi_mode = EPI_GROUP;
  p.acc_unit = 1.0f / 256.0f;
  p.out_dtype = I4TC_BF16;
  p.sp = scale_a;
  p.sq = scale_b;
  p.sp_gstride = num_pairs;
  p.sq_gstride = N;
  p.sq_estride = num_groups * N;
  p.out = out;
  p.out_rows = reinterpret_cast<const unsigned long long*>(out_rows);
  p.ldc = N;
  p.num_q_tiles = (int)((N + bn - 1) / bn);
  p.expert_offsets = expert_offsets;
  p.num_experts = (int)num_experts;
  p.splits = 1;
  p.groups_per_split = (int)num_groups;
  p.status = info->status;
  CUtensorMap tmP, tmQ;
  if (int rc = get_tensor_map(device, a, false, num_pairs, num_groups, 128, &tmP)) return rc;
  // weights of all experts as one [E*G, N, 64] stack
  if (int rc = get_tensor_map(device, b, false, N, num_experts * num_groups, bn, &tmQ)) return rc;
  // upper bound on tiles: every expert may add one partial row tile
  const long long max_tiles = ((num_pairs + 127) / 128 + num_experts) * p.num_q_tiles;
  const int grid = (int)(max_tiles < info->sm_count ? max_tiles : info->sm_count);
  return launch_w4a4_gemm(p, tmP, tmQ, bn, grid, false, epi_warps_for(EPI_GROUP), static_cast<cudaStream_t>(stream));
}
