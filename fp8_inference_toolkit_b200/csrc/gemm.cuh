// W4A4 tile GEMM for sm_100a: declarations shared by the dense and the MoE entry points.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace i4tc {

// How the epilogue turns int32 accumulators into the output.
enum EpiMode : int {
  EPI_INT32 = 0,        // one flush per tile: out int32 = acc
  EPI_CHANNEL = 1,      // one flush per tile: out = cast((acc * s_col) * s_row)  (reference order b then a)
  EPI_GROUP = 2,        // a flush per K-group: f += (acc_g * sa[g,m]) * sb[g,n]; out = bf16(f)
  EPI_GROUP_INT32 = 3,  // a flush per K-group: out int32 [G, M, N] = acc_g
};

// One GEMM problem as the kernel sees it.  "P" is the operand on the 128-row side of the MMA
// (TMEM lanes), "Q" the operand on the BN-column side.  Normally P = activations (rows m) and
// Q = weights (rows n); with `swap` set P = weights and Q = activations (small M).
struct GemmParams {
  int P_rows;        // valid rows of the P operand (dense) or total sorted rows (MoE)
  int Q_rows;        // valid rows of the Q operand
  int G;             // number of 128-element K groups
  int p_rowmajor;    // 1: P tensor map is 2-D [rows, K/2] (x = g*64); 0: 3-D [G', rows, 64] (z = g)
  int q_rowmajor;
  int swap;          // output element (p, q) is out[q, p] instead of out[p, q]
  int i8_operands;   // 1: both operands are int8 already ([rows, K] row-major): TMA loads them straight into the
                     //    swizzled int8 stages and nothing is converted (W4A8: int8 activations, int4 weights held as int8)
  float acc_unit;    // what one unit of the int32 accumulator is worth: 1/256 for packed int4 operands (both carry
                     //    16 x code), 1 for int8 operands
  int epi_mode;      // EpiMode
  int out_dtype;     // I4TC_BF16 / I4TC_FP16 / I4TC_INT32
  const float* sp;   // P-side scales, element (g, p) at sp[g * sp_gstride + p]
  const float* sq;   // Q-side scales, element (g, q) at sq[g * sq_gstride + q]
  long long sp_gstride;
  long long sq_gstride;
  // Optional (per-group epilogue, unswapped, 16-bit output): address of every output row, 16-byte aligned, instead of
  // out + row * ldc -- rows may lie in another GPU's memory (plain stores over NVLink).
  const unsigned long long* out_rows;
  // Zero-point term of asymmetrically quantised activations (EPI_GROUP only; nullptr = none): group g adds
  // zp[g, p] * zq[g, q] to its integer sum before the scales (activation side: azp_adj, weight side: w_col_sum);
  // same strides as sp / sq.
  const float* zp;
  const float* zq;
  void* out;
  long long ldc;        // row stride of out in elements
  long long out_gstride;// EPI_GROUP_INT32: elements between consecutive groups
  int num_p_tiles;   // dense only
  int num_q_tiles;
  // MoE: rows [expert_offsets[e], expert_offsets[e+1]) of P use Q slab e.
  const int* expert_offsets;  // nullptr for a dense problem
  int num_experts;
  long long sq_estride;  // floats between experts in sq
  unsigned int* status;  // device status word, bit 0 = a bounded wait expired
  // Split-K (dense per-group mode, small M): the K groups are cut into `splits` ranges of
  // `groups_per_split`; range s writes fp32 partial sums to split_ws + s * ws_stride ([M, N] each),
  // and a second kernel adds the ranges in ascending order.
  int splits;
  int groups_per_split;
  float* split_ws;
  long long ws_stride;
};

// out[i] = bf16(sum_s ws[s * stride + i]), s ascending.
int launch_split_reduce(const float* ws, long long stride, int splits, long long n, void* out, cudaStream_t st);
// out[m, n] = cast((sum_s ws[s * stride + m * N + n] * sb[n]) * sa[m]): the ranges hold exact integer sums.
int launch_split_reduce_scaled(const float* ws, long long stride, int splits, long long M, long long N, const float* sa,
                               const float* sb, void* out, int out_dtype, cudaStream_t st);

// cta_pair: pairs of CTAs compute 256 x 256 tiles (dense, unswapped, bn = 256, even grid; p.num_p_tiles counts
// 256-row tiles and tmQ has 128-row boxes).
// epi_warps: 8 or 16 epilogue warps per CTA (16 needs bn >= 128).
int launch_w4a4_gemm(const GemmParams& p, const CUtensorMap& tmP, const CUtensorMap& tmQ, int bn, int grid,
                     bool cta_pair, int epi_warps, cudaStream_t st);

// CUDA-core weight-streaming kernel for M <= 8 tokens (per-group or per-channel scales, 16-bit output).
// x / w are the packed operands in either layout (rowmajor: [rows, G * 64]; else [G, rows, 64]).
bool gemv_applicable(long long M, long long N, long long K, int epi_mode);
int launch_w4a4_gemv(const uint8_t* x, const uint8_t* w, const float* sx, const float* sw, void* out, int out_dtype,
                     long long M, long long N, int G, bool rowmajor, int epi_mode, int sm_count, cudaStream_t st);

// Register-fed tensor-core weight-streaming kernel for M <= 32 tokens (same operands and outputs as the kernel above;
// `status` is the device status word that a bounded wait flags).
bool skinny_applicable(long long M, long long N, long long K, int epi_mode, bool rowmajor, int sm_count);
int launch_w4a4_skinny(const uint8_t* x, const uint8_t* w, const float* sx, const float* sw, void* out, int out_dtype,
                       long long M, long long N, int G, bool rowmajor, int epi_mode, int sm_count, unsigned int* status,
                       cudaStream_t st);

// Builds (or fetches from a small per-device cache) a tensor map over packed int4 data.
// rowmajor: 2-D view [rows, row_bytes]; otherwise 3-D view [slabs, rows, 64].
int get_tensor_map(int device, const void* base, bool rowmajor, long long rows, long long row_bytes_or_slabs,
                   int box_rows, CUtensorMap* out);
// Tensor map over int8 data [rows, K] (row pitch K bytes): boxes of 128 bytes (one K group) x box_rows, written to
// shared memory in the 128-byte swizzle the MMA descriptors expect; bytes past K read as zero.
int get_tensor_map_i8(int device, const void* base, long long rows, long long K, int box_rows, CUtensorMap* out);

}  // namespace i4tc
