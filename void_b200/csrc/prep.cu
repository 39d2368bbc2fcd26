// Preparation kernels of the SpMM path: tile index (row_ptr / block_indices), packing of the
// Morton-ordered tiles into tile-row-major core-matrix order, the INT8 / FP8-E4M3 quantisers
// for A tiles and for the columns of B, and the Stream-K worker table.  All of them are
// bandwidth-bound elementwise or gather kernels; none waits on another CTA.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/void_b200.h"

namespace vb {

static inline cudaStream_t as_stream(void_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
static inline int last_status() { return cudaGetLastError() == cudaSuccess ? VOID_OK : VOID_ERR_CUDA; }

// Exclusive prefix sum of n int32 values by ONE block of 1024 threads; out[n] = total.
// in and out may alias.
__device__ void block_exclusive_scan(const int32_t* in, int32_t* out, int n) {
  __shared__ int32_t part[1024];
  const int tid = threadIdx.x;
  const int per = (n + 1023) / 1024;
  const int lo = tid * per < n ? tid * per : n;
  const int hi = (lo + per) < n ? (lo + per) : n;
  int32_t s = 0;
  for (int i = lo; i < hi; ++i) s += in[i];
  part[tid] = s;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int32_t v = (tid >= off) ? part[tid - off] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  int32_t run = part[tid] - s;  // exclusive prefix of this thread's chunk
  for (int i = lo; i < hi; ++i) {
    const int32_t v = in[i];
    out[i] = run;
    run += v;
  }
  if (tid == 1023) out[n] = part[1023];
  __syncthreads();
}

// ------------------------------------------------------------------------------ tile index
// Coordinates outside the block grid are skipped here and in rank_tiles_kernel: the caller sees them (and
// repeated coordinates, which set one bit twice) as row_ptr[nbr] < nnz.
__global__ void mark_tiles_kernel(const int32_t* __restrict__ brow, const int32_t* __restrict__ bcol, int64_t nnz,
                                  int nbr, int nbc, int wpr, uint32_t* __restrict__ bitmap) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nnz) return;
  const int r = brow[i], c = bcol[i];
  if ((unsigned)r >= (unsigned)nbr || (unsigned)c >= (unsigned)nbc) return;
  atomicOr(bitmap + (size_t)r * wpr + (c >> 5), 1u << (c & 31));
}

__global__ void count_rows_kernel(const uint32_t* __restrict__ bitmap, int nbr, int wpr, int32_t* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= nbr) return;
  int c = 0;
  for (int w = lane; w < wpr; w += 32) c += __popc(bitmap[(size_t)warp * wpr + w]);
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if (lane == 0) counts[warp] = c;
}

__global__ void __launch_bounds__(1024) scan_rows_kernel(const int32_t* counts, int32_t* row_ptr, int nbr) {
  block_exclusive_scan(counts, row_ptr, nbr);
}

__global__ void rank_tiles_kernel(const int32_t* __restrict__ brow, const int32_t* __restrict__ bcol, int64_t nnz,
                                  int nbr, int nbc, int wpr, const uint32_t* __restrict__ bitmap,
                                  const int32_t* __restrict__ row_ptr, int32_t* __restrict__ block_indices) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nnz) return;
  const int r = brow[i], c = bcol[i];
  if ((unsigned)r >= (unsigned)nbr || (unsigned)c >= (unsigned)nbc) return;
  const uint32_t* row = bitmap + (size_t)r * wpr;
  int rank = 0;
  for (int w = 0; w < (c >> 5); ++w) rank += __popc(row[w]);
  rank += __popc(row[c >> 5] & ((1u << (c & 31)) - 1u));
  block_indices[row_ptr[r] + rank] = (int32_t)i;
}

// ------------------------------------------------------------------------------ pack
// One thread per 16-byte chunk of the packed tile.  Packed chunk q of a tile holds bytes
// [c16*16, c16*16+16) of tile row r with  q = (r/8)*16 + c16*8 + (r%8): four groups of eight
// rows, each group stored as two 8x16-byte core matrices (k bytes 0..15, then 16..31).
__global__ void pack_tiles_kernel(const uint4* __restrict__ values, const int32_t* __restrict__ block_indices,
                                  int64_t nnz, uint4* __restrict__ packed) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= nnz * 64) return;
  const int64_t j = g >> 6;
  const int q = (int)(g & 63);
  const int r = (q >> 4) * 8 + (q & 7);
  const int c16 = (q >> 3) & 1;
  const int64_t src_tile = block_indices[j];
  packed[g] = values[src_tile * 64 + r * 2 + c16];
}

// The same for elements of ES bytes: a tile row holds KC = 2*ES 16-byte chunks, a packed tile
// 64*ES of them in the order [row / 8][chunk][row % 8].
template <int ES>
__global__ void pack_tiles_fp_kernel(const uint4* __restrict__ values, const int32_t* __restrict__ block_indices,
                                     int64_t nnz, uint4* __restrict__ packed) {
  constexpr int KC = 2 * ES, PER_TILE = 64 * ES;
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= nnz * PER_TILE) return;
  const int64_t j = g / PER_TILE;
  const int q = (int)(g - j * PER_TILE);
  const int r = (q / (8 * KC)) * 8 + (q & 7);
  const int kc = (q >> 3) % KC;
  const int64_t src_tile = block_indices[j];
  uint4 v = values[src_tile * PER_TILE + r * KC + kc];
  if (ES == 4) {
    // The tensor cores read an fp32 operand as TF32 by dropping its low 13 mantissa bits.  Rounding the
    // tiles to the nearest TF32 value here, once, halves the error of that and removes its bias.
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v.x) : "f"(__uint_as_float(v.x)));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v.y) : "f"(__uint_as_float(v.y)));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v.z) : "f"(__uint_as_float(v.z)));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(v.w) : "f"(__uint_as_float(v.w)));
  }
  packed[g] = v;
}

// FP8 tiles with their scales folded in, for the row-accumulate kernel: the tensor cores cannot scale a
// product per tile, so each element a * s_tile / R_row (R_row = the largest tile scale of the tile row) is
// written as a sum of `terms` E4M3 numbers - the nearest E4M3 value, then the nearest E4M3 value of what is
// left, and once more for three terms - and every term is multiplied by the same panel of B.  Two terms carry
// 8 significant bits (relative error below 2^-8 per element, unbiased), three carry 12; the differences
// x - hi and (x - hi) - mid are exact in fp32.  The epilogue multiplies the row's sums by R_row.
// One thread per 16-byte chunk of a packed tile, same chunk order as pack_tiles_kernel; term k of packed
// tile j lies at chunk (j * terms + k) * 64.
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3)));
}
template <int TERMS>
__global__ void pack_tiles_f8_split_kernel(const uint4* __restrict__ values, const float* __restrict__ scales,
                                           int64_t n_scales, const int32_t* __restrict__ block_rows,
                                           const int32_t* __restrict__ block_indices,
                                           const float* __restrict__ row_scale, int64_t nnz,
                                           uint4* __restrict__ packed) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= nnz * 64) return;
  const int64_t j = g >> 6;
  const int q = (int)(g & 63);
  const int r = (q >> 4) * 8 + (q & 7);
  const int c16 = (q >> 3) & 1;
  const int64_t src = block_indices[j];
  const uint4 v = values[src * 64 + r * 2 + c16];
  const float s = (scales == nullptr) ? 1.0f : (n_scales == 1 ? scales[0] : scales[src]);
  const float R = row_scale[block_rows[src]];
  const float ratio = (R > 0.0f) ? __fdiv_rn(s, R) : 0.0f;
  const uint32_t in[4] = {v.x, v.y, v.z, v.w};
  uint32_t out[TERMS][4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
#pragma unroll
    for (int k = 0; k < TERMS; ++k) out[k][w] = 0u;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float x = __fmul_rn(e4m3_to_float((uint8_t)(in[w] >> (8 * e))), ratio);
#pragma unroll
      for (int k = 0; k < TERMS; ++k) {
        const uint8_t t = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
        out[k][w] |= (uint32_t)t << (8 * e);
        x = __fsub_rn(x, e4m3_to_float(t));
      }
    }
  }
#pragma unroll
  for (int k = 0; k < TERMS; ++k) packed[(j * TERMS + k) * 64 + q] = make_uint4(out[k][0], out[k][1], out[k][2], out[k][3]);
}

// Sum of the per-rank partial tiles of the tile rows this GPU owns, then the INT8 epilogue.  One block per
// (owned tile row, 128-column panel), one thread per column n: the slots hold int32 tiles [32 m][128 n], so a
// warp reads 128 contiguous bytes per m.  contrib[row] has bit r set when rank r stored a tile for the row
// (a rank without tiles in the row stores nothing and its slot is not read).
__device__ __forceinline__ float reduce_act(float x, int act) {
  if (act == VOID_ACT_RELU) return fmaxf(x, 0.0f);
  if (act == VOID_ACT_GELU) {
    const float two_u = 1.5957691216f * x * fmaf(0.044715f * x, x, 1.0f);
    return x * __fdividef(1.0f, 1.0f + __expf(-two_u));
  }
  if (act == VOID_ACT_SILU) return x * __fdividef(1.0f, 1.0f + __expf(-x));
  return x;
}
__global__ void __launch_bounds__(128) reduce_slots_kernel(const int32_t* __restrict__ slots, const uint8_t* __restrict__ contrib,
                                                           int n_ranks, int rows_owned, int row0, int n_panels,
                                                           int np, const float* __restrict__ row_scale,
                                                           const float* __restrict__ col_scale, float b_scale,
                                                           const float* __restrict__ bias, int act, void* out,
                                                           long long ldc, int out_dtype, int M, int N) {
  const int item = blockIdx.x;                 // local row * n_panels + panel
  const int lr = item / n_panels, pan = item - lr * n_panels;
  if (lr >= rows_owned) return;
  const int n = pan * 128 + threadIdx.x;
  const unsigned mask = contrib[lr];
  int acc[32];
#pragma unroll
  for (int m = 0; m < 32; ++m) acc[m] = 0;
  for (int r = 0; r < n_ranks; ++r) {
    if (!((mask >> r) & 1u)) continue;
    // slots are laid out as the SpMM kernel writes them: [row][chunk of np panels][rank][panel of the chunk]
    const int n_chunks = (n_panels + np - 1) / np;
    const int32_t* t = slots + ((((size_t)lr * n_chunks + pan / np) * n_ranks + r) * np + pan % np) * 4096 + threadIdx.x;
#pragma unroll
    for (int m = 0; m < 32; ++m) acc[m] += __ldcs(t + m * 128);
  }
  if (n >= N) return;
  const int grow = row0 + lr;                  // global tile row
  const float rs = row_scale[grow];
  const float cs = (col_scale != nullptr ? col_scale[n] : 1.0f) * b_scale;
  const float bi = bias != nullptr ? bias[n] : 0.0f;
#pragma unroll
  for (int m = 0; m < 32; ++m) {
    const long long gm = (long long)grow * 32 + m;
    if (gm >= M) break;
    const float v = reduce_act((__int2float_rn(acc[m]) * rs) * cs + bi, act);
    const size_t o = (size_t)(lr * 32 + m) * ldc + n;
    if (out_dtype == VOID_OUT_F16) reinterpret_cast<__half*>(out)[o] = __float2half_rn(v);
    else if (out_dtype == VOID_OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(out)[o] = v;
  }
}

// largest tile scale of every tile row (0 for an empty row)
__global__ void row_max_scale_kernel(const int32_t* __restrict__ row_ptr, const float* __restrict__ tile_scales, int nbr,
                                     float* __restrict__ row_scale) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= nbr) return;
  float m = 0.0f;
  for (int t = row_ptr[r]; t < row_ptr[r + 1]; ++t) m = fmaxf(m, tile_scales[t]);
  row_scale[r] = m;
}

__global__ void gather_tile_meta_kernel(const int32_t* __restrict__ bcol, const float* __restrict__ scales,
                                        int64_t n_scales, const int32_t* __restrict__ block_indices, int64_t nnz,
                                        int32_t* __restrict__ tile_cols, float* __restrict__ tile_scales) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= nnz) return;
  const int64_t src = block_indices[j];
  tile_cols[j] = bcol[src];
  if (tile_scales != nullptr) tile_scales[j] = (scales == nullptr) ? 1.0f : (n_scales == 1 ? scales[0] : scales[src]);
}

// mean of the row's tile scales, added one by one in row order like the reference's loop
__global__ void row_scale_kernel(const int32_t* __restrict__ row_ptr, const float* __restrict__ tile_scales, int nbr,
                                 float* __restrict__ row_scale) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= nbr) return;
  const int t0 = row_ptr[r], t1 = row_ptr[r + 1];
  float s = 0.0f;
  for (int t = t0; t < t1; ++t) s = __fadd_rn(s, tile_scales[t]);
  row_scale[r] = (t1 > t0) ? __fdiv_rn(s, (float)(t1 - t0)) : 0.0f;
}

// ------------------------------------------------------------------------------ quantisers
__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int8_t quant_i8(float x, float scale) {
  float q = rintf(__fdiv_rn(x, scale));
  q = fminf(fmaxf(q, -128.0f), 127.0f);
  return (int8_t)(int)q;
}
__device__ __forceinline__ uint8_t quant_e4m3(float x, float scale_inv) {
  float s = __fmul_rn(x, scale_inv);
  s = fminf(fmaxf(s, -448.0f), 448.0f);
  return (uint8_t)__nv_cvt_float_to_fp8(s, __NV_SATFINITE, __NV_E4M3);
}

// one warp per tile: 1024 fp32 values, 32 per lane
__global__ void quant_i8_tiles_kernel(const float4* __restrict__ values, int64_t nnz, int8_t* __restrict__ q,
                                      float* __restrict__ scales) {
  const int64_t tile = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tile >= nnz) return;
  const float4* src = values + tile * 256;
  float4 v[8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = src[i * 32 + lane];
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
  }
  amax = warp_max(amax);
  const float scale = fmaxf(__fdiv_rn(amax, 128.0f), 1e-8f);
  if (lane == 0) scales[tile] = scale;
  char4* dst = reinterpret_cast<char4*>(q) + tile * 256;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    char4 o;
    o.x = quant_i8(v[i].x, scale); o.y = quant_i8(v[i].y, scale);
    o.z = quant_i8(v[i].z, scale); o.w = quant_i8(v[i].w, scale);
    dst[i * 32 + lane] = o;
  }
}

__global__ void quant_fp8_tiles_kernel(const float4* __restrict__ values, int64_t nnz, uint8_t* __restrict__ q,
                                       float* __restrict__ scale_out, float* __restrict__ scale_inv_out,
                                       float* __restrict__ amax_out) {
  const int64_t tile = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tile >= nnz) return;
  const float4* src = values + tile * 256;
  float4 v[8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = src[i * 32 + lane];
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
  }
  amax = warp_max(amax);
  const float scale = fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
  const float inv = __fdiv_rn(1.0f, scale);
  if (lane == 0) {
    scale_out[tile] = scale;
    if (scale_inv_out != nullptr) scale_inv_out[tile] = inv;
    if (amax_out != nullptr) amax_out[tile] = amax;
  }
  uchar4* dst = reinterpret_cast<uchar4*>(q) + tile * 256;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uchar4 o;
    o.x = quant_e4m3(v[i].x, inv); o.y = quant_e4m3(v[i].y, inv);
    o.z = quant_e4m3(v[i].z, inv); o.w = quant_e4m3(v[i].w, inv);
    dst[i * 32 + lane] = o;
  }
}

// column absmax of a row-major [K, N] matrix: block = 128 columns x a slab of k rows
constexpr int kColBlock = 128;
constexpr int kRowSlab = 64;
__global__ void col_amax_kernel(const float* __restrict__ b, int64_t ldb, int K, int N, float* __restrict__ amax) {
  const int n = blockIdx.x * kColBlock + threadIdx.x;
  if (n >= N) return;
  const int k0 = blockIdx.y * kRowSlab;
  const int k1 = (k0 + kRowSlab) < K ? (k0 + kRowSlab) : K;
  float m = 0.0f;
  for (int k = k0; k < k1; ++k) m = fmaxf(m, fabsf(b[(size_t)k * ldb + n]));
  // non-negative floats order like their bit patterns
  atomicMax(reinterpret_cast<int*>(amax) + n, __float_as_int(m));
}
__global__ void col_scale_kernel(float* __restrict__ scale, float* __restrict__ scale_inv, int N, int kind) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const float amax = scale[n];
  float s;
  if (kind == VOID_KIND_I8) s = fmaxf(__fdiv_rn(amax, 128.0f), 1e-8f);
  else s = fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
  scale[n] = s;
  if (scale_inv != nullptr) scale_inv[n] = __fdiv_rn(1.0f, s);
}
__global__ void quant_cols_kernel(const float* __restrict__ b, int64_t ldb, int K, int N, int kind,
                                  uint8_t* __restrict__ q, int64_t ldq, const float* __restrict__ scale,
                                  int scale_stride) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int k = blockIdx.y;
  if (n >= ldq) return;
  uint8_t o = 0;
  if (n < N) {
    const float x = b[(size_t)k * ldb + n];
    const float s = scale[(size_t)n * scale_stride];
    if (kind == VOID_KIND_I8) o = (uint8_t)quant_i8(x, s);
    else o = quant_e4m3(x, __fdiv_rn(1.0f, s));
  }
  q[(size_t)k * ldq + n] = o;
}
// four columns per thread (float4 in, 4 bytes out); needs N, ldb, ldq multiples of 4 and aligned rows
__global__ void quant_cols4_kernel(const float* __restrict__ b, int64_t ldb, int K, int N, int kind,
                                   uint8_t* __restrict__ q, int64_t ldq, const float* __restrict__ scale,
                                   int scale_stride) {
  const int n = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const int k = blockIdx.y;
  if (n >= ldq) return;
  uchar4 o = make_uchar4(0, 0, 0, 0);
  if (n < N) {
    const float4 x = *reinterpret_cast<const float4*>(b + (size_t)k * ldb + n);
    float s0, s1, s2, s3;
    if (scale_stride) {
      const float4 s = *reinterpret_cast<const float4*>(scale + n);
      s0 = s.x; s1 = s.y; s2 = s.z; s3 = s.w;
    } else {
      s0 = s1 = s2 = s3 = scale[0];
    }
    if (kind == VOID_KIND_I8) {
      o.x = (uint8_t)quant_i8(x.x, s0); o.y = (uint8_t)quant_i8(x.y, s1);
      o.z = (uint8_t)quant_i8(x.z, s2); o.w = (uint8_t)quant_i8(x.w, s3);
    } else {
      o.x = quant_e4m3(x.x, __fdiv_rn(1.0f, s0)); o.y = quant_e4m3(x.y, __fdiv_rn(1.0f, s1));
      o.z = quant_e4m3(x.z, __fdiv_rn(1.0f, s2)); o.w = quant_e4m3(x.w, __fdiv_rn(1.0f, s3));
    }
  }
  *reinterpret_cast<uchar4*>(q + (size_t)k * ldq + n) = o;
}
// absmax of a whole row-major [K, N] matrix into amax[0] (zero before the launch)
__global__ void tensor_amax_kernel(const float* __restrict__ b, int64_t ldb, int K, int N, float* __restrict__ amax) {
  const int n = blockIdx.x * kColBlock + threadIdx.x;
  const int k0 = blockIdx.y * kRowSlab;
  const int k1 = (k0 + kRowSlab) < K ? (k0 + kRowSlab) : K;
  float m = 0.0f;
  if (n < N)
    for (int k = k0; k < k1; ++k) m = fmaxf(m, fabsf(b[(size_t)k * ldb + n]));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
}

// ------------------------------------------------------------------------------ Stream-K table
__global__ void __launch_bounds__(1024) streamk_offsets_kernel(const int32_t* __restrict__ row_ptr, int nbr,
                                                               int target, int32_t* __restrict__ woff,
                                                               int32_t* __restrict__ n_workers_out) {
  // woff[r] = number of chunks of row r, then scanned in place
  for (int r = threadIdx.x; r < nbr; r += blockDim.x) {
    const int cnt = row_ptr[r + 1] - row_ptr[r];
    woff[r] = (cnt + target - 1) / target;
  }
  __syncthreads();
  block_exclusive_scan(woff, woff, nbr);
  if (threadIdx.x == 0) *n_workers_out = woff[nbr];
}
__global__ void streamk_fill_kernel(const int32_t* __restrict__ row_ptr, int nbr, int target,
                                    const int32_t* __restrict__ woff, int32_t* __restrict__ w_rows,
                                    int32_t* __restrict__ w_start, int32_t* __restrict__ w_end,
                                    uint8_t* __restrict__ w_atomic) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= nbr) return;
  const int rs = row_ptr[r], re = row_ptr[r + 1];
  const int chunks = woff[r + 1] - woff[r];
  int w = woff[r];
  for (int pos = rs; pos < re; pos += target, ++w) {
    const int e = (pos + target) < re ? (pos + target) : re;
    w_rows[w] = r;
    w_start[w] = pos;
    w_end[w] = e;
    w_atomic[w] = chunks > 1 ? 1 : 0;
  }
}

}  // namespace vb

using namespace vb;

extern "C" {

const char* void_strerror(int status) {
  switch (status) {
    case VOID_OK: return "ok";
    case VOID_ERR_BAD_ARG: return "bad argument (null pointer, negative size or unknown enum value)";
    case VOID_ERR_ALIGN: return "pointer or leading dimension breaks an alignment rule";
    case VOID_ERR_SHAPE: return "unsupported shape";
    case VOID_ERR_ARCH: return "current device is not an sm_100 (B200) GPU";
    case VOID_ERR_CUDA: return "a CUDA runtime or driver call failed";
    case VOID_ERR_WORKSPACE: return "workspace too small";
    case VOID_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case VOID_ERR_TOO_LARGE: return "size beyond a documented maximum";
    case VOID_ERR_TENSOR_MAP: return "the driver refused the copy-engine (TMA) descriptor of B";
    default: return "unknown status";
  }
}

int void_b200_abi_version(void) { return VOID_B200_ABI_VERSION; }

size_t void_tile_index_ws_bytes(int32_t nbr, int32_t nbc) {
  if (nbr <= 0 || nbc <= 0) return 16;
  const size_t wpr = ((size_t)nbc + 31) / 32;
  return (size_t)nbr * wpr * 4 + (size_t)nbr * 4 + 16;
}

int void_build_tile_index(const int32_t* block_rows, const int32_t* block_cols, int64_t nnz, int32_t nbr,
                          int32_t nbc, int32_t* row_ptr, int32_t* block_indices, void* ws, size_t ws_bytes,
                          void_stream_t stream) {
  if (nnz < 0 || nbr < 0 || nbc < 0 || row_ptr == nullptr) return VOID_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  if (nbr == 0) return cudaMemsetAsync(row_ptr, 0, 4, st) == cudaSuccess ? VOID_OK : VOID_ERR_CUDA;
  if (nnz > 0 && (block_rows == nullptr || block_cols == nullptr || block_indices == nullptr)) return VOID_ERR_BAD_ARG;
  if (nnz > 0x7fffffffLL) return VOID_ERR_TOO_LARGE;
  if (ws == nullptr || ws_bytes < void_tile_index_ws_bytes(nbr, nbc)) return VOID_ERR_WORKSPACE;
  const int wpr = (nbc + 31) / 32;
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(ws);
  int32_t* counts = reinterpret_cast<int32_t*>(bitmap + (size_t)nbr * wpr);
  if (cudaMemsetAsync(bitmap, 0, (size_t)nbr * wpr * 4, st) != cudaSuccess) return VOID_ERR_CUDA;
  const int tb = 256;
  // every entry of block_indices is a valid position even when the list is rejected afterwards
  if (nnz > 0 && cudaMemsetAsync(block_indices, 0, (size_t)nnz * 4, st) != cudaSuccess) return VOID_ERR_CUDA;
  if (nnz > 0)
    mark_tiles_kernel<<<(unsigned)((nnz + tb - 1) / tb), tb, 0, st>>>(block_rows, block_cols, nnz, nbr, nbc, wpr, bitmap);
  count_rows_kernel<<<(unsigned)(((int64_t)nbr * 32 + tb - 1) / tb), tb, 0, st>>>(bitmap, nbr, wpr, counts);
  scan_rows_kernel<<<1, 1024, 0, st>>>(counts, row_ptr, nbr);
  if (nnz > 0)
    rank_tiles_kernel<<<(unsigned)((nnz + tb - 1) / tb), tb, 0, st>>>(block_rows, block_cols, nnz, nbr, nbc, wpr, bitmap,
                                                                     row_ptr, block_indices);
  return last_status();
}

int void_pack_tiles(const void* values, const float* scales, int64_t n_scales, const int32_t* block_cols,
                    const int32_t* block_indices, const int32_t* row_ptr, int64_t nnz, int32_t nbr, void* packed,
                    int32_t* tile_cols, float* tile_scales, float* row_scale, void_stream_t stream) {
  if (nnz < 0 || nbr < 0) return VOID_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  const int tb = 256;
  if (nnz > 0) {
    if (values == nullptr || block_cols == nullptr || block_indices == nullptr || packed == nullptr ||
        tile_cols == nullptr)
      return VOID_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(values) & 15u) != 0 || (reinterpret_cast<uintptr_t>(packed) & 1023u) != 0)
      return VOID_ERR_ALIGN;
    if (scales != nullptr && n_scales != 1 && n_scales != nnz) return VOID_ERR_BAD_ARG;
    pack_tiles_kernel<<<(unsigned)((nnz * 64 + tb - 1) / tb), tb, 0, st>>>(
        reinterpret_cast<const uint4*>(values), block_indices, nnz, reinterpret_cast<uint4*>(packed));
    gather_tile_meta_kernel<<<(unsigned)((nnz + tb - 1) / tb), tb, 0, st>>>(block_cols, scales, n_scales, block_indices,
                                                                           nnz, tile_cols, tile_scales);
  }
  if (row_scale != nullptr && nbr > 0) {
    if (row_ptr == nullptr || (nnz > 0 && tile_scales == nullptr)) return VOID_ERR_BAD_ARG;
    row_scale_kernel<<<(nbr + tb - 1) / tb, tb, 0, st>>>(row_ptr, tile_scales, nbr, row_scale);
  }
  return last_status();
}

int void_pack_tiles_f8_split(const void* values, const float* scales, int64_t n_scales, const int32_t* block_rows,
                             const int32_t* block_cols, const int32_t* block_indices, const int32_t* row_ptr, int64_t nnz,
                             int32_t nbr, int32_t terms, void* packed, int32_t* tile_cols, float* tile_scales,
                             float* row_scale, void_stream_t stream) {
  if (nnz < 0 || nbr < 0 || (terms != 2 && terms != 3)) return VOID_ERR_BAD_ARG;
  if (row_ptr == nullptr || row_scale == nullptr) return VOID_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  const int tb = 256;
  if (nnz > 0) {
    if (values == nullptr || block_rows == nullptr || block_cols == nullptr || block_indices == nullptr ||
        packed == nullptr || tile_cols == nullptr || tile_scales == nullptr)
      return VOID_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(values) & 15u) != 0 || (reinterpret_cast<uintptr_t>(packed) & 1023u) != 0)
      return VOID_ERR_ALIGN;
    if (scales != nullptr && n_scales != 1 && n_scales != nnz) return VOID_ERR_BAD_ARG;
    gather_tile_meta_kernel<<<(unsigned)((nnz + tb - 1) / tb), tb, 0, st>>>(block_cols, scales, n_scales, block_indices,
                                                                           nnz, tile_cols, tile_scales);
  }
  if (nbr > 0) row_max_scale_kernel<<<(nbr + tb - 1) / tb, tb, 0, st>>>(row_ptr, tile_scales, nbr, row_scale);
  if (nnz > 0) {
    const unsigned blocks = (unsigned)((nnz * 64 + tb - 1) / tb);
    if (terms == 2)
      pack_tiles_f8_split_kernel<2><<<blocks, tb, 0, st>>>(reinterpret_cast<const uint4*>(values), scales, n_scales,
                                                           block_rows, block_indices, row_scale, nnz,
                                                           reinterpret_cast<uint4*>(packed));
    else
      pack_tiles_f8_split_kernel<3><<<blocks, tb, 0, st>>>(reinterpret_cast<const uint4*>(values), scales, n_scales,
                                                           block_rows, block_indices, row_scale, nnz,
                                                           reinterpret_cast<uint4*>(packed));
  }
  return last_status();
}

int void_reduce_slots(const void* slots, const uint8_t* contrib, int32_t n_ranks, int32_t rows_owned, int32_t row0,
                      int32_t n_panels, int32_t panels_per_item, const float* row_scale, const float* col_scale, float b_scale, const float* bias,
                      int32_t act, void* out, int64_t ldc, int32_t out_dtype, int32_t M, int32_t N, void_stream_t stream) {
  if (n_ranks < 1 || n_ranks > 8 || rows_owned < 0 || n_panels < 1 || N < 1 || M < 0) return VOID_ERR_BAD_ARG;
  if (panels_per_item != 1 && panels_per_item != 2 && panels_per_item != 4) return VOID_ERR_BAD_ARG;
  if (out_dtype < VOID_OUT_F32 || out_dtype > VOID_OUT_BF16 || act < VOID_ACT_NONE || act > VOID_ACT_SILU) return VOID_ERR_BAD_ARG;
  if (rows_owned == 0) return VOID_OK;
  if (slots == nullptr || contrib == nullptr || row_scale == nullptr || out == nullptr || ldc < N) return VOID_ERR_BAD_ARG;
  if ((long long)n_panels * 128 < N) return VOID_ERR_SHAPE;
  reduce_slots_kernel<<<(unsigned)(rows_owned * n_panels), 128, 0, as_stream(stream)>>>(
      reinterpret_cast<const int32_t*>(slots), contrib, n_ranks, rows_owned, row0, n_panels, panels_per_item, row_scale, col_scale, b_scale,
      bias, act, out, ldc, out_dtype, M, N);
  return last_status();
}

int void_pack_tiles_fp(const void* values, int32_t elem_bytes, const int32_t* block_cols, const int32_t* block_indices,
                       int64_t nnz, void* packed, int32_t* tile_cols, void_stream_t stream) {
  if (nnz < 0 || (elem_bytes != 2 && elem_bytes != 4)) return VOID_ERR_BAD_ARG;
  if (nnz == 0) return VOID_OK;
  if (values == nullptr || block_cols == nullptr || block_indices == nullptr || packed == nullptr || tile_cols == nullptr)
    return VOID_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(values) & 15u) != 0 || (reinterpret_cast<uintptr_t>(packed) & 1023u) != 0)
    return VOID_ERR_ALIGN;
  cudaStream_t st = as_stream(stream);
  const int tb = 256;
  const unsigned blocks = (unsigned)((nnz * 64 * elem_bytes + tb - 1) / tb);
  if (elem_bytes == 2)
    pack_tiles_fp_kernel<2><<<blocks, tb, 0, st>>>(reinterpret_cast<const uint4*>(values), block_indices, nnz,
                                                   reinterpret_cast<uint4*>(packed));
  else
    pack_tiles_fp_kernel<4><<<blocks, tb, 0, st>>>(reinterpret_cast<const uint4*>(values), block_indices, nnz,
                                                   reinterpret_cast<uint4*>(packed));
  gather_tile_meta_kernel<<<(unsigned)((nnz + tb - 1) / tb), tb, 0, st>>>(block_cols, nullptr, 0, block_indices, nnz,
                                                                         tile_cols, nullptr);
  return last_status();
}

int void_quant_i8_tiles(const float* values, int64_t nnz, int8_t* q, float* scales, void_stream_t stream) {
  if (nnz < 0) return VOID_ERR_BAD_ARG;
  if (nnz == 0) return VOID_OK;
  if (values == nullptr || q == nullptr || scales == nullptr) return VOID_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(values) & 15u) != 0 || (reinterpret_cast<uintptr_t>(q) & 3u) != 0) return VOID_ERR_ALIGN;
  const int tb = 256;
  quant_i8_tiles_kernel<<<(unsigned)((nnz * 32 + tb - 1) / tb), tb, 0, as_stream(stream)>>>(
      reinterpret_cast<const float4*>(values), nnz, q, scales);
  return last_status();
}

int void_quant_fp8_tiles(const float* values, int64_t nnz, uint8_t* q, float* scale, float* scale_inv, float* amax,
                         void_stream_t stream) {
  if (nnz < 0) return VOID_ERR_BAD_ARG;
  if (nnz == 0) return VOID_OK;
  if (values == nullptr || q == nullptr || scale == nullptr) return VOID_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(values) & 15u) != 0 || (reinterpret_cast<uintptr_t>(q) & 3u) != 0) return VOID_ERR_ALIGN;
  const int tb = 256;
  quant_fp8_tiles_kernel<<<(unsigned)((nnz * 32 + tb - 1) / tb), tb, 0, as_stream(stream)>>>(
      reinterpret_cast<const float4*>(values), nnz, q, scale, scale_inv, amax);
  return last_status();
}

static void quant_pass(const float* b, int64_t ldb, int K, int N, int kind, void* q, int64_t ldq, const float* scale,
                       int scale_stride, cudaStream_t st) {
  const bool vec4 = (N % 4 == 0) && (ldb % 4 == 0) && (ldq % 4 == 0) && ((reinterpret_cast<uintptr_t>(b) & 15u) == 0) &&
                    ((reinterpret_cast<uintptr_t>(q) & 3u) == 0) && ((reinterpret_cast<uintptr_t>(scale) & 15u) == 0);
  // blockIdx.y is limited to 65535: quantise in slabs of rows
  for (int k0 = 0; k0 < K; k0 += 65535) {
    const int kk = (K - k0) < 65535 ? (K - k0) : 65535;
    const float* src = b + (size_t)k0 * ldb;
    uint8_t* dst = reinterpret_cast<uint8_t*>(q) + (size_t)k0 * ldq;
    if (vec4) {
      dim3 g2((unsigned)((ldq / 4 + 127) / 128), kk);
      quant_cols4_kernel<<<g2, 128, 0, st>>>(src, ldb, kk, N, kind, dst, ldq, scale, scale_stride);
    } else {
      dim3 g2((unsigned)((ldq + 255) / 256), kk);
      quant_cols_kernel<<<g2, 256, 0, st>>>(src, ldb, kk, N, kind, dst, ldq, scale, scale_stride);
    }
  }
}

int void_quant_cols(const float* b, int64_t ldb, int32_t K, int32_t N, int32_t kind, void* q, int64_t ldq,
                    float* col_scale, float* col_scale_inv, void_stream_t stream) {
  if (K < 0 || N < 0 || (kind != VOID_KIND_I8 && kind != VOID_KIND_F8E4M3)) return VOID_ERR_BAD_ARG;
  if (K == 0 || N == 0) return VOID_OK;
  if (b == nullptr || q == nullptr || col_scale == nullptr) return VOID_ERR_BAD_ARG;
  if (ldb < N || ldq < N) return VOID_ERR_SHAPE;
  if (K > 65535 * kRowSlab) return VOID_ERR_TOO_LARGE;
  cudaStream_t st = as_stream(stream);
  if (cudaMemsetAsync(col_scale, 0, (size_t)N * 4, st) != cudaSuccess) return VOID_ERR_CUDA;
  dim3 g1((N + kColBlock - 1) / kColBlock, (K + kRowSlab - 1) / kRowSlab);
  col_amax_kernel<<<g1, kColBlock, 0, st>>>(b, ldb, K, N, col_scale);
  col_scale_kernel<<<(N + 255) / 256, 256, 0, st>>>(col_scale, col_scale_inv, N, kind);
  quant_pass(b, ldb, K, N, kind, q, ldq, col_scale, 1, st);
  return last_status();
}

int void_quant_i8_tensor(const float* b, int64_t ldb, int32_t K, int32_t N, void* q, int64_t ldq, float* scale,
                         void_stream_t stream) {
  if (K < 0 || N < 0) return VOID_ERR_BAD_ARG;
  if (b == nullptr || q == nullptr || scale == nullptr) return VOID_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  if (cudaMemsetAsync(scale, 0, 4, st) != cudaSuccess) return VOID_ERR_CUDA;
  if (K == 0 || N == 0) return VOID_OK;
  if (ldb < N || ldq < N) return VOID_ERR_SHAPE;
  if (K > 65535 * kRowSlab) return VOID_ERR_TOO_LARGE;
  dim3 g1((N + kColBlock - 1) / kColBlock, (K + kRowSlab - 1) / kRowSlab);
  tensor_amax_kernel<<<g1, kColBlock, 0, st>>>(b, ldb, K, N, scale);
  col_scale_kernel<<<1, 32, 0, st>>>(scale, nullptr, 1, VOID_KIND_I8);
  quant_pass(b, ldb, K, N, VOID_KIND_I8, q, ldq, scale, 0, st);
  return last_status();
}

int64_t void_streamk_table_capacity(int64_t nnz, int32_t nbr) {
  (void)nbr;
  return nnz > 0 ? nnz : 1;
}

int32_t void_streamk_target(int64_t nnz, int32_t n_workers_req, int32_t max_work) {
  // target_work of compute_stream_k_workload, void/stream_k.py:61-67
  if (nnz <= 0) return 0;
  int64_t n_workers = n_workers_req > 0 ? n_workers_req : (nnz < 1024 ? nnz : 1024);
  int64_t target = (nnz + n_workers - 1) / n_workers;
  if (target > max_work) target = max_work;
  return (int32_t)target;
}

int void_streamk_table(const int32_t* row_ptr, int32_t nbr, int64_t nnz, int32_t n_workers_req, int32_t max_work,
                       int32_t* worker_rows, int32_t* worker_block_start, int32_t* worker_block_end,
                       uint8_t* worker_needs_atomic, int32_t* n_workers_out, int32_t* ws, void_stream_t stream) {
  if (row_ptr == nullptr || nbr <= 0 || nnz <= 0 || max_work <= 0) return VOID_ERR_BAD_ARG;
  if (worker_rows == nullptr || worker_block_start == nullptr || worker_block_end == nullptr ||
      worker_needs_atomic == nullptr || n_workers_out == nullptr || ws == nullptr)
    return VOID_ERR_BAD_ARG;
  const int target = void_streamk_target(nnz, n_workers_req, max_work);
  if (target <= 0) return VOID_ERR_BAD_ARG;
  cudaStream_t st = as_stream(stream);
  streamk_offsets_kernel<<<1, 1024, 0, st>>>(row_ptr, nbr, target, ws, n_workers_out);
  streamk_fill_kernel<<<(nbr + 255) / 256, 256, 0, st>>>(row_ptr, nbr, target, ws, worker_rows, worker_block_start,
                                                        worker_block_end, worker_needs_atomic);
  return last_status();
}

}  // extern "C"
