// On-device construction of the VOID format: which 32x32 tiles of a dense or CSR matrix are kept,
// their Morton (Z-order) ranking, and the tile values.
//
// The reference builds the format on the host: dense_to_void (void/format.py:352-446) finds the
// active tiles with torch ops but computes and sorts the Morton codes in numpy, csr_to_void
// (:248-349) does everything in numpy with a Python loop over the nonzeros (:321-327).  Here the
// ranking is a bitmap in Morton-code space: bit morton(r, c) is set for every kept tile, a prefix
// sum of the words' population counts gives every set bit its rank, and rank order IS ascending
// Morton order - no sort.  All kernels are bandwidth-bound passes; none waits on another CTA.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/void_b200.h"

namespace vbf {

constexpr int kTile = 32;
constexpr int kChunkWords = 1024;  // words of the bitmap summed by one block

static inline cudaStream_t as_stream(void_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }
static inline int last_status() { return cudaGetLastError() == cudaSuccess ? VOID_OK : VOID_ERR_CUDA; }

// morton(r, c): bits of r on the even positions, bits of c on the odd ones (void/format.py:41-51)
__host__ __device__ inline uint32_t spread16(uint32_t v) {
  v = (v | (v << 8)) & 0x00FF00FFu;
  v = (v | (v << 4)) & 0x0F0F0F0Fu;
  v = (v | (v << 2)) & 0x33333333u;
  v = (v | (v << 1)) & 0x55555555u;
  return v;
}
__host__ __device__ inline uint32_t compact16(uint32_t v) {
  v &= 0x55555555u;
  v = (v | (v >> 1)) & 0x33333333u;
  v = (v | (v >> 2)) & 0x0F0F0F0Fu;
  v = (v | (v >> 4)) & 0x00FF00FFu;
  v = (v | (v >> 8)) & 0x0000FFFFu;
  return v;
}
__host__ __device__ inline uint32_t morton(uint32_t r, uint32_t c) { return spread16(r) | (spread16(c) << 1); }

// Side of the Morton square that holds the block grid (a power of two), and its bitmap size.
static int morton_side(int nbr, int nbc) {
  int s = 1;
  while (s < nbr || s < nbc) s <<= 1;
  return s;
}
struct WsLayout {
  int64_t words;       // 32-bit words of the bitmap
  int64_t chunks;      // blocks of kChunkWords words
  size_t off_prefix;   // int32 word_prefix[words + 1]
  size_t off_chunk;    // int32 chunk_ptr[chunks + 1]
  size_t off_counts;   // unsigned long long counts[2]: kept tiles, nonzero elements
  size_t bytes;
};
static bool ws_layout(int nbr, int nbc, WsLayout* w) {
  if (nbr <= 0 || nbc <= 0) { nbr = nbr > 0 ? nbr : 1; nbc = nbc > 0 ? nbc : 1; }
  const int64_t side = morton_side(nbr, nbc);
  if (side > 16384) return false;  // 2^28 bits = 32 MiB of bitmap is the largest grid built here
  const int64_t bits = side * side;
  w->words = (bits + 31) / 32;
  w->chunks = (w->words + kChunkWords - 1) / kChunkWords;
  size_t off = (size_t)w->words * 4;
  off = (off + 255) & ~(size_t)255;
  w->off_prefix = off;
  off += (size_t)(w->words + 1) * 4;
  off = (off + 255) & ~(size_t)255;
  w->off_chunk = off;
  off += (size_t)(w->chunks + 1) * 4;
  off = (off + 255) & ~(size_t)255;
  w->off_counts = off;
  off += 16;
  w->bytes = off;
  return true;
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One warp per tile of the block grid: L1 norm and nonzero count of the tile (elements outside the
// matrix count as the zero padding of void/format.py:374-378); the tile is kept when its norm
// exceeds the threshold (:391-394).
template <typename T>
__global__ void dense_mark_kernel(const T* __restrict__ a, int64_t ld, int M, int N, int nbr, int nbc, float threshold,
                                  uint32_t* __restrict__ bitmap, unsigned long long* __restrict__ counts) {
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (int64_t)nbr * nbc) return;
  const int r = (int)(warp / nbc), c = (int)(warp - (int64_t)r * nbc);
  const int col = c * kTile + lane;
  float norm = 0.0f;
  int nz = 0;
  if (col < N) {
    const int row_end = (r + 1) * kTile < M ? (r + 1) * kTile : M;
    for (int row = r * kTile; row < row_end; ++row) {
      const float v = to_float<T>(a[(size_t)row * ld + col]);
      norm += fabsf(v);
      nz += (v != 0.0f) ? 1 : 0;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    norm += __shfl_xor_sync(0xffffffffu, norm, o);
    nz += __shfl_xor_sync(0xffffffffu, nz, o);
  }
  if (lane == 0) {
    if (nz) atomicAdd(counts + 1, (unsigned long long)nz);
    if (norm > threshold) {
      const uint32_t code = morton((uint32_t)r, (uint32_t)c);
      atomicOr(bitmap + (code >> 5), 1u << (code & 31));
    }
  }
}

// One warp per matrix row of a CSR matrix: every stored entry, zero or not, activates its tile
// (void/format.py:287-296).
__global__ void csr_mark_kernel(const int32_t* __restrict__ crow, const int32_t* __restrict__ col, int M,
                                uint32_t* __restrict__ bitmap) {
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= M) return;
  const int r = (int)warp / kTile;
  uint32_t last = 0xffffffffu;
  for (int i = crow[warp] + lane; i < crow[warp + 1]; i += 32) {
    const uint32_t code = morton((uint32_t)r, (uint32_t)(col[i] / kTile));
    if (code != last) atomicOr(bitmap + (code >> 5), 1u << (code & 31));
    last = code;
  }
}

// Level 1 of the prefix sum: set bits per chunk of kChunkWords words.
__global__ void __launch_bounds__(kChunkWords) chunk_count_kernel(const uint32_t* __restrict__ bitmap, int64_t words,
                                                                  int32_t* __restrict__ chunk_ptr) {
  __shared__ int32_t warp_sum[32];
  const int64_t w = (int64_t)blockIdx.x * kChunkWords + threadIdx.x;
  int c = (w < words) ? __popc(bitmap[w]) : 0;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    int s = warp_sum[threadIdx.x];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) chunk_ptr[blockIdx.x] = s;
  }
}

// Level 2: exclusive scan of the chunk counts by one block; the total is the number of kept tiles.
__global__ void __launch_bounds__(1024) chunk_scan_kernel(int32_t* chunk_ptr, int64_t chunks,
                                                          unsigned long long* __restrict__ counts) {
  __shared__ int32_t part[1024];
  const int tid = threadIdx.x;
  const int64_t per = (chunks + 1023) / 1024;
  const int64_t lo = tid * per < chunks ? tid * per : chunks;
  const int64_t hi = lo + per < chunks ? lo + per : chunks;
  int32_t s = 0;
  for (int64_t i = lo; i < hi; ++i) s += chunk_ptr[i];
  part[tid] = s;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int32_t v = (tid >= off) ? part[tid - off] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  int32_t run = part[tid] - s;
  for (int64_t i = lo; i < hi; ++i) {
    const int32_t v = chunk_ptr[i];
    chunk_ptr[i] = run;
    run += v;
  }
  if (tid == 1023) {
    chunk_ptr[chunks] = part[1023];
    counts[0] = (unsigned long long)part[1023];
  }
}

// Level 3: rank of the first set bit of every word.
__global__ void __launch_bounds__(kChunkWords) word_prefix_kernel(const uint32_t* __restrict__ bitmap, int64_t words,
                                                                  const int32_t* __restrict__ chunk_ptr,
                                                                  int32_t* __restrict__ word_prefix) {
  __shared__ int32_t warp_sum[32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int64_t w = (int64_t)blockIdx.x * kChunkWords + threadIdx.x;
  const int c = (w < words) ? __popc(bitmap[w]) : 0;
  int incl = c;
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_sum[wid] = incl;
  __syncthreads();
  if (wid == 0) {
    int s = warp_sum[lane];
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += v;
    }
    warp_sum[lane] = s;  // inclusive over warps
  }
  __syncthreads();
  const int before = (wid ? warp_sum[wid - 1] : 0) + incl - c;
  if (w < words) word_prefix[w] = chunk_ptr[blockIdx.x] + before;
  if (w == words - 1) word_prefix[words] = chunk_ptr[blockIdx.x] + before + c;
}

// One thread per word: writes block_rows / block_cols / morton_codes of its set bits at their ranks.
__global__ void emit_index_kernel(const uint32_t* __restrict__ bitmap, const int32_t* __restrict__ word_prefix,
                                  int64_t words, int32_t* __restrict__ brow, int32_t* __restrict__ bcol,
                                  int64_t* __restrict__ codes) {
  const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= words) return;
  uint32_t bits = bitmap[w];
  int rank = word_prefix[w];
  while (bits) {
    const int b = __ffs(bits) - 1;
    bits &= bits - 1;
    const uint32_t code = (uint32_t)(w * 32 + b);
    brow[rank] = (int32_t)compact16(code);
    bcol[rank] = (int32_t)compact16(code >> 1);
    codes[rank] = (int64_t)code;
    ++rank;
  }
}

// values[i] = tile (block_rows[i], block_cols[i]) of the dense matrix, zero outside the matrix.
// 128 threads per tile, eight elements each (tile rows e/32, e/32 + 4, ...): eight independent loads in flight
// per thread, every warp reading and writing 128 contiguous bytes per instruction.
template <typename T>
__global__ void dense_gather_kernel(const T* __restrict__ a, int64_t ld, int M, int N,
                                    const int32_t* __restrict__ brow, const int32_t* __restrict__ bcol, int64_t n_blocks,
                                    T* __restrict__ values) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t t = g >> 7;
  if (t >= n_blocks) return;
  const int e0 = (int)(g & 127);
  const int row0 = brow[t] * kTile + (e0 >> 5), col = bcol[t] * kTile + (e0 & 31);
  T v[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int row = row0 + 4 * k;
    v[k] = (row < M && col < N) ? a[(size_t)row * ld + col] : T(0.0f);
  }
  T* dst = values + t * (kTile * kTile) + e0;
#pragma unroll
  for (int k = 0; k < 8; ++k) dst[k * 128] = v[k];
}

// One warp per matrix row of the CSR matrix: every stored entry goes to its place in its tile.
// Two entries with the same coordinates (a non-canonical CSR) race; the reference keeps the later one.
__global__ void csr_scatter_kernel(const int32_t* __restrict__ crow, const int32_t* __restrict__ col,
                                   const float* __restrict__ data, int M, const uint32_t* __restrict__ bitmap,
                                   const int32_t* __restrict__ word_prefix, float* __restrict__ values) {
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= M) return;
  const int r = (int)warp / kTile, rr = (int)warp % kTile;
  for (int i = crow[warp] + lane; i < crow[warp + 1]; i += 32) {
    const int c = col[i];
    const uint32_t code = morton((uint32_t)r, (uint32_t)(c / kTile));
    const int rank = word_prefix[code >> 5] + __popc(bitmap[code >> 5] & ((1u << (code & 31)) - 1u));
    values[(size_t)rank * (kTile * kTile) + rr * kTile + (c % kTile)] = data[i];
  }
}

static int rank_bitmap(const WsLayout& w, unsigned char* ws, cudaStream_t st) {
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(ws);
  int32_t* word_prefix = reinterpret_cast<int32_t*>(ws + w.off_prefix);
  int32_t* chunk_ptr = reinterpret_cast<int32_t*>(ws + w.off_chunk);
  unsigned long long* counts = reinterpret_cast<unsigned long long*>(ws + w.off_counts);
  chunk_count_kernel<<<(unsigned)w.chunks, kChunkWords, 0, st>>>(bitmap, w.words, chunk_ptr);
  chunk_scan_kernel<<<1, 1024, 0, st>>>(chunk_ptr, w.chunks, counts);
  word_prefix_kernel<<<(unsigned)w.chunks, kChunkWords, 0, st>>>(bitmap, w.words, chunk_ptr, word_prefix);
  return last_status();
}

}  // namespace vbf

extern "C" {

size_t void_format_ws_bytes(int32_t nbr, int32_t nbc) {
  vbf::WsLayout w;
  return vbf::ws_layout(nbr, nbc, &w) ? w.bytes : 0;
}

int void_dense_mark(const void* matrix, int32_t elem, int64_t ld, int32_t M, int32_t N, float threshold, void* ws,
                    size_t ws_bytes, int64_t* counts_out, void_stream_t stream) {
  if (M < 0 || N < 0 || ld < N || counts_out == nullptr) return VOID_ERR_BAD_ARG;
  if (elem < VOID_ELEM_F32 || elem > VOID_ELEM_BF16) return VOID_ERR_BAD_ARG;
  const int nbr = (M + vbf::kTile - 1) / vbf::kTile, nbc = (N + vbf::kTile - 1) / vbf::kTile;
  vbf::WsLayout w;
  if (!vbf::ws_layout(nbr, nbc, &w)) return VOID_ERR_TOO_LARGE;
  if (ws == nullptr || ws_bytes < w.bytes) return VOID_ERR_WORKSPACE;
  if ((int64_t)nbr * nbc > 0 && matrix == nullptr) return VOID_ERR_BAD_ARG;
  cudaStream_t st = vbf::as_stream(stream);
  unsigned char* base = static_cast<unsigned char*>(ws);
  if (cudaMemsetAsync(base, 0, (size_t)w.words * 4, st) != cudaSuccess) return VOID_ERR_CUDA;
  if (cudaMemsetAsync(base + w.off_counts, 0, 16, st) != cudaSuccess) return VOID_ERR_CUDA;
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(base);
  unsigned long long* counts = reinterpret_cast<unsigned long long*>(base + w.off_counts);
  const int64_t tiles = (int64_t)nbr * nbc;
  if (tiles > 0) {
    const int tb = 256;
    const unsigned blocks = (unsigned)((tiles * 32 + tb - 1) / tb);
    if (elem == VOID_ELEM_F32)
      vbf::dense_mark_kernel<float><<<blocks, tb, 0, st>>>(static_cast<const float*>(matrix), ld, M, N, nbr, nbc,
                                                            threshold, bitmap, counts);
    else if (elem == VOID_ELEM_F16)
      vbf::dense_mark_kernel<__half><<<blocks, tb, 0, st>>>(static_cast<const __half*>(matrix), ld, M, N, nbr, nbc,
                                                             threshold, bitmap, counts);
    else
      vbf::dense_mark_kernel<__nv_bfloat16><<<blocks, tb, 0, st>>>(static_cast<const __nv_bfloat16*>(matrix), ld, M, N,
                                                                    nbr, nbc, threshold, bitmap, counts);
  }
  const int rc = vbf::rank_bitmap(w, base, st);
  if (rc != VOID_OK) return rc;
  if (cudaMemcpyAsync(counts_out, counts, 16, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return VOID_ERR_CUDA;
  return vbf::last_status();
}

int void_csr_mark(const int32_t* crow, const int32_t* col, int32_t M, int32_t N, void* ws, size_t ws_bytes,
                  int64_t* counts_out, void_stream_t stream) {
  if (M < 0 || N < 0 || counts_out == nullptr) return VOID_ERR_BAD_ARG;
  const int nbr = (M + vbf::kTile - 1) / vbf::kTile, nbc = (N + vbf::kTile - 1) / vbf::kTile;
  vbf::WsLayout w;
  if (!vbf::ws_layout(nbr, nbc, &w)) return VOID_ERR_TOO_LARGE;
  if (ws == nullptr || ws_bytes < w.bytes) return VOID_ERR_WORKSPACE;
  if (M > 0 && crow == nullptr) return VOID_ERR_BAD_ARG;  // col may be null for a matrix without entries
  cudaStream_t st = vbf::as_stream(stream);
  unsigned char* base = static_cast<unsigned char*>(ws);
  if (cudaMemsetAsync(base, 0, (size_t)w.words * 4, st) != cudaSuccess) return VOID_ERR_CUDA;
  if (cudaMemsetAsync(base + w.off_counts, 0, 16, st) != cudaSuccess) return VOID_ERR_CUDA;
  if (M > 0) {
    const int tb = 256;
    vbf::csr_mark_kernel<<<(unsigned)(((int64_t)M * 32 + tb - 1) / tb), tb, 0, st>>>(
        crow, col, M, reinterpret_cast<uint32_t*>(base));
  }
  const int rc = vbf::rank_bitmap(w, base, st);
  if (rc != VOID_OK) return rc;
  if (cudaMemcpyAsync(counts_out, base + w.off_counts, 16, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
    return VOID_ERR_CUDA;
  return vbf::last_status();
}

int void_morton_emit(const void* ws, int32_t nbr, int32_t nbc, int64_t n_blocks, int32_t* block_rows,
                     int32_t* block_cols, int64_t* morton_codes, void_stream_t stream) {
  vbf::WsLayout w;
  if (!vbf::ws_layout(nbr, nbc, &w)) return VOID_ERR_TOO_LARGE;
  if (n_blocks < 0 || ws == nullptr) return VOID_ERR_BAD_ARG;
  if (n_blocks == 0) return VOID_OK;
  if (block_rows == nullptr || block_cols == nullptr || morton_codes == nullptr) return VOID_ERR_BAD_ARG;
  const unsigned char* base = static_cast<const unsigned char*>(ws);
  const int tb = 256;
  vbf::emit_index_kernel<<<(unsigned)((w.words + tb - 1) / tb), tb, 0, vbf::as_stream(stream)>>>(
      reinterpret_cast<const uint32_t*>(base), reinterpret_cast<const int32_t*>(base + w.off_prefix), w.words,
      block_rows, block_cols, morton_codes);
  return vbf::last_status();
}

int void_dense_gather(const void* matrix, int32_t elem, int64_t ld, int32_t M, int32_t N, const int32_t* block_rows,
                      const int32_t* block_cols, int64_t n_blocks, void* values, void_stream_t stream) {
  if (n_blocks < 0 || M < 0 || N < 0 || ld < N) return VOID_ERR_BAD_ARG;
  if (elem < VOID_ELEM_F32 || elem > VOID_ELEM_BF16) return VOID_ERR_BAD_ARG;
  if (n_blocks == 0) return VOID_OK;
  if (matrix == nullptr || block_rows == nullptr || block_cols == nullptr || values == nullptr) return VOID_ERR_BAD_ARG;
  cudaStream_t st = vbf::as_stream(stream);
  const int tb = 256;
  const unsigned blocks = (unsigned)((n_blocks * 128 + tb - 1) / tb);
  if (elem == VOID_ELEM_F32)
    vbf::dense_gather_kernel<float><<<blocks, tb, 0, st>>>(static_cast<const float*>(matrix), ld, M, N, block_rows,
                                                            block_cols, n_blocks, static_cast<float*>(values));
  else if (elem == VOID_ELEM_F16)
    vbf::dense_gather_kernel<__half><<<blocks, tb, 0, st>>>(static_cast<const __half*>(matrix), ld, M, N, block_rows,
                                                             block_cols, n_blocks, static_cast<__half*>(values));
  else
    vbf::dense_gather_kernel<__nv_bfloat16><<<blocks, tb, 0, st>>>(static_cast<const __nv_bfloat16*>(matrix), ld, M, N,
                                                                    block_rows, block_cols, n_blocks,
                                                                    static_cast<__nv_bfloat16*>(values));
  return vbf::last_status();
}

int void_csr_scatter(const int32_t* crow, const int32_t* col, const float* data, int32_t M, int32_t N, const void* ws,
                     int64_t n_blocks, float* values, void_stream_t stream) {
  if (M < 0 || N < 0 || n_blocks < 0) return VOID_ERR_BAD_ARG;
  if (n_blocks == 0 || M == 0) return VOID_OK;
  if (crow == nullptr || col == nullptr || data == nullptr || ws == nullptr || values == nullptr) return VOID_ERR_BAD_ARG;
  const int nbr = (M + vbf::kTile - 1) / vbf::kTile, nbc = (N + vbf::kTile - 1) / vbf::kTile;
  vbf::WsLayout w;
  if (!vbf::ws_layout(nbr, nbc, &w)) return VOID_ERR_TOO_LARGE;
  cudaStream_t st = vbf::as_stream(stream);
  if (cudaMemsetAsync(values, 0, (size_t)n_blocks * 4096, st) != cudaSuccess) return VOID_ERR_CUDA;
  const unsigned char* base = static_cast<const unsigned char*>(ws);
  const int tb = 256;
  vbf::csr_scatter_kernel<<<(unsigned)(((int64_t)M * 32 + tb - 1) / tb), tb, 0, st>>>(
      crow, col, data, M, reinterpret_cast<const uint32_t*>(base), reinterpret_cast<const int32_t*>(base + w.off_prefix),
      values);
  return vbf::last_status();
}

}  // extern "C"
