// Gradient of the floating-point SpMM with respect to the stored tiles of A:
//
//     dA_tile(br, bc) = dC[32 br : 32 br + 32, :] . B[32 bc : 32 bc + 32, :]^T          (32 x N) . (N x 32)
//
// for every stored tile only - the backward-A kernel of the reference, void_spmm_backward_a_kernel,
// void/autograd.py:14-96 (one Triton program per tile, fp32 accumulation over N in steps of TILE_N).
//
// Here up to four tiles of one tile row share their dC rows in one tcgen05.mma:
//
//     D[(j, k), m] += sum_n  B[32 bc_j + k, n] * dC[32 br + m, n]         j < 4, k < 32, m < 32
//
// Instruction operand A (M = 128) = the B row blocks of the four tiles stacked, operand B (N = 32) =
// the dC row block; both have the reduction index n contiguous in memory, i.e. both are K-major
// operands with the ordinary 128-byte swizzle, loaded by 2-D TMA boxes of 32 rows x 128 bytes.  One
// ring stage holds one 128-byte slice of n for the five row blocks (20 KB) and feeds four MMAs
// (32 bytes of n each).  The accumulator (128 lanes x 32 columns of fp32, double-buffered in tensor
// memory) is read back by four warps, warp j holding tile j: lane k, column m = dA_tile_j[m][k], so
// every store instruction writes 32 consecutive elements of one tile row.
//
// Work items (tile row, first tile, tile count <= 4) come from the caller (they depend on A's
// structure only).  Every wait is bounded like in the SpMM kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "../../include/void_b200.h"
#include "ptx.cuh"

namespace vbg {

using namespace vb;

constexpr int kTile = 32;
constexpr int kBlockBytes = 4096;          // 32 rows x 128 bytes: one row block, one slice of n
constexpr int kStageBytes = 5 * kBlockBytes;
constexpr int kStages = 4;
constexpr int kThreads = 32 * 6;           // producer, MMA, four epilogue warps
constexpr int kMaxBars = 8;

struct GradParams {
  const int32_t* items;          // [n_items][4]: tile row, first packed tile, tile count, unused
  const int32_t* tile_cols;      // [nnz] block column of every packed tile
  const int32_t* block_indices;  // [nnz] packed position -> index of the tile in the caller's order
  void* grad;                    // [nnz][32][32] in the caller's order
  int32_t* status;
  int n_items;
  int n_slices;                  // ceil(N * element bytes / 128)
  int slice_elems;               // elements per 128 bytes
  int out_dtype;
  unsigned long long desc_hi;
  unsigned int idesc;
};

struct __align__(8) Bars {
  uint64_t full[kMaxBars];
  uint64_t empty[kMaxBars];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
};

template <int KIND>
__device__ __forceinline__ void issue(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if (KIND == VOID_KIND_TF32) mma_tf32(d, a, b, idesc, acc);
  else mma_f16(d, a, b, idesc, acc);
}

template <int KIND>
__global__ void __launch_bounds__(kThreads, 2) tile_grad_kernel(const __grid_constant__ CUtensorMap tmap_b,
                                                                const __grid_constant__ CUtensorMap tmap_g,
                                                                const __grid_constant__ GradParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Bars bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s[2];   // abort flag, wait limit in ms

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abort_flag = abort_s;
  constexpr uint32_t kTmemCols = 64;  // two accumulators of 32 columns

  if (threadIdx.x == 0) {
    abort_s[0] = 0;
    abort_s[1] = kDefaultWaitLimitMs;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars.acc_full[b]), 1);
      mbar_init(smem_u32(&bars.acc_empty[b]), 4);
    }
    fence_mbar_init();
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_g);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // producer: lanes 0..3 fetch the B row blocks of the item's tiles, lane 4 the dC row block
    uint32_t g = 0;
    bool alive = true;
    for (int i = blockIdx.x; i < p.n_items && alive; i += gridDim.x) {
      const int4 it = __ldg(reinterpret_cast<const int4*>(p.items) + i);
      const int row = it.x, t0 = it.y, cnt = it.z;
      int y = 0;
      if (lane < cnt) y = __ldg(p.tile_cols + t0 + lane) * kTile;
      if (lane == 4) y = row * kTile;
      const bool mine = lane < cnt || lane == 4;
      for (int s = 0; s < p.n_slices; ++s, ++g) {
        const int stage = (int)(g % kStages);
        const uint32_t phase = (g / kStages) & 1u;
        const uint32_t full = smem_u32(&bars.full[stage]);
        const uint32_t base = ring + (uint32_t)stage * kStageBytes;
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&bars.empty[stage]), phase ^ 1u, abort_flag) ? 1 : 0;
          if (ok) mbar_expect_tx(full, (uint32_t)(cnt + 1) * kBlockBytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { alive = false; break; }
        if (mine) tma_load_2d(base + (uint32_t)lane * kBlockBytes, lane == 4 ? &tmap_g : &tmap_b, s * p.slice_elems, y, full);
      }
    }
  } else if (warp == 1) {
    {
      // the warp walks the loop and waits together, one elected lane issues the MMAs and commits: the loop
      // stays convergent, so descriptors and addresses can live in the warp's uniform registers
      const bool leader = elect_one();
      const uint32_t idesc = p.idesc;
      const uint64_t hi = p.desc_hi;
      uint32_t g = 0, n = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < p.n_items && ok; i += gridDim.x, ++n) {
        const uint32_t buf = n & 1u, aph = (n >> 1) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.acc_empty[buf]), aph ^ 1u, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d = tmem_base + buf * 32u;
        uint32_t acc = 0u;
        for (int s = 0; s < p.n_slices; ++s, ++g) {
          const int stage = (int)(g % kStages);
          const uint32_t phase = (g / kStages) & 1u;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[stage]), phase, abort_flag));
          if (!ok) break;
          tc_fence_after();
          const uint32_t base = ring + (uint32_t)stage * kStageBytes;
          const uint64_t ad = smem_desc(hi, base), bd = smem_desc(hi, base + 4u * kBlockBytes);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {  // 32 bytes of n per MMA: the start address moves inside the swizzle atom
            if (leader) issue<KIND>(d, ad + 2u * kk, bd + 2u * kk, idesc, acc);
            acc = 1u;
          }
          if (leader) tc_commit(smem_u32(&bars.empty[stage]));
        }
        if (!ok) break;
        if (leader) {
          if (p.n_slices > 0) tc_commit(smem_u32(&bars.acc_full[buf]));
          else mbar_arrive(smem_u32(&bars.acc_full[buf]));
        }
      }
    }
    __syncwarp();
  } else {
    // epilogue warp: TMEM lane quadrant = warp id mod 4 = tile j of the item
    const int j = warp & 3;
    const uint32_t lane_sel = (uint32_t)(j * 32) << 16;
    uint32_t n = 0;
    for (int i = blockIdx.x; i < p.n_items; i += gridDim.x, ++n) {
      const int4 it = __ldg(reinterpret_cast<const int4*>(p.items) + i);
      const int t0 = it.y, cnt = it.z;
      const uint32_t buf = n & 1u, aph = (n >> 1) & 1u;
      long long orig = 0;
      if (j < cnt) orig = __ldg(p.block_indices + t0 + j);
      int ok = 1;
      if (lane == 0) ok = mbar_wait(smem_u32(&bars.acc_full[buf]), aph, abort_flag) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      uint32_t r[32];
      if (j < cnt && p.n_slices > 0) {
        tmem_ld_32x32(tmem_base + lane_sel + buf * 32u, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int m = 0; m < 32; ++m) r[m] = 0u;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty[buf]));
      if (j < cnt) {
        const size_t first = (size_t)orig * (kTile * kTile) + lane;   // element [m][k = lane]
        if (p.out_dtype == VOID_OUT_F32) {
          float* dst = reinterpret_cast<float*>(p.grad) + first;
#pragma unroll
          for (int m = 0; m < 32; ++m) dst[m * kTile] = __uint_as_float(r[m]);
        } else if (p.out_dtype == VOID_OUT_F16) {
          __half* dst = reinterpret_cast<__half*>(p.grad) + first;
#pragma unroll
          for (int m = 0; m < 32; ++m) dst[m * kTile] = __float2half_rn(__uint_as_float(r[m]));
        } else {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.grad) + first;
#pragma unroll
          for (int m = 0; m < 32; ++m) dst[m * kTile] = __float2bfloat16_rn(__uint_as_float(r[m]));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (abort_s[0]) {
    const uint64_t t0 = globaltimer_ns();  // let copies still in flight land before shared memory is given back
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, 1);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

static PFN_cuTensorMapEncodeTiled_v12000 encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(f);
  });
  return fn;
}

// [rows, N] row-major matrix as a tensor of 128-byte-wide, 32-row boxes with the 128-byte swizzle.
static bool row_block_map(CUtensorMap* m, const void* base, int64_t ld_bytes, int rows, int N, int es) {
  PFN_cuTensorMapEncodeTiled_v12000 enc = encoder();
  if (enc == nullptr) return false;
  const CUtensorMapDataType dt = (es == 2) ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  const cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)ld_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / es), (cuuint32_t)kTile};
  const cuuint32_t estride[2] = {1, 1};
  return enc(m, dt, 2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace vbg

extern "C" int void_spmm_tile_grad(const void* grad_out, int64_t ldg, const void* b, int64_t ldb, int32_t M, int32_t K,
                                   int32_t N, int32_t kind, const int32_t* items, int32_t n_items,
                                   const int32_t* tile_cols, const int32_t* block_indices, void* grad_tiles,
                                   int32_t out_dtype, int32_t* status, void_stream_t stream) {
  using namespace vbg;
  if (M < 0 || K < 0 || N < 0 || n_items < 0) return VOID_ERR_BAD_ARG;
  if (kind != VOID_KIND_TF32 && kind != VOID_KIND_F16 && kind != VOID_KIND_BF16) return VOID_ERR_BAD_ARG;
  if (out_dtype < VOID_OUT_F32 || out_dtype > VOID_OUT_BF16) return VOID_ERR_BAD_ARG;
  if (n_items == 0) return VOID_OK;
  if (items == nullptr || tile_cols == nullptr || block_indices == nullptr || grad_tiles == nullptr) return VOID_ERR_BAD_ARG;
  const int es = (kind == VOID_KIND_TF32) ? 4 : 2;
  if (N > 0) {
    if (grad_out == nullptr || b == nullptr) return VOID_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(grad_out) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u) || (ldg & 15) || (ldb & 15) ||
        ldg < (int64_t)N * es || ldb < (int64_t)N * es)
      return VOID_ERR_ALIGN;
  }
  int dev = 0, cc = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return VOID_ERR_CUDA;
  cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cc != 10) return VOID_ERR_ARCH;

  GradParams p;
  p.items = items;
  p.tile_cols = tile_cols;
  p.block_indices = block_indices;
  p.grad = grad_tiles;
  p.status = status;
  p.n_items = n_items;
  p.slice_elems = 128 / es;
  p.n_slices = (N + p.slice_elems - 1) / p.slice_elems;
  p.out_dtype = out_dtype;
  // K-major operands with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
  p.desc_hi = smem_desc_hi(16, 1024, kLayoutSw128);
  const uint32_t fmt = (kind == VOID_KIND_TF32) ? 2u : (kind == VOID_KIND_BF16 ? 1u : 0u);
  p.idesc = instr_desc(/*c f32*/ 1, fmt, fmt, /*a K-major*/ 0, /*b K-major*/ 0, 128, 32);

  CUtensorMap map_b, map_g;
  memset(&map_b, 0, sizeof(map_b));
  memset(&map_g, 0, sizeof(map_g));
  if (N > 0) {
    if (!row_block_map(&map_b, b, ldb, K, N, es) || !row_block_map(&map_g, grad_out, ldg, M, N, es))
      return VOID_ERR_TENSOR_MAP;
  }
  const int smem = kStages * kStageBytes + 1024;
  int grid = 2 * sms;
  if (grid > n_items) grid = n_items;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (kind == VOID_KIND_TF32) {
      if (cudaFuncSetAttribute(tile_grad_kernel<VOID_KIND_TF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return VOID_ERR_CUDA;
    } else {
      if (cudaFuncSetAttribute(tile_grad_kernel<VOID_KIND_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return VOID_ERR_CUDA;
    }
  }
  if (kind == VOID_KIND_TF32) tile_grad_kernel<VOID_KIND_TF32><<<grid, kThreads, smem, st>>>(map_b, map_g, p);
  else tile_grad_kernel<VOID_KIND_F16><<<grid, kThreads, smem, st>>>(map_b, map_g, p);
  return cudaGetLastError() == cudaSuccess ? VOID_OK : VOID_ERR_CUDA;
}
