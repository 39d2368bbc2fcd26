// Quantized block-sparse SpMM for B200 (sm_100a):  C = act(dequant(A_q . B_q) + bias).
//
// A is the packed VOID tensor (tile-row-major 32x32 8-bit tiles, each stored as 8x16-byte
// core matrices), B is a row-major [K, N] 8-bit matrix.  The product is computed transposed
// on the tensor cores so that the 32-row tile sits in the N slot of the instruction:
//
//     D[n, m] (+)= sum_k  B[kcol*32 + k, n0 + n] * A_tile[m, k]        n < 128, m < 32, k < 32
//
// i.e. one tcgen05.mma (M=128, N=32, K=32) per (tile, 128-column panel of B).  The "A"
// operand of the instruction is the B panel exactly as it lies in memory (n contiguous:
// MN-major, 128-byte swizzle, written by a 2-D TMA load); the "B" operand is the packed tile
// (K-major, no swizzle, written by a linear bulk copy).  Accumulators live in tensor memory:
// lane = output column n, column = tile row m.
//
// Warp roles in a 192-thread CTA: warp 0 streams tiles and panels into a shared-memory ring,
// warp 1 issues the MMAs, warps 2..5 read accumulators back (each warp owns the 32 TMEM lanes
// of its quadrant), apply scales / bias / activation and store C.
//
// Two kernels share this pipeline:
//   spmm_rowacc_kernel  one accumulator per (tile row, column chunk), scaled once by the
//                       row's mean tile scale (the INT8 semantic of void/int_quant.py:479-526);
//                       rows cut into several segments by a work plan are finished by the
//                       CTA that arrives last.
//   spmm_drain_kernel   every tile's product lands in its own TMEM slot and is folded into
//                       registers with that tile's scale (the FP8 semantic of
//                       void/fp8.py:638-659; also exact per-block INT8 dequantisation).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "../../include/void_b200.h"
#include "ptx.cuh"

namespace vb {

constexpr int kTile = 32;
constexpr int kTileBytes = 1024;
constexpr int kPanelN = 128;
constexpr int kPanelBytes = kTile * kPanelN;  // 4096
constexpr int kMaxStages = 16;
constexpr int kMaxSlots = 16;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;

// device status codes (written to the status word)
constexpr int kStatusTimeout = 1;

struct SpmmParams {
  const uint8_t* tiles;
  const int32_t* tile_cols;
  const float* tile_scales;
  const int32_t* row_ptr;
  const float* row_scale;
  int nbr, n_chunks, N, M;
  const float* col_scale;
  float b_scale;
  const float* bias;
  void* out;
  long long ldc;
  int out_dtype, act;
  void* acc_out;
  const int32_t* segs;
  const int32_t* cta_seg_ptr;
  int32_t* partials;
  int32_t* counters;
  int32_t* worker_partials;
  int32_t* status;
  int np;      // panels per work item
  int stages;  // ring depth
  int n_items; // without a plan: nbr * n_chunks
  unsigned long long desc_hi_a;  // B panel  (instruction operand A: MN-major, 128B swizzle)
  unsigned long long desc_hi_b;  // A tile   (instruction operand B: K-major, no swizzle)
  unsigned int idesc;
};

struct Seg {
  int row, chunk, t0, t1, nseg, slot0, my_idx, ctr;
};

__device__ __forceinline__ Seg load_seg(const SpmmParams& p, int i) {
  Seg s;
  if (p.segs != nullptr) {
    const int4* q = reinterpret_cast<const int4*>(p.segs) + 2 * (size_t)i;
    const int4 a = __ldg(q), b = __ldg(q + 1);
    s.row = a.x; s.chunk = a.y; s.t0 = a.z; s.t1 = a.w;
    s.nseg = b.x; s.slot0 = b.y; s.my_idx = b.z; s.ctr = b.w;
  } else {
    s.row = i / p.n_chunks;
    s.chunk = i - s.row * p.n_chunks;
    s.t0 = __ldg(p.row_ptr + s.row);
    s.t1 = __ldg(p.row_ptr + s.row + 1);
    s.nseg = 1; s.slot0 = 0; s.my_idx = 0; s.ctr = 0;
  }
  return s;
}

// Range of segment indices of this CTA: [begin, end) with stride step.
__device__ __forceinline__ void seg_range(const SpmmParams& p, int& begin, int& end, int& step) {
  if (p.segs != nullptr) {
    begin = __ldg(p.cta_seg_ptr + blockIdx.x);
    end = __ldg(p.cta_seg_ptr + blockIdx.x + 1);
    step = 1;
  } else {
    begin = blockIdx.x;
    end = p.n_items;
    step = gridDim.x;
  }
}

__device__ __forceinline__ int panels_in_chunk(const SpmmParams& p, int chunk) {
  const int total = (p.N + kPanelN - 1) / kPanelN;
  const int left = total - chunk * p.np;
  return left < p.np ? left : p.np;
}

// GELU in the tanh form written with a sigmoid, void/fusion.py:38-43.
__device__ __forceinline__ float gelu_tanh_sigmoid(float x) {
  const float inner = 0.7978845608f * (x + 0.044715f * x * x * x);
  const float sig = 1.0f / (1.0f + expf(-2.0f * inner));
  const float t = 2.0f * sig - 1.0f;
  return x * 0.5f * (1.0f + t);
}
__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case VOID_ACT_RELU: return fmaxf(x, 0.0f);
    case VOID_ACT_GELU: return gelu_tanh_sigmoid(x);
    case VOID_ACT_SILU: return x * (1.0f / (1.0f + expf(-x)));
    default: return x;
  }
}

// Store 32 finished values of one output column n (tile rows m = 0..31 of tile row `row`).
__device__ __forceinline__ void store_column(const SpmmParams& p, int row, int n, const float (&v)[32]) {
  if (n >= p.N) return;
  const int r0 = row * kTile;
  const int rows = (p.M - r0) < kTile ? (p.M - r0) : kTile;
  if (p.out_dtype == VOID_OUT_F16) {
    __half* o = reinterpret_cast<__half*>(p.out) + (size_t)r0 * p.ldc + n;
#pragma unroll
    for (int m = 0; m < 32; ++m)
      if (m < rows) o[(size_t)m * p.ldc] = __float2half_rn(v[m]);
  } else if (p.out_dtype == VOID_OUT_BF16) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)r0 * p.ldc + n;
#pragma unroll
    for (int m = 0; m < 32; ++m)
      if (m < rows) o[(size_t)m * p.ldc] = __float2bfloat16_rn(v[m]);
  } else {
    float* o = reinterpret_cast<float*>(p.out) + (size_t)r0 * p.ldc + n;
#pragma unroll
    for (int m = 0; m < 32; ++m)
      if (m < rows) o[(size_t)m * p.ldc] = v[m];
  }
}

// Epilogue of one output column: raw accumulators -> dequantised, biased, activated values.
template <int KIND>
__device__ __forceinline__ void finish_column(const SpmmParams& p, int row, int n, const uint32_t (&r)[32],
                                              float row_scale) {
  if (n >= p.N) return;
  if (p.acc_out != nullptr) {
    uint32_t* a = reinterpret_cast<uint32_t*>(p.acc_out) + (size_t)row * kTile * p.N + n;
#pragma unroll
    for (int m = 0; m < 32; ++m) a[(size_t)m * p.N] = r[m];
  }
  const float cs = (p.col_scale != nullptr) ? __ldg(p.col_scale + n) * p.b_scale : p.b_scale;
  const float bias = (p.bias != nullptr) ? __ldg(p.bias + n) : 0.0f;
  float v[32];
#pragma unroll
  for (int m = 0; m < 32; ++m) {
    const float x = (KIND == VOID_KIND_I8) ? __int2float_rn((int)r[m]) : __uint_as_float(r[m]);
    v[m] = apply_act((x * row_scale) * cs + bias, p.act);
  }
  store_column(p, row, n, v);
}

struct __align__(8) PipeBars {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[kMaxSlots];
  uint64_t acc_empty[kMaxSlots];
};

// warp 0: stream (tile, panels) units of this CTA's segments into the ring.
__device__ __forceinline__ void producer_loop(const SpmmParams& p, const CUtensorMap* tmap, PipeBars* bars,
                                              uint32_t ring_base, uint32_t stage_bytes, volatile int* abort_flag,
                                              int lane) {
  int begin, end, step;
  seg_range(p, begin, end, step);
  int stage = 0;
  uint32_t phase = 0;
  for (int i = begin; i < end; i += step) {
    const Seg s = load_seg(p, i);
    const int npan = panels_in_chunk(p, s.chunk);
    const int n0 = s.chunk * p.np * kPanelN;
    for (int tb = s.t0; tb < s.t1; tb += 32) {
      const int cnt = (s.t1 - tb) < 32 ? (s.t1 - tb) : 32;
      const int my_col = (lane < cnt) ? __ldg(p.tile_cols + tb + lane) : 0;
      for (int j = 0; j < cnt; ++j) {
        const int col = __shfl_sync(0xffffffffu, my_col, j);
        int ok = 1;
        if (lane == 0) ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return;
        if (lane == 0) {
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sbase = ring_base + (uint32_t)stage * stage_bytes;
          mbar_expect_tx(full, (uint32_t)(kTileBytes + npan * kPanelBytes));
          bulk_load(sbase + (uint32_t)p.np * kPanelBytes, p.tiles + (size_t)(tb + j) * kTileBytes, kTileBytes, full);
          for (int q = 0; q < npan; ++q)
            tma_load_2d(sbase + (uint32_t)q * kPanelBytes, tmap, n0 + q * kPanelN, col * kTile, full);
        }
        if (++stage == p.stages) { stage = 0; phase ^= 1u; }
      }
    }
  }
}

template <int KIND>
__device__ __forceinline__ void issue_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if (KIND == VOID_KIND_I8) mma_i8(d, a, b, idesc, acc);
  else mma_f8(d, a, b, idesc, acc);
}

// ------------------------------------------------------------------------------------------
// Row-accumulate kernel.
// ------------------------------------------------------------------------------------------
template <int KIND>
__global__ void __launch_bounds__(kThreads) spmm_rowacc_kernel(const __grid_constant__ CUtensorMap tmap_b,
                                                               const SpmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ PipeBars bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int last_s;
  __shared__ int ok_s[2];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t ring_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_bytes = (uint32_t)(p.np * kPanelBytes + kTileBytes);
  const uint32_t acc_cols = (uint32_t)p.np * 32u;  // TMEM columns of one accumulator buffer
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2u * acc_cols) tmem_cols <<= 1;
  volatile int* abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    last_s = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars.acc_full[b]), 1);
      mbar_init(smem_u32(&bars.acc_empty[b]), 4);
    }
    fence_mbar_init();
    if (p.tiles != nullptr) prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    producer_loop(p, &tmap_b, &bars, ring_base, stage_bytes, abort_flag, lane);
  } else if (warp == 1) {
    if (lane == 0) {
      int begin, end, step;
      seg_range(p, begin, end, step);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int i = begin; i < end && ok; i += step, ++it) {
        const Seg s = load_seg(p, i);
        const int npan = panels_in_chunk(p, s.chunk);
        const uint32_t buf = it & 1u, aph = (it >> 1) & 1u;
        ok = mbar_wait(smem_u32(&bars.acc_empty[buf]), aph ^ 1u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * acc_cols;
        for (int t = s.t0; t < s.t1; ++t) {
          ok = mbar_wait(smem_u32(&bars.full[stage]), phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sbase = ring_base + (uint32_t)stage * stage_bytes;
          const uint64_t bdesc = smem_desc(p.desc_hi_b, sbase + (uint32_t)p.np * kPanelBytes);
          for (int q = 0; q < npan; ++q) {
            const uint64_t adesc = smem_desc(p.desc_hi_a, sbase + (uint32_t)q * kPanelBytes);
            issue_mma<KIND>(d0 + (uint32_t)q * 32u, adesc, bdesc, p.idesc, t > s.t0 ? 1u : 0u);
          }
          tc_commit(smem_u32(&bars.empty[stage]));
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (s.t1 > s.t0) tc_commit(smem_u32(&bars.acc_full[buf]));
        else mbar_arrive(smem_u32(&bars.acc_full[buf]));
      }
    }
    __syncwarp();
  } else {
    // epilogue warps 2..5; TMEM lane quadrant = warp id mod 4
    const int quad = warp & 3;
    const int epi_tid = (int)threadIdx.x - 64;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    int begin, end, step;
    seg_range(p, begin, end, step);
    uint32_t it = 0;
    for (int i = begin; i < end; i += step, ++it) {
      const Seg s = load_seg(p, i);
      const int npan = panels_in_chunk(p, s.chunk);
      const uint32_t buf = it & 1u, aph = (it >> 1) & 1u;
      const bool has = s.t1 > s.t0;
      const float rs = (p.row_scale != nullptr) ? __ldg(p.row_scale + s.row) : 1.0f;
      // one thread waits, the named barrier hands its verdict to all four epilogue warps, so
      // that they leave the loop together if the wait gave up
      if (epi_tid == 0) ok_s[it & 1u] = mbar_wait(smem_u32(&bars.acc_full[buf]), aph, abort_flag) ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!ok_s[it & 1u]) break;
      tc_fence_after();
      const int n_base = s.chunk * p.np * kPanelN + quad * 32 + lane;
      for (int q = 0; q < npan; ++q) {
        uint32_t r[32];
        if (has) {
          tmem_ld_32x32(tmem_base + lane_sel + buf * acc_cols + (uint32_t)q * 32u, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int m = 0; m < 32; ++m) r[m] = 0u;
        }
        if (q == npan - 1) {  // accumulator buffer is free again
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty[buf]));
        }
        const int n = n_base + q * kPanelN;
        if (p.worker_partials != nullptr && n < p.N) {
          uint32_t* w = reinterpret_cast<uint32_t*>(p.worker_partials) + ((size_t)i * kTile) * p.N + n;
#pragma unroll
          for (int m = 0; m < 32; ++m) w[(size_t)m * p.N] = r[m];
        }
        if (s.nseg == 1) {
          finish_column<KIND>(p, s.row, n, r, rs);
        } else {
          // partial sum of a split row: park it, 128 contiguous bytes per thread
          uint4* dst = reinterpret_cast<uint4*>(p.partials) +
                       (((size_t)(s.slot0 + s.my_idx) * p.np + q) * kPanelN + (quad * 32 + lane)) * 8;
#pragma unroll
          for (int c = 0; c < 8; ++c) dst[c] = make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
        }
      }
      if (s.nseg > 1) {
        // the CTA that arrives last adds the parked partial sums and finishes the row
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (epi_tid == 0) {
          const int old = atomicAdd(p.counters + s.ctr, 1);
          const int last = (old == s.nseg - 1) ? 1 : 0;
          if (last) p.counters[s.ctr] = 0;  // left clean for the next launch
          last_s = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int last = last_s;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (last) {
          __threadfence();
          for (int q = 0; q < npan; ++q) {
            uint32_t r[32];
#pragma unroll
            for (int m = 0; m < 32; ++m) r[m] = 0u;
            for (int j = 0; j < s.nseg; ++j) {
              const uint4* src = reinterpret_cast<const uint4*>(p.partials) +
                                 (((size_t)(s.slot0 + j) * p.np + q) * kPanelN + (quad * 32 + lane)) * 8;
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                const uint4 v = __ldcg(src + c);
                if (KIND == VOID_KIND_I8) {
                  r[4 * c] += v.x; r[4 * c + 1] += v.y; r[4 * c + 2] += v.z; r[4 * c + 3] += v.w;
                } else {
                  r[4 * c] = __float_as_uint(__uint_as_float(r[4 * c]) + __uint_as_float(v.x));
                  r[4 * c + 1] = __float_as_uint(__uint_as_float(r[4 * c + 1]) + __uint_as_float(v.y));
                  r[4 * c + 2] = __float_as_uint(__uint_as_float(r[4 * c + 2]) + __uint_as_float(v.z));
                  r[4 * c + 3] = __float_as_uint(__uint_as_float(r[4 * c + 3]) + __uint_as_float(v.w));
                }
              }
            }
            finish_column<KIND>(p, s.row, n_base + q * kPanelN, r, rs);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (abort_s) {
    // let copies that may still be in flight land before shared memory is given back
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kStatusTimeout);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// ------------------------------------------------------------------------------------------
// Per-tile drain kernel: every tile's product is scaled by that tile's scale.
// ------------------------------------------------------------------------------------------
template <int KIND, int NP>
__global__ void __launch_bounds__(kThreads) spmm_drain_kernel(const __grid_constant__ CUtensorMap tmap_b,
                                                              const SpmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ PipeBars bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  constexpr uint32_t kSlotCols = NP * 32;
  constexpr uint32_t kTmemCols = 512;
  constexpr int kSlots = (kTmemCols / kSlotCols) < kMaxSlots ? (kTmemCols / kSlotCols) : kMaxSlots;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t ring_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_bytes = (uint32_t)(NP * kPanelBytes + kTileBytes);
  volatile int* abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    for (int b = 0; b < kSlots; ++b) {
      mbar_init(smem_u32(&bars.acc_full[b]), 1);
      mbar_init(smem_u32(&bars.acc_empty[b]), 4);
    }
    fence_mbar_init();
    if (p.tiles != nullptr) prefetch_tmap(&tmap_b);
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
    producer_loop(p, &tmap_b, &bars, ring_base, stage_bytes, abort_flag, lane);
  } else if (warp == 1) {
    if (lane == 0) {
      int begin, end, step;
      seg_range(p, begin, end, step);
      int stage = 0, slot = 0;
      uint32_t phase = 0, sphase = 0;
      bool ok = true;
      for (int i = begin; i < end && ok; i += step) {
        const Seg s = load_seg(p, i);
        const int npan = panels_in_chunk(p, s.chunk);
        for (int t = s.t0; t < s.t1; ++t) {
          ok = mbar_wait(smem_u32(&bars.full[stage]), phase, abort_flag);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&bars.acc_empty[slot]), sphase ^ 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sbase = ring_base + (uint32_t)stage * stage_bytes;
          const uint64_t bdesc = smem_desc(p.desc_hi_b, sbase + (uint32_t)NP * kPanelBytes);
          const uint32_t d0 = tmem_base + (uint32_t)slot * kSlotCols;
          for (int q = 0; q < npan; ++q) {
            const uint64_t adesc = smem_desc(p.desc_hi_a, sbase + (uint32_t)q * kPanelBytes);
            issue_mma<KIND>(d0 + (uint32_t)q * 32u, adesc, bdesc, p.idesc, 0u);
          }
          tc_commit(smem_u32(&bars.empty[stage]));
          tc_commit(smem_u32(&bars.acc_full[slot]));
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
          if (++slot == kSlots) { slot = 0; sphase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    int begin, end, step;
    seg_range(p, begin, end, step);
    int slot = 0;
    uint32_t sphase = 0;
    bool alive = true;
    for (int i = begin; i < end && alive; i += step) {
      const Seg s = load_seg(p, i);
      const int npan = panels_in_chunk(p, s.chunk);
      float acc[NP][32];
#pragma unroll
      for (int q = 0; q < NP; ++q)
#pragma unroll
        for (int m = 0; m < 32; ++m) acc[q][m] = 0.0f;
      for (int t = s.t0; t < s.t1; ++t) {
        const float ts = __ldg(p.tile_scales + t);
        int ok = 1;
        if (lane == 0) ok = mbar_wait(smem_u32(&bars.acc_full[slot]), sphase, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { alive = false; break; }
        tc_fence_after();
#pragma unroll
        for (int q = 0; q < NP; ++q) {
          if (q < npan) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + lane_sel + (uint32_t)slot * kSlotCols + (uint32_t)q * 32u, r);
            tmem_ld_wait();
            if (q == npan - 1) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty[slot]));
            }
#pragma unroll
            for (int m = 0; m < 32; ++m) {
              const float x = (KIND == VOID_KIND_I8) ? __int2float_rn((int)r[m]) : __uint_as_float(r[m]);
              acc[q][m] = fmaf(ts, x, acc[q][m]);
            }
          }
        }
        if (++slot == kSlots) { slot = 0; sphase ^= 1u; }
      }
      if (!alive) break;
      const int n_base = s.chunk * NP * kPanelN + quad * 32 + lane;
#pragma unroll
      for (int q = 0; q < NP; ++q) {
        if (q < npan) {
          const int n = n_base + q * kPanelN;
          if (n < p.N) {
            if (p.acc_out != nullptr) {
              float* a = reinterpret_cast<float*>(p.acc_out) + (size_t)s.row * kTile * p.N + n;
#pragma unroll
              for (int m = 0; m < 32; ++m) a[(size_t)m * p.N] = acc[q][m];
            }
            const float cs = (p.col_scale != nullptr) ? __ldg(p.col_scale + n) * p.b_scale : p.b_scale;
            const float bias = (p.bias != nullptr) ? __ldg(p.bias + n) : 0.0f;
            float v[32];
#pragma unroll
            for (int m = 0; m < 32; ++m) v[m] = apply_act(acc[q][m] * cs + bias, p.act);
            store_column(p, s.row, n, v);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (abort_s) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kStatusTimeout);
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------------
// Host side: tensor map, launch shape, argument checks.
// ------------------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  return g_encode;
}

static int g_desc_variant = -1;  // debugging aid: alternative descriptor encodings
static int desc_variant() {
  if (g_desc_variant < 0) {
    const char* e = getenv("VOID_B200_DESC_VARIANT");
    g_desc_variant = e ? atoi(e) : 0;
  }
  return g_desc_variant;
}

struct DeviceInfo {
  int sms = 0, cc_major = 0, cc_minor = 0, max_smem = 0;
  bool ok = false;
};
static DeviceInfo device_info() {
  static DeviceInfo cache[64];
  int dev = 0;
  DeviceInfo none;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return none;
  if (!cache[dev].ok) {
    DeviceInfo d;
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return none;
    cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    d.ok = true;
    cache[dev] = d;
  }
  return cache[dev];
}

template <typename K>
static int set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -1;
}

static int spmm_launch(const void_spmm_args* a, int kind, cudaStream_t stream) {
  if (a == nullptr) return VOID_ERR_BAD_ARG;
  if (a->M < 0 || a->N < 0 || a->K < 0 || a->nbr < 0 || a->nnz < 0) return VOID_ERR_BAD_ARG;
  if (a->M == 0 || a->N == 0) return VOID_OK;
  if (a->out == nullptr || a->row_ptr == nullptr) return VOID_ERR_BAD_ARG;
  if (a->nnz > 0 && (a->tiles == nullptr || a->tile_cols == nullptr || a->b == nullptr)) return VOID_ERR_BAD_ARG;
  if (a->out_dtype < VOID_OUT_F32 || a->out_dtype > VOID_OUT_BF16) return VOID_ERR_BAD_ARG;
  if (a->act < VOID_ACT_NONE || a->act > VOID_ACT_SILU) return VOID_ERR_BAD_ARG;
  if (a->scale_mode != VOID_SCALE_ROW_MEAN && a->scale_mode != VOID_SCALE_PER_TILE) return VOID_ERR_BAD_ARG;
  if (a->scale_mode == VOID_SCALE_PER_TILE && a->nnz > 0 && a->tile_scales == nullptr) return VOID_ERR_BAD_ARG;
  if ((long long)a->nbr * kTile < a->M) return VOID_ERR_SHAPE;
  if (a->ldc < a->N) return VOID_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a->tiles) & 1023u) != 0) return VOID_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(a->b) & 15u) != 0 || (a->ldb & 15) != 0 || a->ldb < a->N) return VOID_ERR_ALIGN;

  const DeviceInfo dev = device_info();
  if (!dev.ok) return VOID_ERR_CUDA;
  if (dev.cc_major != 10) return VOID_ERR_ARCH;

  const bool drain = (a->scale_mode == VOID_SCALE_PER_TILE);
  const int total_panels = (a->N + kPanelN - 1) / kPanelN;
  int np = a->panels_per_item;
  if (np != 0 && np != 1 && np != 2 && np != 4) return VOID_ERR_BAD_ARG;
  if (np == 0) {
    np = total_panels >= 4 ? 4 : (total_panels >= 2 ? 2 : 1);
    if (drain && np > 2) np = 2;
    if (a->segs == nullptr) {  // keep enough work items to fill the machine
      while (np > 1 && (long long)a->nbr * ((total_panels + np - 1) / np) < 2ll * dev.sms) np >>= 1;
    }
  }
  const int n_chunks = (total_panels + np - 1) / np;
  const int ctas_per_sm = drain ? 1 : (np == 4 ? 1 : 2);
  const int stage_bytes = np * kPanelBytes + kTileBytes;
  int stages = a->stages;
  if (stages == 0) {
    const int budget = (200 * 1024) / ctas_per_sm;
    stages = budget / stage_bytes;
    if (stages > 12) stages = 12;
  }
  if (stages < 2 || stages > kMaxStages) return VOID_ERR_BAD_ARG;
  const int smem_bytes = stages * stage_bytes + 1024;
  if (smem_bytes > dev.max_smem) return VOID_ERR_SHAPE;

  SpmmParams p;
  p.tiles = a->nnz > 0 ? reinterpret_cast<const uint8_t*>(a->tiles) : nullptr;  // null: no tensor map either
  p.tile_cols = a->tile_cols;
  p.tile_scales = a->tile_scales;
  p.row_ptr = a->row_ptr;
  p.row_scale = a->row_scale;
  p.nbr = a->nbr;
  p.n_chunks = n_chunks;
  p.N = a->N;
  p.M = a->M;
  p.col_scale = a->col_scale;
  p.b_scale = a->b_scale;
  p.bias = a->bias;
  p.out = a->out;
  p.ldc = a->ldc;
  p.out_dtype = a->out_dtype;
  p.act = a->act;
  p.acc_out = a->acc_out;
  p.segs = a->segs;
  p.cta_seg_ptr = a->cta_seg_ptr;
  p.partials = reinterpret_cast<int32_t*>(a->partials);
  p.counters = a->counters;
  p.worker_partials = reinterpret_cast<int32_t*>(a->worker_partials);
  p.status = a->status;
  p.np = np;
  p.stages = stages;
  p.n_items = a->nbr * n_chunks;

  // operand descriptors (see the header comment for the two shared-memory layouts)
  uint32_t tile_lbo = 128, tile_sbo = 256, tile_layout = kLayoutNone;
  const int variant = desc_variant();
  if (variant & 1) { tile_lbo = 256; tile_sbo = 128; }
  if (variant & 2) { tile_lbo = 16; tile_sbo = 256; tile_layout = kLayoutSw32; }
  p.desc_hi_b = smem_desc_hi(tile_lbo, tile_sbo, tile_layout);
  // one 128-byte swizzle atom along n, four 8-row groups along k, 1024 bytes apart
  p.desc_hi_a = smem_desc_hi(1024, 1024, kLayoutSw128);
  if (kind == VOID_KIND_I8) p.idesc = instr_desc(/*c s32*/ 2, /*a s8*/ 1, /*b s8*/ 1, /*a MN*/ 1, /*b K*/ 0, 128, 32);
  else p.idesc = instr_desc(/*c f32*/ 1, /*a e4m3*/ 0, /*b e4m3*/ 0, 1, 0, 128, 32);

  int grid;
  if (a->segs != nullptr) {
    if (a->cta_seg_ptr == nullptr || a->n_cta <= 0 || a->panels_per_item == 0) return VOID_ERR_BAD_ARG;
    if (drain) return VOID_ERR_BAD_ARG;  // split rows are finished by the row-accumulate kernel only
    grid = a->n_cta;
  } else {
    grid = a->grid > 0 ? a->grid : dev.sms * ctas_per_sm;
    if (grid > p.n_items) grid = p.n_items;
    if (grid < 1) grid = 1;
  }

  // B as a 2-D tensor: dim0 = n (contiguous), dim1 = k; box = one panel (128 x 32), 128-byte swizzle.
  // Out-of-range parts of a box (n >= N, k >= K) are filled with zeros by the copy engine.
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  if (a->nnz > 0) {
    PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode();
    if (enc == nullptr) return VOID_ERR_CUDA;
    const cuuint64_t gdim[2] = {(cuuint64_t)a->N, (cuuint64_t)a->K};
    const cuuint64_t gstride[1] = {(cuuint64_t)a->ldb};
    const cuuint32_t box[2] = {(cuuint32_t)kPanelN, (cuuint32_t)kTile};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(a->b), gdim, gstride, box,
                           estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return VOID_ERR_CUDA;
  }

  cudaError_t err = cudaSuccess;
  if (!drain) {
    if (kind == VOID_KIND_I8) {
      if (set_smem(spmm_rowacc_kernel<VOID_KIND_I8>, smem_bytes)) return VOID_ERR_CUDA;
      spmm_rowacc_kernel<VOID_KIND_I8><<<grid, kThreads, smem_bytes, stream>>>(tmap, p);
    } else {
      if (set_smem(spmm_rowacc_kernel<VOID_KIND_F8E4M3>, smem_bytes)) return VOID_ERR_CUDA;
      spmm_rowacc_kernel<VOID_KIND_F8E4M3><<<grid, kThreads, smem_bytes, stream>>>(tmap, p);
    }
  } else {
#define VB_LAUNCH_DRAIN(KIND, NP)                                                      \
  do {                                                                                 \
    if (set_smem(spmm_drain_kernel<KIND, NP>, smem_bytes)) return VOID_ERR_CUDA;       \
    spmm_drain_kernel<KIND, NP><<<grid, kThreads, smem_bytes, stream>>>(tmap, p);      \
  } while (0)
    if (kind == VOID_KIND_I8) {
      if (np == 1) VB_LAUNCH_DRAIN(VOID_KIND_I8, 1);
      else if (np == 2) VB_LAUNCH_DRAIN(VOID_KIND_I8, 2);
      else VB_LAUNCH_DRAIN(VOID_KIND_I8, 4);
    } else {
      if (np == 1) VB_LAUNCH_DRAIN(VOID_KIND_F8E4M3, 1);
      else if (np == 2) VB_LAUNCH_DRAIN(VOID_KIND_F8E4M3, 2);
      else VB_LAUNCH_DRAIN(VOID_KIND_F8E4M3, 4);
    }
#undef VB_LAUNCH_DRAIN
  }
  err = cudaGetLastError();
  return err == cudaSuccess ? VOID_OK : VOID_ERR_CUDA;
}

}  // namespace vb

extern "C" {

int void_spmm_i8(const void_spmm_args* args, void_stream_t stream) {
  return vb::spmm_launch(args, VOID_KIND_I8, reinterpret_cast<cudaStream_t>(stream));
}
int void_spmm_f8(const void_spmm_args* args, void_stream_t stream) {
  return vb::spmm_launch(args, VOID_KIND_F8E4M3, reinterpret_cast<cudaStream_t>(stream));
}
int void_device_sm_count(void) {
  const vb::DeviceInfo d = vb::device_info();
  return d.ok ? d.sms : 0;
}

}  // extern "C"
