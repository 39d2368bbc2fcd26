// Block-sparse SpMM for B200 (sm_100a):  C = act(dequant(A . B) + bias), A quantized to 8 bits (INT8 or
// FP8 E4M3 with per-block scales) or floating point (fp16 / bf16, or fp32 multiplied as TF32).
//
// A is the packed VOID tensor (tile-row-major 32x32 tiles, each stored as 8-row x 16-byte core
// matrices), B is a row-major [K, N] matrix of the same element size.  The product is computed
// transposed on the tensor cores so that the 32-row tile sits in the N slot of the instruction:
//
//     D[n, m] (+)= sum_k  B[kcol*32 + k, n0 + n] * A_tile[m, k]        n < 128, m < 32, k < 32
//
// i.e. tcgen05.mma (M=128, N=32, 32 bytes of k) once per (tile, 128-column panel of B) for 8-bit
// elements, twice for 16-bit, four times for 32-bit.  The "A" operand of the instruction is the B
// panel exactly as it lies in memory (n contiguous: MN-major, 128-byte swizzle, written by a tiled
// TMA load); the "B" operand is the packed tile (K-major, no swizzle, written by a linear bulk
// copy).  Accumulators live in tensor memory: lane = output column n, column = tile row m.
//
// Warp roles (struct Shape): producer warps stream tiles and panels into a shared-memory ring, one
// warp issues the MMAs and owns the tensor-memory allocation, epilogue warps read accumulators back
// (one or two warps per 32-lane TMEM quadrant), apply scales / bias / activation and store C.
//
// The ring moves GROUPS of up to `group` consecutive tiles of a tile row per stage: a group needs one
// wait + one expect_tx + one bulk copy (its tiles are contiguous in the packed store) and one tiled TMA
// per tile, the TMAs issued by different lanes in the same instruction, and the producer warps take the
// groups round-robin so that several stage turns are in flight at once.  Measured on B200, a stage's
// round trip (copies requested, landed, MMAs issued and retired, stage handed back) takes 1.2 - 1.3 us
// whatever its size, so a CTA streams what its ring holds per round trip and the launcher gives the
// ring all the shared memory that four CTAs per SM leave each other.  When N is a whole number of
// 128-byte column blocks the TMA is 3-D (B viewed as [column block][k][128 bytes]) and fetches all panels
// of the work item at once.
//
// Two kernels share this pipeline:
//   spmm_rowacc_kernel  one accumulator per (tile row, column chunk), scaled once by the
//                       row's mean tile scale (the INT8 semantic of void/int_quant.py:479-526), by
//                       the row's reference scale (FP8 tiles packed with their scales folded in: each
//                       tile is then two or three E4M3 terms that multiply the same panel), or
//                       not at all (floating point, void/ops.py:93-146); rows cut into several
//                       segments by a work plan are finished by the CTA that arrives last - the
//                       segments of a row may belong to different GPUs (sum over ranks: partial tiles
//                       go to the owning rank through peer pointers).
//   spmm_drain_kernel   every tile's product lands in its own TMEM slot and is folded into
//                       registers with that tile's scale (the exact FP8 semantic of
//                       void/fp8.py:638-659; also exact per-block INT8 dequantisation).
//
// Launch order: the kernels use programmatic dependent launch.  Set-up touches no global memory; every
// role then waits for the previous kernel of the stream where it first needs data that kernel may have
// written.  When the caller vouches that the packed A is not being written by any kernel in flight, the
// index of A and the first tiles are read ahead of that wait.
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
// Bytes per element of the operands of a kind: the 8-bit kinds, fp16 / bf16, fp32 read as TF32.  A tile
// takes kTileBytes * ES bytes, a 128-column panel kPanelBytes * ES (stored as ES blocks of 32 k-rows x
// 128 bytes, one swizzle atom wide each), and one (tile, panel) product takes ES MMAs of 32 bytes of k.
template <int KIND>
struct Elem {
  static constexpr int ES = (KIND == VOID_KIND_TF32) ? 4 : ((KIND == VOID_KIND_F16 || KIND == VOID_KIND_BF16) ? 2 : 1);
};
constexpr int kMaxStages = 16;
constexpr int kMaxSlots = 16;
// Warp roles of a CTA: PW producer warps (0..PW-1) stream tiles and panels, warp PW issues the MMAs
// and owns the TMEM allocation, EW epilogue warps follow (EW/4 per TMEM lane quadrant, each taking
// 32/(EW/4) accumulator columns).  Two shapes are built: a wide one (4 + 1 + 8 warps, two CTAs per
// SM) and a slim one (2 + 1 + 4 warps, four CTAs per SM).  A CTA's stream is bound by the round trip of
// its ring, so four slim CTAs per SM move more tiles than two wide ones.
template <int PW_, int EW_, int CTAS_>
struct Shape {
  static constexpr int PW = PW_;
  static constexpr int EW = EW_;
  static constexpr int MMA = PW_;
  static constexpr int EPI0 = PW_ + 1;
  static constexpr int EPI_THREADS = 32 * EW_;
  static constexpr int THREADS = 32 * (PW_ + 1 + EW_);
  static constexpr int COLS = 32 / (EW_ / 4);  // accumulator columns one epilogue warp reads
  static constexpr int CTAS_PER_SM = CTAS_;
};
using Wide = Shape<4, 8, 2>;
using Slim = Shape<2, 4, 4>;
// Shapes of the per-tile kernel, three CTAs per SM so that an epilogue thread can hold 32 raw products in
// registers next to its running sums: four epilogue warps with all 32 accumulator columns each, or eight
// with 16 each (two tiles per round trip to tensor memory).
// (The register file is split over the four schedulers of an SM, so what a thread may use follows from the
// warps per scheduler: 28 warps -> 72 registers, 24 or 21 -> 80, 30 -> 64.)
using Slim3 = Shape<2, 4, 3>;
using Drain8 = Shape<1, 8, 3>;
using Slim1 = Shape<1, 4, 4>;
constexpr int kDefaultDrainShape = 2;   // cta_shape the one-panel per-tile kernel runs with by default

// device status codes (written to the status word)
constexpr int kStatusTimeout = 1;
constexpr int kStatusBadPlan = 2;   // a split row of the plan points outside the scratch the caller provided

struct SpmmParams {
  const uint8_t* tiles;
  const int32_t* tile_cols;
  const float* tile_scales;
  const int32_t* row_ptr;
  const int32_t* row_order;  // launches without a plan: tile row of the k-th row taken, or null for k
  const float* row_scale;
  int nbr, nbc, n_chunks, N, M;
  long long nnz;
  const float* col_scale;
  float b_scale;
  const float* bias;
  const float* row_bias;
  void* out;
  long long ldc;
  int out_dtype, act;
  void* acc_out;
  const int32_t* segs;
  const int32_t* cta_seg_ptr;
  int32_t* partials;
  int32_t* counters;
  int32_t* worker_partials;
  // Split rows whose sums live on other GPUs (reduction across ranks): n_peers > 0 makes field slot0 of a
  // segment the owner of its tile row; the row's accumulator, arrival counter and rows of C are the owner's,
  // reached through peer pointers (peer_out is offset so that the GLOBAL tile row indexes it).
  int n_peers;
  int peer_slots;   // 1: every contributing rank stores its partial tile into its own slot of the owner's scratch
                    // (plain stores, no counters); a second kernel on the owner adds the slots (void_reduce_slots)
  int32_t* peer_partials[8];
  int32_t* peer_counters[8];
  void* peer_out[8];
  int32_t* status;
  unsigned long long* trace;  // diagnostic instantiations only: 64 timestamps per CTA
  int np;       // panels per work item
  int terms;    // packed tiles per stored tile: 1, or 2 / 3 when an FP8 tile is stored as a sum of E4M3 terms
  int group;    // tiles per ring stage
  int stages;   // ring depth
  int last_group;   // tiles of the ring's last stage (1 .. group): the shared memory left over by the full stages
  int use3d;    // B panels of a tile fetched by one 3-D TMA
  int tma_store;  // 16-bit outputs leave through a staging tile in shared memory and a tiled TMA store
  int tmem_cols;  // tensor-memory columns of the drain kernel (256: two CTAs per SM, 512: one)
  int n_items;  // without a plan: nbr * n_chunks
  int a_stable;   // A's packed arrays and the plan were complete before the stream's kernels in flight started:
                  // they may be read before the wait on the previous kernel
  int ctr_limit;  // split rows the scratch (partials, counters) has room for
  int wait_limit_ms;  // limit of every device-side wait
  int drop_group;     // test hook: the producers never fill the ring stage of each CTA's first group of tiles
  unsigned long long desc_hi_a;  // B panel  (instruction operand A: MN-major, 128B swizzle)
  unsigned long long desc_hi_b;  // A tile   (instruction operand B: K-major, no swizzle)
  unsigned int idesc;
};

// Time stamps exist in the diagnostic instantiations (TRACE) only; the kernels every ordinary launch runs
// are compiled without them.
template <bool TRACE>
__device__ __forceinline__ void stamp(const SpmmParams& p, int slot) {
  if constexpr (TRACE) {
    if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * 64 + slot] = globaltimer_ns();
  }
}

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
    const int k = i / p.n_chunks;   // k-th tile row taken
    s.chunk = i - k * p.n_chunks;
    s.row = k;
    if (p.row_order != nullptr) {
      const int r = __ldg(p.row_order + k);
      s.row = r < 0 ? 0 : (r >= p.nbr ? p.nbr - 1 : r);
    }
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

// GELU in the tanh form written with a sigmoid, void/fusion.py:38-43.  exp and the reciprocal use
// the hardware approximations (a few ulp; far inside the path's 1e-3 bar): with the full-precision
// versions this epilogue, run by two warps per scheduler, cost more than the product itself.
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh_sigmoid(float x) {
  // x * 0.5 * (1 + (2 sigmoid(2u) - 1)) = x * sigmoid(2u),  2u = 1.5957691216 (x + 0.044715 x^3)
  const float two_u = 1.5957691216f * x * fmaf(0.044715f * x, x, 1.0f);
  return x * fast_sigmoid(two_u);
}
// What an epilogue thread needs to know about C, read from the kernel parameters once.
struct OutDesc {
  void* out;
  long long ldc;
  void* acc_out;
  const float* row_bias;  // [M] added per output row before the activation (linear-layer bias), or null
  int M, N, dtype, act;
};
__device__ __forceinline__ OutDesc out_desc(const SpmmParams& p) {
  OutDesc o;
  o.out = p.out; o.ldc = p.ldc; o.acc_out = p.acc_out; o.row_bias = p.row_bias; o.M = p.M; o.N = p.N; o.dtype = p.out_dtype; o.act = p.act;
  return o;
}

// Store eight finished values of output column n: matrix rows row*32 + m0 .. + 7.
__device__ __forceinline__ void store8(const OutDesc& o, int row, int n, int m0, float (&v)[8]) {
  const int r0 = row * kTile + m0;
  const int rows = o.M - r0;  // rows left below r0
  if (o.row_bias != nullptr) {
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < rows) v[k] += __ldg(o.row_bias + r0 + k);
  }
  switch (o.act) {
    case VOID_ACT_RELU:
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = fmaxf(v[k], 0.0f);
      break;
    case VOID_ACT_GELU:
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = gelu_tanh_sigmoid(v[k]);
      break;
    case VOID_ACT_SILU:
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = v[k] * fast_sigmoid(v[k]);
      break;
    default:
      break;
  }
  if (o.dtype == VOID_OUT_F16) {
    __half* dst = reinterpret_cast<__half*>(o.out) + (size_t)r0 * o.ldc + n;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < rows) dst[(size_t)k * o.ldc] = __float2half_rn(v[k]);
  } else if (o.dtype == VOID_OUT_BF16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(o.out) + (size_t)r0 * o.ldc + n;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < rows) dst[(size_t)k * o.ldc] = __float2bfloat16_rn(v[k]);
  } else {
    float* dst = reinterpret_cast<float*>(o.out) + (size_t)r0 * o.ldc + n;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < rows) dst[(size_t)k * o.ldc] = v[k];
  }
}

// Epilogue of eight raw accumulators of one output column: dequantise, bias, activation, store.
template <int KIND>
__device__ __forceinline__ void finish8(const OutDesc& o, int row, int n, int m0, const uint32_t (&r)[8],
                                        float row_scale, float cs, float bias) {
  if (n >= o.N) return;
  if (o.acc_out != nullptr) {
    uint32_t* a = reinterpret_cast<uint32_t*>(o.acc_out) + ((size_t)row * kTile + m0) * o.N + n;
#pragma unroll
    for (int k = 0; k < 8; ++k) a[(size_t)k * o.N] = r[k];
  }
  float v[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float x = (KIND == VOID_KIND_I8) ? __int2float_rn((int)r[k]) : __uint_as_float(r[k]);
    v[k] = (x * row_scale) * cs + bias;
  }
  store8(o, row, n, m0, v);
}

// Fast epilogue of sixteen raw accumulators of output column n (tile rows m0 .. m0 + 15) straight to C
// (no raw-accumulator dump, no split row), stores specialised per output type.
template <int KIND>
__device__ __forceinline__ void finish16(const OutDesc& o, int row, int n, int m0, const uint32_t* r,
                                         float row_scale, float cs, float bias) {
  if (n >= o.N) return;
  float v[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float x = (KIND == VOID_KIND_I8) ? __int2float_rn((int)r[k]) : __uint_as_float(r[k]);
    v[k] = (x * row_scale) * cs + bias;
  }
  const int r0 = row * kTile + m0;
  const int rows = o.M - r0;
  if (o.row_bias != nullptr) {
#pragma unroll
    for (int k = 0; k < 16; ++k)
      if (k < rows) v[k] += __ldg(o.row_bias + r0 + k);
  }
  if (o.act != VOID_ACT_NONE) {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (o.act == VOID_ACT_GELU) v[k] = gelu_tanh_sigmoid(v[k]);
      else if (o.act == VOID_ACT_RELU) v[k] = fmaxf(v[k], 0.0f);
      else v[k] = v[k] * fast_sigmoid(v[k]);
    }
  }
  const size_t first = (size_t)r0 * o.ldc + n;
  if (o.dtype == VOID_OUT_F16) {
    __half* dst = reinterpret_cast<__half*>(o.out) + first;
#pragma unroll
    for (int k = 0; k < 16; ++k, dst += o.ldc)
      if (k < rows) *dst = __float2half_rn(v[k]);
  } else if (o.dtype == VOID_OUT_BF16) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(o.out) + first;
#pragma unroll
    for (int k = 0; k < 16; ++k, dst += o.ldc)
      if (k < rows) *dst = __float2bfloat16_rn(v[k]);
  } else {
    float* dst = reinterpret_cast<float*>(o.out) + first;
#pragma unroll
    for (int k = 0; k < 16; ++k, dst += o.ldc)
      if (k < rows) *dst = v[k];
  }
}

// Sixteen finished 16-bit values of output column n into a staging tile [32 m][PITCH n] in shared memory
// (stage_col points at element [0][n - n0]); same arithmetic as finish16.
template <int KIND, int PITCH>
__device__ __forceinline__ void finish16_stage(const OutDesc& o, int row, int n, int m0, const uint32_t* r,
                                               float row_scale, float cs, float bias, uint16_t* stage_col) {
  float v[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float x = (KIND == VOID_KIND_I8) ? __int2float_rn((int)r[k]) : __uint_as_float(r[k]);
    v[k] = (x * row_scale) * cs + bias;
  }
  const int r0 = row * kTile + m0;
  const int rows = o.M - r0;
  if (o.row_bias != nullptr) {
#pragma unroll
    for (int k = 0; k < 16; ++k)
      if (k < rows) v[k] += __ldg(o.row_bias + r0 + k);
  }
  if (o.act != VOID_ACT_NONE) {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (o.act == VOID_ACT_GELU) v[k] = gelu_tanh_sigmoid(v[k]);
      else if (o.act == VOID_ACT_RELU) v[k] = fmaxf(v[k], 0.0f);
      else v[k] = v[k] * fast_sigmoid(v[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    uint16_t h;
    if (o.dtype == VOID_OUT_F16) h = __half_as_ushort(__float2half_rn(v[k]));
    else h = __bfloat16_as_ushort(__float2bfloat16_rn(v[k]));
    stage_col[(m0 + k) * PITCH] = h;
  }
}

// Transposed output (C stored as [N, M], m contiguous): the thread owns output row n and sixteen consecutive
// columns m0 .. m0 + 15 of it, so the values leave in 16-byte stores.  bias_n is the bias of this n, the
// per-m bias (o.row_bias) is the same for every thread of the warp.
template <int KIND>
__device__ __forceinline__ void finish16_tr(const OutDesc& o, int row, int n, int m0, const uint32_t* r,
                                            float row_scale, float cs, float bias_n) {
  if (n >= o.N) return;
  const int c0 = row * kTile + m0;   // first output column (a row index of A)
  const int cols = o.M - c0;         // columns left
  if (cols <= 0) return;
  float v[16];
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const float x = (KIND == VOID_KIND_I8) ? __int2float_rn((int)r[k]) : __uint_as_float(r[k]);
    v[k] = (x * row_scale) * cs + bias_n;
  }
  if (o.row_bias != nullptr) {
#pragma unroll
    for (int k = 0; k < 16; ++k)
      if (k < cols) v[k] += __ldg(o.row_bias + c0 + k);
  }
  if (o.act != VOID_ACT_NONE) {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      if (o.act == VOID_ACT_GELU) v[k] = gelu_tanh_sigmoid(v[k]);
      else if (o.act == VOID_ACT_RELU) v[k] = fmaxf(v[k], 0.0f);
      else v[k] = v[k] * fast_sigmoid(v[k]);
    }
  }
  const size_t first = (size_t)n * o.ldc + c0;
  if (o.dtype == VOID_OUT_F32) {
    float* dst = reinterpret_cast<float*>(o.out) + first;
    if (cols >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
      for (int k = 0; k < 16; k += 4) *reinterpret_cast<float4*>(dst + k) = make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]);
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k)
        if (k < cols) dst[k] = v[k];
    }
  } else {
    uint32_t h[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (o.dtype == VOID_OUT_F16) {
        const __half2 t = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
        h[k] = *reinterpret_cast<const uint32_t*>(&t);
      } else {
        const __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
        h[k] = *reinterpret_cast<const uint32_t*>(&t);
      }
    }
    uint16_t* dst = reinterpret_cast<uint16_t*>(o.out) + first;
    if (cols >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<uint4*>(dst + 8) = make_uint4(h[4], h[5], h[6], h[7]);
    } else {
#pragma unroll
      for (int k = 0; k < 16; ++k)
        if (k < cols) dst[k] = (uint16_t)(h[k >> 1] >> ((k & 1) * 16));
    }
  }
}

struct __align__(8) PipeBars {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[kMaxSlots];
  uint64_t acc_empty[kMaxSlots];
};

// shared-memory offsets inside one ring stage
template <int ES>
__device__ __forceinline__ uint32_t panel_off(const SpmmParams& p, int j, int q) {
  return (uint32_t)(j * p.np + q) * (kPanelBytes * ES);
}
// A stage holds the panels of its tiles first, then the tiles; `cap` is the stage's capacity in tiles
template <int ES>
__device__ __forceinline__ uint32_t tile_off(const SpmmParams& p, int cap, int j) {
  return (uint32_t)(cap * p.np) * (kPanelBytes * ES) + (uint32_t)(j * p.terms) * (kTileBytes * ES);
}
// Capacity of a ring stage: every stage takes p.group tiles except the last, which takes what is left of the
// shared memory (p.last_group).  The groups of a tile row follow the stages they fall on: a group is
// min(capacity of its stage, tiles left in the row) consecutive tiles.
__device__ __forceinline__ int stage_cap(const SpmmParams& p, int stage) {
  return stage == p.stages - 1 ? p.last_group : p.group;
}

// Producer warp `pw` of C::PW: the CTA's groups of tiles are numbered in the order the MMA warp
// consumes them; group g uses ring stage g % stages and belongs to warp g % C::PW.
//
// The wait on the previous kernel of the stream sits where the first read of data that kernel may
// have produced is.  When the caller vouches for A (p.a_stable: the packed tiles, their index arrays
// and the plan were complete before the kernels now in flight started) the warp reads the index,
// claims its first ring stage and starts the bulk copy of that stage's tiles BEFORE the wait, while the
// previous kernel is still draining; only the panels of B - typically that kernel's output - are
// requested after it.
template <class C, int ES, bool TR, bool TRACE>
__device__ __forceinline__ void producer_loop(const SpmmParams& p, const CUtensorMap* tmap, PipeBars* bars,
                                              uint32_t ring_base, uint32_t stage_bytes, volatile int* ctl,
                                              int lane, int pw) {
  bool waited = p.a_stable == 0;
  if (waited) grid_dependency_wait();
  if (TRACE && pw == 0 && lane == 0) stamp<TRACE>(p, 56);   // producer starts
  int begin, end, step;
  seg_range(p, begin, end, step);
  const int S = p.stages;
  // position of the next group in the ring: its stage, the parity of the stage's use, the warp it belongs to
  int stage = 0, owner = 0, gcount = 0;
  uint32_t phase = 0;
  Seg seg_next = {};  // the next segment's descriptor is fetched one item ahead
  if (begin < end) seg_next = load_seg(p, begin);
  for (int i = begin; i < end; i += step) {
    const Seg s = seg_next;
    if (i + step < end) seg_next = load_seg(p, i + step);
    const int npan = panels_in_chunk(p, s.chunk);
    const int n0 = s.chunk * p.np * kPanelN;
    const uint32_t unit_bytes = (uint32_t)((kTileBytes * p.terms + ((p.use3d && !TR) ? p.np : npan) * kPanelBytes) * ES);
    if (TRACE && i == begin && pw == 0 && lane == 0) {
      asm volatile("" ::"r"(s.t1) : "memory");
      stamp<TRACE>(p, 57);   // the row's tile range has arrived
    }
    // block column of this lane's tile in the warp's next group, fetched one group of its own ahead; (ct, cs):
    // first tile and stage of that group
    int ct = s.t0, cs = stage;
    for (int o = owner; o != pw && ct < s.t1; o = (o + 1 == C::PW) ? 0 : o + 1) {
      ct += stage_cap(p, cs);
      cs = (cs + 1 == S) ? 0 : cs + 1;
    }
    int col = 0;
    if (ct + lane < s.t1 && lane < stage_cap(p, cs)) col = __ldg(p.tile_cols + ct + lane);
    if (TRACE && i == begin && pw == 0 && lane == 0) {
      asm volatile("" ::"r"(col) : "memory");
      stamp<TRACE>(p, 58);   // the first block columns have arrived
    }
    int k = 0;   // group of the segment
    for (int t = s.t0; t < s.t1; ++k, ++gcount) {
      const int cap = stage_cap(p, stage);
      const int gcnt = (s.t1 - t) < cap ? (s.t1 - t) : cap;
      if (owner == pw) {
        // this warp's group after this one
        int nt = t, ns = stage;
        for (int o = 0; o < C::PW && nt < s.t1; ++o) {
          nt += stage_cap(p, ns);
          ns = (ns + 1 == S) ? 0 : ns + 1;
        }
        int col_next = 0;
        if (nt + lane < s.t1 && lane < stage_cap(p, ns)) col_next = __ldg(p.tile_cols + nt + lane);
        const uint32_t full = smem_u32(&bars->full[stage]);
        const uint32_t sbase = ring_base + (uint32_t)stage * stage_bytes;
        // test hook: the first group of the CTA is never delivered, so the consumer's bounded wait runs out
        const bool drop = p.drop_group != 0 && gcount == 0;
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, ctl) ? 1 : 0;
          if (ok && !drop) {
            mbar_expect_tx(full, unit_bytes * (uint32_t)gcnt);
            bulk_load(sbase + tile_off<ES>(p, cap, 0), p.tiles + (size_t)t * (size_t)(kTileBytes * ES * p.terms),
                      (uint32_t)(gcnt * p.terms) * (kTileBytes * ES), full);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return;
        if (TRACE && i == begin && pw == 0 && lane == 0 && k == 0) stamp<TRACE>(p, 59);   // tiles of the first group requested
        if (!waited) {  // B may be the output of the previous kernel
          grid_dependency_wait();
          waited = true;
        }
        if (TRACE && i == begin && pw == 0 && lane == 0 && k == 0) stamp<TRACE>(p, 60);   // past the wait on the previous kernel
        if (lane < gcnt && !drop) {
          if (TR) {
            // B stored transposed ([N, K], k contiguous): one box of 128 rows of n x 32 k per panel
            for (int q = 0; q < npan; ++q)
              tma_load_2d(sbase + panel_off<ES>(p, lane, q), tmap, col * kTile, n0 + q * kPanelN, full);
          } else if (p.use3d) {
            tma_load_3d(sbase + panel_off<ES>(p, lane, 0), tmap, 0, col * kTile, s.chunk * p.np * ES, full);
          } else {
            // one copy per 128-byte-wide block of columns: ES blocks of 128 / ES columns per panel
            for (int q = 0; q < npan * ES; ++q)
              tma_load_2d(sbase + panel_off<ES>(p, lane, 0) + (uint32_t)q * kPanelBytes, tmap,
                          n0 + q * (kPanelN / ES), col * kTile, full);
          }
        }
        if (TRACE && lane == 0 && i == begin && k < 16) stamp<TRACE>(p, 32 + k);
        col = col_next;
      }
      t += gcnt;
      owner = (owner + 1 == C::PW) ? 0 : owner + 1;
      if (++stage == S) { stage = 0; phase ^= 1u; }
    }
  }
  if (!waited) grid_dependency_wait();
}

template <int KIND>
__device__ __forceinline__ void issue_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  if (KIND == VOID_KIND_I8) mma_i8(d, a, b, idesc, acc);
  else if (KIND == VOID_KIND_F8E4M3) mma_f8(d, a, b, idesc, acc);
  else if (KIND == VOID_KIND_TF32) mma_tf32(d, a, b, idesc, acc);
  else mma_f16(d, a, b, idesc, acc);
}

// Barriers, tensor memory and the launch of the next kernel's set-up.  Nothing here touches global memory,
// so all of it overlaps the tail of the previous kernel of the stream (programmatic dependent launch);
// every role then waits for that kernel where it first needs data the kernel may have written.
template <class C, int ES, bool TRACE>
__device__ __forceinline__ void pipeline_setup(const SpmmParams& p, const CUtensorMap* tmap, PipeBars& bars,
                                               uint32_t* tmem_base_s, int* ctl_s, int n_acc, uint32_t tmem_cols) {
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) stamp<TRACE>(p, 62);
  if constexpr (TRACE) {   // slot 63: the SM this CTA runs on
    if (threadIdx.x == 0 && p.trace != nullptr) {
      uint32_t smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      p.trace[(size_t)blockIdx.x * 64 + 63] = smid;
    }
  }
  if (threadIdx.x == 0) {
    ctl_s[0] = 0;
    ctl_s[1] = p.wait_limit_ms;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    for (int b = 0; b < n_acc; ++b) {
      mbar_init(smem_u32(&bars.acc_full[b]), 1);
      mbar_init(smem_u32(&bars.acc_empty[b]), C::EW);
    }
    fence_mbar_init();
    if (p.tiles != nullptr) prefetch_tmap(tmap);
  }
  if (warp == C::MMA) {
    tmem_alloc(smem_u32(tmem_base_s), tmem_cols);
    tmem_relinquish();
  }
  grid_launch_dependents();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) stamp<TRACE>(p, 1);
}

template <class C, bool TRACE>
__device__ __forceinline__ void pipeline_teardown(const SpmmParams& p, int* ctl_s, uint32_t tmem_base,
                                                  uint32_t tmem_cols) {
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) stamp<TRACE>(p, 7);
  if (ctl_s[0]) {
    // let copies that may still be in flight land before shared memory is given back
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, kStatusTimeout);
    __syncthreads();
  }
  if ((threadIdx.x >> 5) == C::MMA) tmem_dealloc(tmem_base, tmem_cols);
}

// ------------------------------------------------------------------------------------------
// Row-accumulate kernel.
// ------------------------------------------------------------------------------------------
// All COLS accumulator columns of one epilogue warp, requested together (no wait).
template <int COLS>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[COLS]) {
#pragma unroll
  for (int c = 0; c < COLS; c += 16) tmem_ld_32x16p(taddr + (uint32_t)c, &r[c]);
}

template <int KIND, class C, bool TR = false, bool TRACE = false>
__global__ void __launch_bounds__(C::THREADS, C::CTAS_PER_SM) spmm_rowacc_kernel(const __grid_constant__ CUtensorMap tmap_b,
                                                               const __grid_constant__ CUtensorMap tmap_c,
                                                               const __grid_constant__ SpmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ PipeBars bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int ctl_s[2];   // abort flag, wait limit in ms
  __shared__ int last_s;
  __shared__ int ok_s[2];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t ring_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int ES = Elem<KIND>::ES;
  const uint32_t unit_smem = (uint32_t)((p.np * kPanelBytes + kTileBytes * p.terms) * ES);
  const uint32_t stage_bytes = (uint32_t)p.group * unit_smem;   // the last stage may be shorter (p.last_group tiles)
  const uint32_t ring_bytes = (uint32_t)((p.stages - 1) * p.group + p.last_group) * unit_smem;
  const uint32_t acc_cols = (uint32_t)p.np * 32u;  // TMEM columns of one accumulator buffer
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2u * acc_cols) tmem_cols <<= 1;
  volatile int* ctl = ctl_s;

  if (threadIdx.x == 0) last_s = 0;
  pipeline_setup<C, ES, TRACE>(p, &tmap_b, bars, &tmem_base_s, ctl_s, 2, tmem_cols);
  const uint32_t tmem_base = tmem_base_s;

  if (warp < C::PW) {
    producer_loop<C, ES, TR, TRACE>(p, &tmap_b, &bars, ring_base, stage_bytes, ctl, lane, warp);
    if (warp == 0 && lane == 0) stamp<TRACE>(p, 2);
  } else if (warp == C::MMA) {
    {
      // The whole warp walks the loop and waits on the barriers together; one elected lane issues the MMAs and
      // the commits.  The control flow stays convergent, so the addresses, descriptors and counters are the
      // same in every lane and the compiler may keep them in the warp's uniform registers, where the
      // instruction operands have to be: a loop run by a single lane computes them per thread and moves them
      // over before every MMA.
      // The warp reads the index of A and the plan only; everything else reaches it through the ring.
      const bool leader = elect_one();
      if (!p.a_stable) grid_dependency_wait();
      const uint32_t idesc = p.idesc;
      const uint64_t hi_a = p.desc_hi_a, hi_b = p.desc_hi_b;
      const int S = p.stages, np = p.np, terms = p.terms;
      constexpr uint64_t kPanelStep = (kPanelBytes * ES) >> 4, kTileStep = (kTileBytes * ES) >> 4;
      // one MMA covers 32 bytes of k: 32 / ES k-rows of the panel (8-row groups 1024 bytes apart) and two
      // 16-byte k-chunks of the packed tile (128 bytes apart)
      // (transposed B: the panel is K-major, 32 bytes of k lie inside one row of its swizzle atom)
      constexpr uint64_t kPanelKStep = TR ? 2 : ((kPanelBytes / ES) >> 4), kTileKStep = 256 >> 4;
      int begin, end, step;
      seg_range(p, begin, end, step);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t sbase = ring_base;
      uint32_t it = 0;
      bool ok = true;
      Seg seg_next = {};  // the next segment's descriptor is fetched one item ahead
      if (begin < end) seg_next = load_seg(p, begin);
      for (int i = begin; i < end && ok; i += step, ++it) {
        const Seg s = seg_next;
        if (i + step < end) seg_next = load_seg(p, i + step);
        const int npan = panels_in_chunk(p, s.chunk);
        const uint32_t buf = it & 1u, aph = (it >> 1) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.acc_empty[buf]), aph ^ 1u, ctl));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * acc_cols;
        uint32_t acc = 0u;
        int gidx = 0;
        for (int t = s.t0; t < s.t1; ++gidx) {
          const int cap = stage_cap(p, stage);
          const int gcnt = (s.t1 - t) < cap ? (s.t1 - t) : cap;
          t += gcnt;
          if (TRACE && leader && i == begin && gidx < 8) stamp<TRACE>(p, 48 + gidx);
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[stage]), phase, ctl));
          if (!ok) break;
          if (TRACE && leader && i == begin && gidx < 12) stamp<TRACE>(p, 16 + gidx);   // slots 28 .. 31: last arriver of a split row
          tc_fence_after();
          uint64_t ad = smem_desc(hi_a, sbase);
          uint64_t bd = smem_desc(hi_b, sbase + tile_off<ES>(p, cap, 0));
          for (int j = 0; j < gcnt; ++j) {
            uint64_t adq = ad;
            uint32_t d = d0;
            for (int q = 0; q < npan; ++q) {
              if (leader) issue_mma<KIND>(d, adq, bd, idesc, acc);
#pragma unroll
              for (int kk = 1; kk < ES; ++kk)
                if (leader) issue_mma<KIND>(d, adq + kk * kPanelKStep, bd + kk * kTileKStep, idesc, 1u);
              // a tile stored as a sum of terms: every further term multiplies the same panel
              if (KIND == VOID_KIND_F8E4M3)
                for (int v = 1; v < terms; ++v)
                  if (leader) issue_mma<KIND>(d, adq, bd + (uint64_t)v * kTileStep, idesc, 1u);
              adq += kPanelStep;
              d += 32u;
            }
            ad += kPanelStep * (uint64_t)np;
            bd += kTileStep * (uint64_t)terms;
            acc = 1u;
          }
          if (leader) tc_commit(smem_u32(&bars.empty[stage]));
          sbase += stage_bytes;
          if (++stage == S) { stage = 0; phase ^= 1u; sbase = ring_base; }
        }
        if (!ok) break;
        if (leader) {
          if (s.t1 > s.t0) tc_commit(smem_u32(&bars.acc_full[buf]));
          else mbar_arrive(smem_u32(&bars.acc_full[buf]));
          if (i == begin) stamp<TRACE>(p, 3);
        }
      }
      if (leader) stamp<TRACE>(p, 4);
    }
    __syncwarp();
  } else {
    // epilogue warps: TMEM lane quadrant = warp id mod 4; the two warps of a quadrant split the
    // 32 accumulator columns (tile rows m) in halves
    const int quad = warp & 3;
    const int half = (warp - C::EPI0) >> 2;
    const int epi_tid = (int)threadIdx.x - 32 * C::EPI0;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    const int m_first = half * C::COLS;
    const OutDesc od = out_desc(p);
    // staging tile of the TMA-store epilogue: behind the ring
    const uint32_t stage_u32 = ring_base + ring_bytes;
    uint16_t* stage_tile = reinterpret_cast<uint16_t*>(smem_raw + (stage_u32 - smem_u32(smem_raw)));
    bool store_pending = false;
    // the column scales and biases this role reads and the C it writes may be the previous kernel's; the index
    // of A may be read ahead of it when the caller vouches for A
    if (!p.a_stable) grid_dependency_wait();
    int begin, end, step;
    seg_range(p, begin, end, step);
    uint32_t it = 0;
    Seg seg_next = {};  // the next segment's descriptor is fetched one item ahead
    if (begin < end) seg_next = load_seg(p, begin);
    if (p.a_stable) grid_dependency_wait();
    if (epi_tid == 0) stamp<TRACE>(p, 0);
    for (int i = begin; i < end; i += step, ++it) {
      const Seg s = seg_next;
      if (i + step < end) seg_next = load_seg(p, i + step);
      const int npan = panels_in_chunk(p, s.chunk);
      const uint32_t buf = it & 1u, aph = (it >> 1) & 1u;
      const bool has = s.t1 > s.t0;
      // an empty tile row is zeros (+ bias): nothing to scale, no scales to wait for
      const float rs = (p.row_scale != nullptr && (has || s.nseg > 1)) ? __ldg(p.row_scale + s.row) : 1.0f;
      const int n_base = s.chunk * p.np * kPanelN + quad * 32 + lane;
      // per-column scale and bias of the first panel are fetched before the accumulator is ready
      float cs = p.b_scale, bias = 0.0f;
      if (n_base < p.N) {
        if (p.col_scale != nullptr && (has || s.nseg > 1)) cs = __ldg(p.col_scale + n_base) * p.b_scale;
        if (p.bias != nullptr) bias = __ldg(p.bias + n_base);
      }
      // a split row whose scratch index lies outside what the caller provided is skipped and reported
      const bool peers = p.n_peers > 0 && s.nseg > 1;
      const bool bad_split = s.nseg > 1 && (s.ctr < 0 || s.ctr >= p.ctr_limit || (peers && (unsigned)s.slot0 >= (unsigned)p.n_peers));
      int32_t* split_partials = p.partials;
      int32_t* split_counters = p.counters;
      if (peers && !bad_split) {
        split_partials = p.peer_partials[s.slot0];
        split_counters = p.peer_counters[s.slot0];
      }
      if (bad_split && epi_tid == 0 && p.status != nullptr) atomicCAS(p.status, 0, kStatusBadPlan);
      // one thread waits, the named barrier hands its verdict to all epilogue warps, so that they
      // leave the loop together if the wait gave up (a warp that went on alone would wait at the next
      // named barrier for ever)
      if (epi_tid == 0) ok_s[it & 1u] = mbar_wait(smem_u32(&bars.acc_full[buf]), aph, ctl) ? 1 : 0;
      asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_THREADS) : "memory");
      if (!ok_s[it & 1u]) break;
      if (epi_tid == 0 && i == begin) stamp<TRACE>(p, 5);
      if (epi_tid == 0) stamp<TRACE>(p, 8);
      tc_fence_after();
      const bool fast = s.nseg == 1 && od.acc_out == nullptr && p.worker_partials == nullptr;
#pragma unroll 1
      for (int q = 0; q < npan; ++q) {
        const int n = n_base + q * kPanelN;
        const uint32_t acc_addr = tmem_base + lane_sel + buf * acc_cols + (uint32_t)(q * 32 + m_first);
        if (fast) {
          // All of this warp's columns of the panel are requested at once and awaited once; the
          // accumulator buffer goes back to the MMA warp as soon as the values sit in registers.
          float csq = cs, biasq = bias;
          if (q > 0) {
            csq = p.b_scale; biasq = 0.0f;
            if (n < p.N) {
              if (p.col_scale != nullptr) csq = __ldg(p.col_scale + n) * p.b_scale;
              if (p.bias != nullptr) biasq = __ldg(p.bias + n);
            }
          }
          uint32_t r[C::COLS];
          if (has) {
            tmem_ld_cols<C::COLS>(acc_addr, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int k = 0; k < C::COLS; ++k) r[k] = 0u;
          }
          if (epi_tid == 0 && q == 0) stamp<TRACE>(p, 9);
          if (q == npan - 1) {  // this warp is done with the accumulator buffer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty[buf]));
          }
          if (!TR && p.tma_store == 2) {
            // 16-bit outputs, one store per epilogue warp: the warp puts its 32 x 32 part of the result tile
            // together in its own 2 KB of shared memory and sends it off itself - no barrier between the warps.
            // The copy engine clips at the edges of C; the part is free again once the previous store has read it.
            if (store_pending) {
              if (lane == 0) bulk_wait_read();
              __syncwarp();
            }
            uint16_t* part = stage_tile + quad * (32 * 32);
            if (!has && p.bias == nullptr && p.row_bias == nullptr) {
              // an empty tile row without bias is zeros under every activation: 2 KB of zero words, no conversions
              uint4* z = reinterpret_cast<uint4*>(part) + lane;
#pragma unroll
              for (int k = 0; k < 4; ++k) z[k * 32] = make_uint4(0u, 0u, 0u, 0u);
            } else {
#pragma unroll
              for (int c = 0; c < C::COLS; c += 16)
                finish16_stage<KIND, 32>(od, s.row, n, m_first + c, &r[c], rs, csq, biasq, part + lane);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_c, stage_u32 + (uint32_t)quad * (32 * 32 * 2), (s.chunk * p.np + q) * kPanelN + quad * 32,
                           s.row * kTile);
              bulk_commit();
            }
            store_pending = true;
          } else if (!TR && p.tma_store) {
            // 16-bit outputs: the 32 x 128 result tile is put together in shared memory and leaves in one
            // tiled store; the copy engine clips it at the edges of C.  The staging tile is free again once
            // the previous store has read it.
            if (store_pending) {
              if (epi_tid == 0) bulk_wait_read();
              asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_THREADS) : "memory");
            }
#pragma unroll
            for (int c = 0; c < C::COLS; c += 16)
              finish16_stage<KIND, kPanelN>(od, s.row, n, m_first + c, &r[c], rs, csq, biasq, stage_tile + quad * 32 + lane);
            fence_proxy_async_smem();
            asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_THREADS) : "memory");
            if (epi_tid == 0) {
              tma_store_2d(&tmap_c, stage_u32, (s.chunk * p.np + q) * kPanelN, s.row * kTile);
              bulk_commit();
            }
            store_pending = true;
          } else {
#pragma unroll
            for (int c = 0; c < C::COLS; c += 16) {
              if (TR) finish16_tr<KIND>(od, s.row, n, m_first + c, &r[c], rs, csq, biasq);
              else finish16<KIND>(od, s.row, n, m_first + c, &r[c], rs, csq, biasq);
            }
          }
          if (epi_tid == 0 && q == 0) stamp<TRACE>(p, 10);
          continue;
        }
        float csq = p.b_scale, biasq = 0.0f;
        if (n < p.N) {
          if (p.col_scale != nullptr) csq = __ldg(p.col_scale + n) * p.b_scale;
          if (p.bias != nullptr) biasq = __ldg(p.bias + n);
        }
        // (raw accumulators wanted, or a piece of a split row) all columns of the panel with one wait, then the
        // accumulator buffer goes back to the MMA warp
        uint32_t ra[C::COLS];
        if (has) {
          tmem_ld_cols<C::COLS>(acc_addr, ra);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int k = 0; k < C::COLS; ++k) ra[k] = 0u;
        }
        if (q == npan - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty[buf]));
        }
#pragma unroll
        for (int c = 0; c < C::COLS; c += 8) {
          const int m0 = m_first + c;
          uint32_t r[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) r[k] = ra[c + k];
          if (p.worker_partials != nullptr && n < p.N) {
            uint32_t* w = reinterpret_cast<uint32_t*>(p.worker_partials) + ((size_t)i * kTile + m0) * p.N + n;
#pragma unroll
            for (int k = 0; k < 8; ++k) w[(size_t)k * p.N] = r[k];
          }
          if (s.nseg == 1) {
            finish8<KIND>(od, s.row, n, m0, r, rs, csq, biasq);
          } else if (!bad_split && has) {
            // partial sum of a split row: added into the row's int32 accumulator in global memory
            // (integer adds commute, so the total does not depend on which CTA - or which GPU - comes first)
            int32_t* dst = split_partials + ((size_t)s.ctr * p.np + q) * (kTile * kPanelN) + (size_t)m0 * kPanelN +
                           (quad * 32 + lane);
            if (peers && p.peer_slots) {
              // this rank's own slot of the row: nothing else writes it, plain stores (NVLink writes for a remote owner)
              int32_t* slot = split_partials + (((size_t)s.ctr * p.n_peers + s.my_idx) * p.np + q) * (kTile * kPanelN) +
                              (size_t)m0 * kPanelN + (quad * 32 + lane);
#pragma unroll
              for (int k = 0; k < 8; ++k) slot[k * kPanelN] = (int32_t)r[k];
            } else if (p.n_peers > 0) {   // the accumulator may be another GPU's: system-wide adds over NVLink
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                if (KIND == VOID_KIND_I8) atomicAdd_system(dst + k * kPanelN, (int32_t)r[k]);
                else atomicAdd_system(reinterpret_cast<float*>(dst) + k * kPanelN, __uint_as_float(r[k]));
              }
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                if (KIND == VOID_KIND_I8) red_add_s32(dst + k * kPanelN, (int32_t)r[k]);
                else red_add_f32(reinterpret_cast<float*>(dst) + k * kPanelN, __uint_as_float(r[k]));
              }
            }
          }
        }
      }
      if (s.nseg > 1 && !bad_split && !(peers && p.peer_slots)) {
        // the CTA that arrives last reads the completed sums back and finishes the row
        if (epi_tid == 0) stamp<TRACE>(p, 12);
        // The arrival is one release-acquire add by one thread after a barrier of the epilogue warps: the barrier
        // orders every warp's additions before it, the release makes them visible before the count, and the
        // acquire lets the last arriver - after the second barrier - read what the other CTAs added.
        if (peers) __threadfence_system();
        asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_THREADS) : "memory");
        if (epi_tid == 0) stamp<TRACE>(p, 13);
        if (epi_tid == 0) {
          const int old = peers ? atomicAdd_system(split_counters + s.ctr, 1) : atom_add_acq_rel(split_counters + s.ctr, 1);
          const int last = (old == s.nseg - 1) ? 1 : 0;
          if (last) split_counters[s.ctr] = 0;  // left clean for the next launch
          last_s = last;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_THREADS) : "memory");
        const int last = last_s;
        asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_THREADS) : "memory");
        if (epi_tid == 0) stamp<TRACE>(p, 14);
        if (TRACE && epi_tid == 0 && p.trace != nullptr) p.trace[(size_t)blockIdx.x * 64 + 15] = (unsigned long long)last;
        if (last) {
          if (peers) __threadfence_system();
          if (epi_tid == 0) stamp<TRACE>(p, 28);
          OutDesc od2 = od;
          od2.acc_out = nullptr;
          if (peers) od2.out = p.peer_out[s.slot0];   // the owner's rows of C
#pragma unroll 1
          for (int q = 0; q < npan; ++q) {
            const int n = n_base + q * kPanelN;
            float csq = cs, biasq = bias;   // the first panel's were read before the accumulator was ready
            if (q > 0) {
              csq = p.b_scale; biasq = 0.0f;
              if (n < p.N) {
                if (p.col_scale != nullptr) csq = __ldg(p.col_scale + n) * p.b_scale;
                if (p.bias != nullptr) biasq = __ldg(p.bias + n);
              }
            }
            // all of this warp's sums of the panel are requested at once (one L2 round trip), then
            // the accumulator is cleared for the next launch
            int32_t* src = split_partials + ((size_t)s.ctr * p.np + q) * (kTile * kPanelN) + (size_t)m_first * kPanelN +
                           (quad * 32 + lane);
            uint32_t rl[C::COLS];
            if (TRACE && epi_tid == 0 && q == 0) { asm volatile("" ::"f"(csq), "f"(biasq) : "memory"); stamp<TRACE>(p, 29); }
#pragma unroll
            for (int k = 0; k < C::COLS; ++k)
              rl[k] = (uint32_t)(peers ? __ldcv(src + k * kPanelN) : __ldcg(src + k * kPanelN));
            if (TRACE && epi_tid == 0 && q == 0) { asm volatile("" ::"r"(rl[0]), "r"(rl[C::COLS - 1]) : "memory"); stamp<TRACE>(p, 30); }
            if (epi_tid == 0 && q == 0) stamp<TRACE>(p, 31);
            if (!TR && p.tma_store == 2 && !peers && od.acc_out == nullptr) {
              // 16-bit outputs leave as in the unsplit case: the warp's 32 x 32 part through shared memory and one tiled store
              if (store_pending) {
                if (lane == 0) bulk_wait_read();
                __syncwarp();
              }
              uint16_t* part = stage_tile + quad * (32 * 32);
#pragma unroll
              for (int c = 0; c < C::COLS; c += 16)
                finish16_stage<KIND, 32>(od, s.row, n, m_first + c, &rl[c], rs, csq, biasq, part + lane);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tmap_c, stage_u32 + (uint32_t)quad * (32 * 32 * 2), (s.chunk * p.np + q) * kPanelN + quad * 32,
                             s.row * kTile);
                bulk_commit();
              }
              store_pending = true;
              // (cleared after the store has been issued: the fence in front of it would wait for these writes)
#pragma unroll
              for (int k = 0; k < C::COLS; ++k) src[k * kPanelN] = 0;
              continue;
            }
#pragma unroll
            for (int k = 0; k < C::COLS; ++k) src[k * kPanelN] = 0;
#pragma unroll
            for (int c = 0; c < C::COLS; c += 16) {
              if (od.acc_out != nullptr && n < od.N) {
                uint32_t* a = reinterpret_cast<uint32_t*>(od.acc_out) + ((size_t)s.row * kTile + m_first + c) * od.N + n;
#pragma unroll
                for (int k = 0; k < 16; ++k) a[(size_t)k * od.N] = rl[c + k];
              }
              finish16<KIND>(od2, s.row, n, m_first + c, &rl[c], rs, csq, biasq);
            }
          }
        }
      }
    }
    // the staging tile must have been read before shared memory is given back; the writes themselves
    // complete with the kernel
    if (store_pending && (p.tma_store == 2 ? lane == 0 : epi_tid == 0)) bulk_wait_read();
    if (epi_tid == 0) stamp<TRACE>(p, 6);
  }
  pipeline_teardown<C, TRACE>(p, ctl_s, tmem_base, tmem_cols);
}

// ------------------------------------------------------------------------------------------
// Per-tile drain kernel: every tile's product is scaled by that tile's scale.
// ------------------------------------------------------------------------------------------
template <int KIND, int NP, class C, bool TRACE = false>
__global__ void __launch_bounds__(C::THREADS, (NP == 4) ? 1 : C::CTAS_PER_SM) spmm_drain_kernel(const __grid_constant__ CUtensorMap tmap_b,
                                                              const __grid_constant__ SpmmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ PipeBars bars;
  __shared__ uint32_t tmem_base_s;
  __shared__ int ctl_s[2];   // abort flag, wait limit in ms

  // Tensor memory is cut into slot groups: one group receives the products of the tiles of one ring
  // stage (up to p.group tiles, NP panels each), so that MMA warp and epilogue hand over once per
  // stage, not once per tile.
  constexpr uint32_t kTileCols = NP * 32;   // TMEM columns of one tile's product
  const uint32_t kTmemCols = (uint32_t)p.tmem_cols;
  constexpr int CW = C::COLS;
  // Products are read back in batches of 32 registers per thread with ONE wait per batch: both halves of a
  // tile for a warp that owns all 32 accumulator columns, the halves of two tiles for a warp that owns 16.
  // A read of tensor memory is a round trip of a few hundred cycles whatever its width, and the fold that
  // follows depends on it, so the number of round trips per tile is what this role's speed hangs on.
  constexpr int TPW = 32 / CW;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t ring_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_bytes = (uint32_t)(p.group * (NP * kPanelBytes + kTileBytes));
  const uint32_t group_cols = (uint32_t)p.group * kTileCols;
  const int n_slots = (int)(kTmemCols / group_cols);   // >= 2: checked at launch
  volatile int* ctl = ctl_s;

  pipeline_setup<C, 1, TRACE>(p, &tmap_b, bars, &tmem_base_s, ctl_s, n_slots, kTmemCols);
  const uint32_t tmem_base = tmem_base_s;

  if (warp < C::PW) {
    producer_loop<C, 1, false, TRACE>(p, &tmap_b, &bars, ring_base, stage_bytes, ctl, lane, warp);
    if (warp == 0 && lane == 0) stamp<TRACE>(p, 2);
  } else if (warp == C::MMA) {
    {
      // as in the row-accumulate kernel: the warp walks the loop together, one elected lane issues
      const bool leader = elect_one();
      if (!p.a_stable) grid_dependency_wait();
      const uint32_t idesc = p.idesc;
      const uint64_t hi_a = p.desc_hi_a, hi_b = p.desc_hi_b;
      const int G = p.group, S = p.stages;   // (the per-tile kernel runs with stages of equal size)
      const uint32_t tiles_at = (uint32_t)(G * NP) * kPanelBytes;
      constexpr uint64_t kPanelStep = kPanelBytes >> 4, kTileStep = kTileBytes >> 4;
      int begin, end, step;
      seg_range(p, begin, end, step);
      int stage = 0, slot = 0;
      uint32_t phase = 0, sphase = 0;
      uint32_t sbase = ring_base;
      bool ok = true;
      Seg seg_next = {};  // the next segment's descriptor is fetched one item ahead
      if (begin < end) seg_next = load_seg(p, begin);
      for (int i = begin; i < end && ok; i += step) {
        const Seg s = seg_next;
        if (i + step < end) seg_next = load_seg(p, i + step);
        const int npan = panels_in_chunk(p, s.chunk);
        for (int t = s.t0; t < s.t1; t += G) {
          const int gcnt = (s.t1 - t) < G ? (s.t1 - t) : G;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.full[stage]), phase, ctl));
          if (!ok) break;
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.acc_empty[slot]), sphase ^ 1u, ctl));
          if (!ok) break;
          tc_fence_after();
          uint64_t ad = smem_desc(hi_a, sbase);
          uint64_t bd = smem_desc(hi_b, sbase + tiles_at);
          uint32_t d = tmem_base + (uint32_t)slot * group_cols;
          for (int j = 0; j < gcnt; ++j) {
            uint64_t adq = ad;
            uint32_t dq = d;
            for (int q = 0; q < npan; ++q) {
              if (leader) issue_mma<KIND>(dq, adq, bd, idesc, 0u);
              adq += kPanelStep;
              dq += 32u;
            }
            ad += kPanelStep * (uint64_t)NP;
            bd += kTileStep;
            d += kTileCols;
          }
          if (leader) {
            tc_commit(smem_u32(&bars.acc_full[slot]));
            tc_commit(smem_u32(&bars.empty[stage]));
          }
          if (++slot == n_slots) { slot = 0; sphase ^= 1u; }
          sbase += stage_bytes;
          if (++stage == S) { stage = 0; phase ^= 1u; sbase = ring_base; }
        }
      }
      if (leader) stamp<TRACE>(p, 4);
    }
    __syncwarp();
  } else {
    const int quad = warp & 3;
    const int half = (warp - C::EPI0) >> 2;
    const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
    const int m_first = half * CW;
    const int G = p.group;
    grid_dependency_wait();
    int begin, end, step;
    seg_range(p, begin, end, step);
    int slot = 0;
    uint32_t sphase = 0;
    bool alive = true;
    Seg seg_next = {};  // the next segment's descriptor is fetched one item ahead
    if (begin < end) seg_next = load_seg(p, begin);
    for (int i = begin; i < end && alive; i += step) {
      const Seg s = seg_next;
      if (i + step < end) seg_next = load_seg(p, i + step);
      const int npan = panels_in_chunk(p, s.chunk);
      float acc[NP][CW];
#pragma unroll
      for (int q = 0; q < NP; ++q)
#pragma unroll
        for (int m = 0; m < CW; ++m) acc[q][m] = 0.0f;
      for (int t = s.t0; t < s.t1; t += G) {
        const int gcnt = (s.t1 - t) < G ? (s.t1 - t) : G;
        // scale of lane j's tile, fetched before the products are ready
        const float my_ts = (lane < gcnt) ? __ldg(p.tile_scales + t + lane) : 0.0f;
        int ok = 1;
        if (lane == 0) ok = mbar_wait(smem_u32(&bars.acc_full[slot]), sphase, ctl) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { alive = false; break; }
        tc_fence_after();
        const uint32_t slot_addr = tmem_base + lane_sel + (uint32_t)slot * group_cols + (uint32_t)m_first;
        for (int j = 0; j < gcnt; j += TPW) {
#pragma unroll
          for (int q = 0; q < NP; ++q) {
            if (q < npan) {
              uint32_t r[TPW][CW];
#pragma unroll
              for (int u = 0; u < TPW; ++u) {
                if (j + u < gcnt) {
#pragma unroll
                  for (int c = 0; c < CW; c += 16)
                    tmem_ld_32x16p(slot_addr + (uint32_t)(j + u) * kTileCols + (uint32_t)(q * 32 + c), &r[u][c]);
                }
              }
              tmem_ld_wait();
              if (j + TPW >= gcnt && q == npan - 1) {  // this warp has read the whole slot group
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty[slot]));
              }
#pragma unroll
              for (int u = 0; u < TPW; ++u) {
                if (j + u < gcnt) {   // tiles are folded in their stored order, one after the other
                  const float ts = __shfl_sync(0xffffffffu, my_ts, j + u);
#pragma unroll
                  for (int m = 0; m < CW; ++m) {
                    const float x = (KIND == VOID_KIND_I8) ? __int2float_rn((int)r[u][m]) : __uint_as_float(r[u][m]);
                    acc[q][m] = fmaf(ts, x, acc[q][m]);
                  }
                }
              }
            }
          }
        }
        if (++slot == n_slots) { slot = 0; sphase ^= 1u; }
      }
      if (!alive) break;
      const OutDesc od = out_desc(p);   // read here, not before the loop: registers are what this role is short of
      const int n_base = s.chunk * NP * kPanelN + quad * 32 + lane;
#pragma unroll
      for (int q = 0; q < NP; ++q) {
        if (q < npan) {
          const int n = n_base + q * kPanelN;
          if (n < p.N) {
            if (p.acc_out != nullptr) {
              float* a = reinterpret_cast<float*>(p.acc_out) + ((size_t)s.row * kTile + m_first) * p.N + n;
#pragma unroll
              for (int m = 0; m < CW; ++m) a[(size_t)m * p.N] = acc[q][m];
            }
            const float cs = (p.col_scale != nullptr) ? __ldg(p.col_scale + n) * p.b_scale : p.b_scale;
            const float bias = (p.bias != nullptr) ? __ldg(p.bias + n) : 0.0f;
#pragma unroll
            for (int c = 0; c < CW; c += 8) {
              float v[8];
#pragma unroll
              for (int k = 0; k < 8; ++k) v[k] = acc[q][c + k] * cs + bias;
              store8(od, s.row, n, m_first + c, v);
            }
          }
        }
      }
    }
    if (threadIdx.x == 32 * C::EPI0) stamp<TRACE>(p, 6);
  }
  pipeline_teardown<C, TRACE>(p, ctl_s, tmem_base, kTmemCols);
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

struct DeviceInfo {
  int sms = 0, cc_major = 0, cc_minor = 0, max_smem = 0, smem_per_sm = 0;
  bool ok = false;
};
static DeviceInfo device_info() {
  static DeviceInfo cache[64];
  static std::mutex mu;
  int dev = 0;
  DeviceInfo none;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return none;
  std::lock_guard<std::mutex> lock(mu);   // a record is filled and read under the lock: no half-written fields
  if (!cache[dev].ok) {
    DeviceInfo d;
    if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return none;
    cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&d.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    d.ok = true;
    cache[dev] = d;
  }
  return cache[dev];
}

// cudaFuncSetAttribute per (kernel, device), repeated only when a larger ring is asked for.
// All kernels share one C++ function-pointer type, so the record is keyed by the pointer value.  The table
// holds every instantiation of this file on up to 16 devices; beyond that the attribute is simply set again
// on every launch of the pairs that found no room (correct, a little slower).
static int ensure_smem(const void* kernel, int bytes) {
  struct Rec { const void* fn; int dev; int bytes; };
  constexpr int kRecs = 48 * 16;
  static Rec recs[kRecs];
  static int n_recs = 0;
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  std::lock_guard<std::mutex> lock(mu);
  Rec* r = nullptr;
  for (int i = 0; i < n_recs; ++i)
    if (recs[i].fn == kernel && recs[i].dev == dev) r = &recs[i];
  if (r != nullptr && r->bytes >= bytes) return 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return -1;
  if (r == nullptr && n_recs < kRecs) r = &recs[n_recs++];
  if (r != nullptr) { r->fn = kernel; r->dev = dev; r->bytes = bytes; }
  return 0;
}

template <typename Kernel, typename... Args>
static void launch_pdl(Kernel kernel, int grid, int threads, int smem_bytes, cudaStream_t stream, const Args&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, args...);
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
  if (a->segs != nullptr && a->partials_bytes > 0 && a->n_peers == 0 && (a->partials == nullptr || a->counters == nullptr))
    return VOID_ERR_BAD_ARG;
  if ((long long)a->nbr * kTile < a->M) return VOID_ERR_SHAPE;
  const bool tr = a->transposed != 0;
  if (a->transposed != 0 && a->transposed != 1) return VOID_ERR_BAD_ARG;
  if (a->ldc < (tr ? a->M : a->N)) return VOID_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a->tiles) & 1023u) != 0) return VOID_ERR_ALIGN;
  if (kind < VOID_KIND_I8 || kind > VOID_KIND_TF32) return VOID_ERR_BAD_ARG;
  const int es = (kind == VOID_KIND_TF32) ? 4 : ((kind == VOID_KIND_F16 || kind == VOID_KIND_BF16) ? 2 : 1);
  const bool floating = es > 1;
  if ((reinterpret_cast<uintptr_t>(a->b) & 15u) != 0 || (a->ldb & 15) != 0 ||
      a->ldb < (long long)(tr ? a->K : a->N) * es)
    return VOID_ERR_ALIGN;
  // transposed operands: row-accumulate kernel without a plan or raw-accumulator outputs
  if (tr && (kind == VOID_KIND_F8E4M3 || a->scale_mode != VOID_SCALE_ROW_MEAN || a->segs != nullptr ||
             a->acc_out != nullptr || a->worker_partials != nullptr))
    return VOID_ERR_BAD_ARG;
  if (floating && (a->scale_mode != VOID_SCALE_ROW_MEAN || a->row_scale != nullptr)) return VOID_ERR_BAD_ARG;

  const DeviceInfo dev = device_info();
  if (!dev.ok) return VOID_ERR_CUDA;
  if (dev.cc_major != 10) return VOID_ERR_ARCH;

  const bool drain = (a->scale_mode == VOID_SCALE_PER_TILE);
  const int total_panels = (a->N + kPanelN - 1) / kPanelN;
  int np = a->panels_per_item;
  if (np != 0 && np != 1 && np != 2 && np != 4) return VOID_ERR_BAD_ARG;
  if (floating && np > 2) return VOID_ERR_BAD_ARG;  // ring stages of wider items do not fit
  if (np == 0 && floating) np = 1;
  if (np == 0) {
    // two panels per item keep two CTAs on an SM, which measured faster than four panels with one
    np = total_panels >= 2 ? 2 : 1;
    if (a->segs == nullptr) {  // keep enough work items to fill the machine
      while (np > 1 && (long long)a->nbr * ((total_panels + np - 1) / np) < 4ll * dev.sms) np >>= 1;
    }
  }
  const int n_chunks = (total_panels + np - 1) / np;
  // CTA shape: the slim one (four CTAs per SM) for the row-accumulate kernel with at most two panels
  // per item; the wide one for the per-tile kernel and for four-panel items (TMEM: 2 x np x 32
  // columns per row-accumulate CTA, 512 per SM)
  int shape = a->cta_shape;
  if (shape < 0 || shape > 5) return VOID_ERR_BAD_ARG;
  if (tr && np > 2) return VOID_ERR_BAD_ARG;
  if (tr && shape == 1) return VOID_ERR_BAD_ARG;  // built for the slim shape only
  if (shape == 0) shape = (!drain && np <= 2) ? 2 : ((drain && np == 1) ? kDefaultDrainShape : 1);
  if (shape == 2 && (np > 2 || (drain && np > 1))) return VOID_ERR_BAD_ARG;
  if (shape >= 3 && (!drain || np != 1 || tr)) return VOID_ERR_BAD_ARG;  // shapes of the per-tile kernel
  const bool slim = (shape == 2);
  const int producer_warps = (shape == 1) ? Wide::PW : ((shape >= 4) ? 1 : Slim::PW);
  const int ctas_per_sm = (slim || shape == 5) ? 4 : (shape >= 3 ? 3 : ((np == 4) ? 1 : Wide::CTAS_PER_SM));
  int group = a->tiles_per_stage;  // 0 = default
  // What a CTA streams is bounded by the bytes its ring keeps in flight over a stage's round trip, so the defaults fill
  // the shared memory four CTAs per SM leave each other: nine (tile + panel) units as 3 stages x 3 for one 8-bit panel per
  // item (swept on B200, headline / 70 % / 16384^2: 2 x 4 units 7.02 / 11.06 / 69.9 us, 3 x 3: 6.76 / 10.21 / 65.1,
  // 4 x 2: 6.96 / 10.87 / 69.4, 9 x 1: 8.64 / 16.2 / 111); stages of one or two tiles pay the fixed cost of a stage too often
  if (group == 0) group = (np == 1) ? 3 : 2;
  if (a->tiles_per_stage == 0 && floating) group = (es == 2 && np == 1) ? 2 : 1;
  // wider tiles (an FP8 tile stored as two or three terms): 3 stages x 2 (headline 7.66 us, 2 x 3: 7.93)
  if (a->tiles_per_stage == 0 && a->tile_terms > 1) group = (np == 1) ? 2 : 1;
  if (group < 1 || group > 8) return VOID_ERR_BAD_ARG;
  if (drain && np == 1 && shape != 1 && a->tiles_per_stage == 0) group = 2;
  int drain_tmem = 32;   // the largest power of two that lets ctas_per_sm CTAs share the SM's 512 columns
  while (drain_tmem * 2 * ctas_per_sm <= 512) drain_tmem *= 2;
  if (drain && group * np * 32 * 2 > drain_tmem) return VOID_ERR_BAD_ARG;  // two slot groups of products in TMEM
  int terms = a->tile_terms == 0 ? 1 : a->tile_terms;
  if (terms < 1 || terms > 3) return VOID_ERR_BAD_ARG;
  if (terms > 1 && (kind != VOID_KIND_F8E4M3 || drain || tr)) return VOID_ERR_BAD_ARG;  // FP8 row-accumulate only
  // 16-bit outputs of the slim row-accumulate kernel leave through a staging tile (32 x 128 x 2 bytes behind the
  // ring) and a tiled TMA store, when C qualifies as a tensor for the copy engine (16-byte aligned base and pitch)
  // (with a plan, whole-row segments take this route and the pieces of split rows the ordinary one)
  const bool tma_store = !drain && !tr && slim && a->acc_out == nullptr &&
                         a->worker_partials == nullptr && (a->flags & 2) == 0 &&
                         (a->out_dtype == VOID_OUT_F16 || a->out_dtype == VOID_OUT_BF16) &&
                         (reinterpret_cast<uintptr_t>(a->out) & 15u) == 0 && ((a->ldc * 2) & 15) == 0;
  const int stage_bytes = group * (np * kPanelBytes + kTileBytes * terms) * es;
  const int staging_bytes = tma_store ? kTile * kPanelN * 2 : 0;
  int stages = a->stages;
  if (stages == 0) {
    // dynamic shared memory a CTA may use so that ctas_per_sm of them fit an SM: the SM's bytes less the kilobyte
    // the system keeps per CTA and the kernel's static variables, less this kernel's 1 KB of slack for alignment
    // and the staging tile
    const int budget = dev.smem_per_sm / ctas_per_sm - 1024 - 640 - 1024 - staging_bytes;
    stages = budget / stage_bytes;
    if (stages > 8) stages = 8;
  }
  // The shared memory the full stages leave over becomes a shorter last stage (row-accumulate kernel, ring sized
  // here) when it adds at least a fifth to the tiles in flight: 2 + 2 + 1 tiles of two 8-bit panels each take 63.8 us
  // at 16384^2 and 64.0 on an eight-rank shard of 65536^2 against 68.9 and 70.8 with 2 + 2; a seventh tile behind
  // 3 x 2 FP8 tiles of two terms costs more in stage turns than it brings (7.49 against 7.44 us, 13.54 against 13.25)
  int last_group = group;
  if (a->stages == 0 && !drain) {
    const int budget = dev.smem_per_sm / ctas_per_sm - 1024 - 640 - 1024 - staging_bytes;
    const int left = (budget - stages * stage_bytes) / (stage_bytes / group);
    if (left >= 1 && 5 * left >= stages * group && stages < kMaxStages) {
      last_group = left < group ? left : group;
      stages += 1;
    }
  }
  // A producer warp may run up to (producer warps - 1) groups ahead of the consumer's order; the
  // parity of a ring barrier only tells two consecutive uses of a stage apart, so the ring must
  // hold at least one stage per producer warp.
  if (stages < producer_warps || stages > kMaxStages) return VOID_ERR_BAD_ARG;
  const int smem_bytes = ((stages - 1) * group + last_group) * (stage_bytes / group) + 1024 + staging_bytes;
  if (smem_bytes > dev.max_smem) return VOID_ERR_SHAPE;

  SpmmParams p;
  p.tiles = a->nnz > 0 ? reinterpret_cast<const uint8_t*>(a->tiles) : nullptr;  // null: no tensor map either
  p.tile_cols = a->tile_cols;
  p.tile_scales = a->tile_scales;
  p.row_ptr = a->row_ptr;
  p.row_order = a->segs == nullptr ? a->row_order : nullptr;
  p.row_scale = a->row_scale;
  p.nbr = a->nbr;
  p.nbc = a->nbc;
  p.nnz = a->nnz;
  p.n_chunks = n_chunks;
  p.N = a->N;
  p.M = a->M;
  p.col_scale = a->col_scale;
  p.b_scale = a->b_scale;
  p.bias = a->bias;
  p.row_bias = a->row_bias;
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
  p.n_peers = a->n_peers;
  p.peer_slots = a->peer_slots ? 1 : 0;
  if (a->n_peers < 0 || a->n_peers > 8) return VOID_ERR_BAD_ARG;
  if (a->peer_slots != 0 && (a->n_peers == 0 || kind != VOID_KIND_I8)) return VOID_ERR_BAD_ARG;
  if (a->n_peers > 0) {
    // reduction across GPUs: a plan whose segments name the owner of their tile row; INT8 / floating row-accumulate
    if (a->segs == nullptr || drain || tr || a->acc_out != nullptr || a->worker_partials != nullptr) return VOID_ERR_BAD_ARG;
    for (int r = 0; r < a->n_peers; ++r) {
      if (a->peer_partials[r] == nullptr) return VOID_ERR_BAD_ARG;
      if (!a->peer_slots && (a->peer_counters[r] == nullptr || a->peer_out[r] == nullptr)) return VOID_ERR_BAD_ARG;
      p.peer_partials[r] = reinterpret_cast<int32_t*>(a->peer_partials[r]);
      p.peer_counters[r] = a->peer_counters[r];
      p.peer_out[r] = a->peer_out[r];
    }
  }
  p.trace = reinterpret_cast<unsigned long long*>(a->trace);
  p.np = np;
  p.terms = terms;
  p.group = group;
  p.stages = stages;
  p.last_group = last_group;
  p.use3d = (!tr && a->N % (kPanelN / es) == 0) ? 1 : 0;
  p.tmem_cols = drain_tmem;
  p.tma_store = tma_store ? ((a->flags & 16) ? 1 : 2) : 0;   // 2: one store per epilogue warp; 1: one per tile
  p.n_items = a->nbr * n_chunks;
  p.a_stable = (a->flags & 4) ? 1 : 0;
  // room of the split-row scratch, in rows: the kernel refuses segments whose counter index lies beyond it
  p.ctr_limit = 0;
  if (a->segs != nullptr && ((a->partials != nullptr && a->counters != nullptr) || a->n_peers > 0) && a->partials_bytes > 0) {
    const long long per_row = (long long)np * kPanelN * kTile * (long long)sizeof(int32_t) * (a->peer_slots ? a->n_peers : 1);
    const long long rows = a->partials_bytes / per_row;
    p.ctr_limit = rows > 0x7fffffffll ? 0x7fffffff : (int)rows;
  }
  // test hooks (args->test_hooks): bits 0..15 = limit of every device-side wait in milliseconds (0: the
  // default), bit 16 = the producers never deliver the first group of tiles of each CTA
  p.wait_limit_ms = (a->test_hooks & 0xffff) ? (a->test_hooks & 0xffff) : kDefaultWaitLimitMs;
  p.drop_group = (a->test_hooks >> 16) & 1;
  if (a->trace != nullptr && !((kind == VOID_KIND_I8 && !drain && slim && !tr) ||
                               (kind == VOID_KIND_F8E4M3 && drain && np == 1 && shape >= 2)))
    return VOID_ERR_BAD_ARG;   // time stamps exist in the diagnostic instantiations only

  // Operand descriptors.  Packed tile (instruction operand B, K-major, no swizzle): 8x16-byte core
  // matrices, 128 bytes between the two k-halves (leading offset), 256 bytes between 8-row groups
  // (stride offset).  B panel (operand A, MN-major, 128-byte swizzle): one swizzle atom along n,
  // four 8-row groups along k, 1024 bytes apart.
  p.desc_hi_b = smem_desc_hi(128, 256, kLayoutNone);
  // Wider elements: the tile's row groups are 256 * es bytes apart; the panel is es swizzle atoms wide
  // along n, 4096 bytes apart (leading offset), its 8-row k groups stay 1024 bytes apart.
  // 32-bit elements in an MN-major operand need the swizzle that permutes 32-byte pieces of a 128-byte
  // row (pattern of 4 rows, so k groups of 4 rows, 512 bytes apart); the copy engine writes the same
  // pattern with its 32-byte-atom mode.
  if (floating) {
    p.desc_hi_b = smem_desc_hi(128, 256 * es, kLayoutNone);
    p.desc_hi_a = (es == 4) ? smem_desc_hi(4096, 512, kLayoutSw128Base32) : smem_desc_hi(4096, 1024, kLayoutSw128);
  } else {
    p.desc_hi_a = smem_desc_hi(1024, 1024, kLayoutSw128);
  }
  // Transposed B ([N, K], k contiguous) is a K-major operand: rows of 32 * es bytes (one swizzle span of 32,
  // 64 or 128 bytes), groups of 8 rows 256 * es bytes apart.
  const uint32_t a_mn = tr ? 0u : 1u;
  if (tr) p.desc_hi_a = smem_desc_hi(16, 256 * es, es == 4 ? kLayoutSw128 : (es == 2 ? kLayoutSw64 : kLayoutSw32));
  if (kind == VOID_KIND_I8) p.idesc = instr_desc(/*c s32*/ 2, /*a s8*/ 1, /*b s8*/ 1, a_mn, /*b K*/ 0, 128, 32);
  else if (kind == VOID_KIND_F8E4M3) p.idesc = instr_desc(/*c f32*/ 1, /*a e4m3*/ 0, /*b e4m3*/ 0, a_mn, 0, 128, 32);
  else if (kind == VOID_KIND_F16) p.idesc = instr_desc(1, /*a f16*/ 0, /*b f16*/ 0, a_mn, 0, 128, 32);
  else if (kind == VOID_KIND_BF16) p.idesc = instr_desc(1, /*a bf16*/ 1, /*b bf16*/ 1, a_mn, 0, 128, 32);
  else p.idesc = instr_desc(1, /*a tf32*/ 2, /*b tf32*/ 2, a_mn, 0, 128, 32);

  int grid;
  if (a->segs != nullptr) {
    if (a->cta_seg_ptr == nullptr || a->n_cta <= 0 || a->panels_per_item == 0) return VOID_ERR_BAD_ARG;
    if (drain || kind == VOID_KIND_F8E4M3) return VOID_ERR_BAD_ARG;  // split rows: row-accumulate kernel only
    grid = a->n_cta;
  } else {
    grid = a->grid > 0 ? a->grid : dev.sms * ctas_per_sm;
    if (grid > p.n_items) grid = p.n_items;
    if (grid < 1) grid = 1;
  }

  // B as a tensor for the copy engine, 128-byte swizzle, zero fill outside [K, N]:
  //   3-D (N a multiple of 128): dim0 = 128 columns of a panel, dim1 = k, dim2 = panel; box 128 x 32 x np
  //   2-D (ragged N):            dim0 = n, dim1 = k;                                      box 128 x 32
  CUtensorMap tmap;
  memset(&tmap, 0, sizeof(tmap));
  if (a->nnz > 0) {
    PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode();
    if (enc == nullptr) return VOID_ERR_CUDA;
    CUresult r = CUDA_ERROR_INVALID_VALUE;
    // elements of es bytes: every box is 128 bytes (kPanelN / es columns) wide, a panel takes es of them
    const CUtensorMapDataType dt = (es == 1) ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : (es == 2) ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    const int box_n = kPanelN / es;
    const CUtensorMapSwizzle swz = (es == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    if (tr) {
      //   transposed: dim0 = k, dim1 = n; box 32 k x 128 n, swizzle span = the 32 * es bytes of a row
      const cuuint64_t gdim[2] = {(cuuint64_t)a->K, (cuuint64_t)a->N};
      const cuuint64_t gstride[1] = {(cuuint64_t)a->ldb};
      const cuuint32_t box[2] = {(cuuint32_t)kTile, (cuuint32_t)kPanelN};
      const cuuint32_t estride[2] = {1, 1};
      const CUtensorMapSwizzle sw = (es == 4) ? CU_TENSOR_MAP_SWIZZLE_128B
                                    : (es == 2) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
      r = enc(&tmap, dt, 2, const_cast<void*>(a->b), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (p.use3d) {
      const cuuint64_t gdim[3] = {(cuuint64_t)box_n, (cuuint64_t)a->K, (cuuint64_t)(a->N / box_n)};
      const cuuint64_t gstride[2] = {(cuuint64_t)a->ldb, (cuuint64_t)kPanelN};
      const cuuint32_t box[3] = {(cuuint32_t)box_n, (cuuint32_t)kTile, (cuuint32_t)(np * es)};
      const cuuint32_t estride[3] = {1, 1, 1};
      r = enc(&tmap, dt, 3, const_cast<void*>(a->b), gdim, gstride, box, estride,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) p.use3d = 0;  // fall back to one 2-D copy per panel
    }
    if (!p.use3d && !tr) {
      const cuuint64_t gdim[2] = {(cuuint64_t)a->N, (cuuint64_t)a->K};
      const cuuint64_t gstride[1] = {(cuuint64_t)a->ldb};
      const cuuint32_t box[2] = {(cuuint32_t)box_n, (cuuint32_t)kTile};
      const cuuint32_t estride[2] = {1, 1};
      r = enc(&tmap, dt, 2, const_cast<void*>(a->b), gdim, gstride, box, estride,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return VOID_ERR_TENSOR_MAP;
  }

  CUtensorMap tmap_c;
  memset(&tmap_c, 0, sizeof(tmap_c));
  if (tma_store) {
    PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode();
    if (enc == nullptr) return VOID_ERR_CUDA;
    const cuuint64_t gdim[2] = {(cuuint64_t)a->N, (cuuint64_t)a->M};
    const cuuint64_t gstride[1] = {(cuuint64_t)a->ldc * 2};
    const cuuint32_t box[2] = {(cuuint32_t)((a->flags & 16) ? kPanelN : 32), (cuuint32_t)kTile};
    const cuuint32_t estride[2] = {1, 1};
    if (enc(&tmap_c, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a->out, gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return VOID_ERR_TENSOR_MAP;
  }

#define VB_LAUNCH(KERNEL, SHAPE)                                                               \
  do {                                                                                        \
    if (ensure_smem((const void*)KERNEL, smem_bytes)) return VOID_ERR_CUDA;                   \
    launch_pdl(KERNEL, grid, SHAPE::THREADS, smem_bytes, stream, tmap, p);                    \
  } while (0)
#define VB_LAUNCH_ROWACC(KERNEL, SHAPE)                                                        \
  do {                                                                                        \
    if (ensure_smem((const void*)KERNEL, smem_bytes)) return VOID_ERR_CUDA;                   \
    launch_pdl(KERNEL, grid, SHAPE::THREADS, smem_bytes, stream, tmap, tmap_c, p);            \
  } while (0)
  const bool traced = a->trace != nullptr;
  if (tr) {
    if (kind == VOID_KIND_TF32) VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_TF32, Slim, true>), Slim);
    else if (kind == VOID_KIND_I8) VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_I8, Slim, true>), Slim);
    else VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_F16, Slim, true>), Slim);
  } else if (floating) {
    if (kind == VOID_KIND_TF32) {
      if (slim) VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_TF32, Slim>), Slim);
      else VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_TF32, Wide>), Wide);
    } else {  // fp16 and bf16 differ in the instruction descriptor only
      if (slim) VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_F16, Slim>), Slim);
      else VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_F16, Wide>), Wide);
    }
  } else if (!drain) {
    if (kind == VOID_KIND_I8) {
      if (slim && traced) VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_I8, Slim, false, true>), Slim);
      else if (slim) VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_I8, Slim>), Slim);
      else VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_I8, Wide>), Wide);
    } else {
      if (slim) VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_F8E4M3, Slim>), Slim);
      else VB_LAUNCH_ROWACC((spmm_rowacc_kernel<VOID_KIND_F8E4M3, Wide>), Wide);
    }
  } else if (kind == VOID_KIND_I8) {
    if (np == 1 && shape == 2) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_I8, 1, Slim>), Slim);
    else if (np == 1 && shape == 3) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_I8, 1, Slim3>), Slim3);
    else if (np == 1 && shape == 4) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_I8, 1, Drain8>), Drain8);
    else if (np == 1 && shape == 5) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_I8, 1, Slim1>), Slim1);
    else if (np == 1) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_I8, 1, Wide>), Wide);
    else if (np == 2) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_I8, 2, Wide>), Wide);
    else VB_LAUNCH((spmm_drain_kernel<VOID_KIND_I8, 4, Wide>), Wide);
  } else {
    if (np == 1 && shape == 2 && traced) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Slim, true>), Slim);
    else if (np == 1 && shape == 3 && traced) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Slim3, true>), Slim3);
    else if (np == 1 && shape == 4 && traced) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Drain8, true>), Drain8);
    else if (np == 1 && shape == 5 && traced) return VOID_ERR_BAD_ARG;
    else if (np == 1 && shape == 2) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Slim>), Slim);
    else if (np == 1 && shape == 3) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Slim3>), Slim3);
    else if (np == 1 && shape == 4) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Drain8>), Drain8);
    else if (np == 1 && shape == 5) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Slim1>), Slim1);
    else if (np == 1) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 1, Wide>), Wide);
    else if (np == 2) VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 2, Wide>), Wide);
    else VB_LAUNCH((spmm_drain_kernel<VOID_KIND_F8E4M3, 4, Wide>), Wide);
  }
#undef VB_LAUNCH
#undef VB_LAUNCH_ROWACC
  return cudaGetLastError() == cudaSuccess ? VOID_OK : VOID_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------
// Built-in scratch for callers that cannot allocate device memory.
// ------------------------------------------------------------------------------------------
// int32 accumulators of split tile rows followed by their arrival counters.  The array lives in the
// library's device image: every GPU that loads the library holds these bytes until the process
// exits.
constexpr size_t kStaticPartialsBytes = 8u << 20;    // 8 MiB of int32 row accumulators
constexpr int kStaticCounters = 4096;                // arrival counters (16 KiB)
static __device__ __align__(256) unsigned char g_static_scratch[kStaticPartialsBytes + kStaticCounters * 4];

// Device address of g_static_scratch on the current device.  In host code the array's name is only
// a handle for the runtime, not an address a kernel could use; the address has to be asked for,
// once per device, with that device current.
static int static_scratch_ptr(unsigned char** out) {
  static unsigned char* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return VOID_ERR_CUDA;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return VOID_ERR_CUDA;
    ptrs[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = ptrs[dev];
  return VOID_OK;
}

static int spmm_i8_static_scratch(const void_spmm_args* a, int32_t n_split_rows, cudaStream_t stream) {
  if (a == nullptr || n_split_rows < 0) return VOID_ERR_BAD_ARG;
  if (a->segs == nullptr || a->panels_per_item == 0) return VOID_ERR_BAD_ARG;  // a split-row plan is the point
  const size_t acc_bytes = (size_t)a->panels_per_item * kPanelN * kTile * sizeof(int32_t);  // one split row
  if ((size_t)n_split_rows * acc_bytes > kStaticPartialsBytes || n_split_rows > kStaticCounters) return VOID_ERR_TOO_LARGE;
  unsigned char* base = nullptr;
  const int st = static_scratch_ptr(&base);
  if (st != VOID_OK) return st;
  void_spmm_args b = *a;
  b.partials = base;
  // the room the kernel may use is what this call clears: a segment of the plan whose counter index is
  // n_split_rows or more is skipped and reported through the status word instead of touching the rest
  b.partials_bytes = (int64_t)((size_t)n_split_rows * acc_bytes);
  b.counters = reinterpret_cast<int32_t*>(base + kStaticPartialsBytes);
  // The array keeps whatever the previous call left.  Row accumulators and counters must start at
  // zero (a launch that ran to the end leaves them so, a launch that gave up may not), so the part
  // this call uses is cleared in stream order before the launch.
  if (n_split_rows > 0) {
    if (cudaMemsetAsync(b.partials, 0, (size_t)n_split_rows * acc_bytes, stream) != cudaSuccess) return VOID_ERR_CUDA;
    if (cudaMemsetAsync(b.counters, 0, (size_t)n_split_rows * sizeof(int32_t), stream) != cudaSuccess)
      return VOID_ERR_CUDA;
  }
  return spmm_launch(&b, VOID_KIND_I8, stream);
}

// A kernel that does nothing but take part in programmatic dependent launch the way the SpMM kernels do.
__global__ void floor_kernel() {
  grid_launch_dependents();
  grid_dependency_wait();
}

}  // namespace vb

extern "C" {

int void_launch_floor(int32_t grid, int32_t threads, int32_t smem_bytes, void_stream_t stream) {
  if (grid < 1 || threads < 32 || threads > 1024 || smem_bytes < 0) return VOID_ERR_BAD_ARG;
  if (vb::ensure_smem((const void*)vb::floor_kernel, smem_bytes)) return VOID_ERR_CUDA;
  vb::launch_pdl(vb::floor_kernel, grid, threads, smem_bytes, reinterpret_cast<cudaStream_t>(stream));
  return cudaGetLastError() == cudaSuccess ? VOID_OK : VOID_ERR_CUDA;
}

int void_spmm_i8_static_scratch(const void_spmm_args* args, int32_t n_split_rows, void_stream_t stream) {
  return vb::spmm_i8_static_scratch(args, n_split_rows, reinterpret_cast<cudaStream_t>(stream));
}

int void_spmm_i8(const void_spmm_args* args, void_stream_t stream) {
  return vb::spmm_launch(args, VOID_KIND_I8, reinterpret_cast<cudaStream_t>(stream));
}
int void_spmm_f8(const void_spmm_args* args, void_stream_t stream) {
  return vb::spmm_launch(args, VOID_KIND_F8E4M3, reinterpret_cast<cudaStream_t>(stream));
}
int void_spmm_fp(const void_spmm_args* args, int32_t kind, void_stream_t stream) {
  if (kind != VOID_KIND_F16 && kind != VOID_KIND_BF16 && kind != VOID_KIND_TF32) return VOID_ERR_BAD_ARG;
  return vb::spmm_launch(args, kind, reinterpret_cast<cudaStream_t>(stream));
}
int void_device_sm_count(void) {
  const vb::DeviceInfo d = vb::device_info();
  return d.ok ? d.sms : 0;
}

}  // extern "C"
