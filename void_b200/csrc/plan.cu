// Device-side work splitter of the SpMM kernels.
//
// The work of one launch is the sequence of "virtual rows" v = (column chunk c, tile row r),
// v = c * nbr + r, each worth (tiles in row r) + row_cost units.  row_cost stands for the epilogue:
// reading the accumulator back, dequantising, activating and storing 32 x chunk columns costs as
// much as several tiles of products, and empty rows still have to be written as zeros.  Because
// row_ptr is already a prefix sum, the start position of a virtual row on that axis is closed-form:
// P(v) = c * (nnz + row_cost * nbr) + row_ptr[r] + row_cost * r.  The axis is cut into n_cta shares of
// equal length; cut k lands inside some row and is then moved
//   mode 0  to the nearer tile-row boundary (rows are never split),
//   mode 1  to the nearer tile-row boundary if the row is light, else to the nearest multiple of
//           `chunk_tiles` inside the row (the chunk boundaries of the Stream-K worker table,
//           void/stream_k.py:84-97), so that a heavy row is shared by several CTAs,
//   mode 2  always to the nearest chunk boundary, and every chunk becomes a segment of its
//           own (one segment per worker of the reference table; used to check partial sums).
// A row that ends up in several segments gets a counter and one partial-sum slot per segment;
// the SpMM kernel's last arriver adds the slots up.
//
// The same code runs as one 1024-thread block on the device (the product path) and, for
// tests of the splitting arithmetic on machines without a GPU, as plain loops on the host.
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "../../include/void_b200.h"

namespace vb {

struct PlanIn {
  const int32_t* row_ptr;
  const int32_t* woff;  // mode 2: workers before each row (nbr + 1), else null
  int nbr, n_chunks, n_cta, mode, chunk_tiles;
  int row_cost;  // what finishing one (tile row, chunk) costs, in units of one tile's work
};

struct PlanWs {       // all arrays have n_cta + 2 entries
  int32_t* bv;        // boundary: virtual row
  int32_t* bo;        // boundary: tile offset inside the row
  int32_t* lead_nseg; // segments of the split row whose first interior cut is this boundary, else 0
  int32_t* lead_flag; // 1 at such a boundary
  int32_t* slot_off;  // exclusive scans of the two above
  int32_t* ctr_off;
  int32_t* nseg_cta;  // segments per CTA, scanned into cta_seg_ptr
};

__host__ __device__ inline int row_cnt(const PlanIn& in, int v) {
  const int r = v % in.nbr;
  return in.row_ptr[r + 1] - in.row_ptr[r];
}

// phase 1: boundary j in [0, n_cta]
__host__ __device__ inline void plan_boundary(const PlanIn& in, const PlanWs& ws, int j) {
  const long long c0 = in.row_cost;
  const long long nnz = in.row_ptr[in.nbr];
  const long long wrow = nnz + c0 * in.nbr;
  const long long W = wrow * in.n_chunks;
  const int V = in.nbr * in.n_chunks;
  if (j >= in.n_cta) {
    ws.bv[j] = V;
    ws.bo[j] = 0;
    return;
  }
  const long long x = (W * j) / in.n_cta;
  const int c = (int)(x / wrow);
  const long long y = x - (long long)c * wrow;
  int lo = 0, hi = in.nbr - 1;  // largest r with row_ptr[r] + c0 * r <= y
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((long long)in.row_ptr[mid] + c0 * mid <= y) lo = mid;
    else hi = mid - 1;
  }
  const int r = lo;
  const long long d = y - ((long long)in.row_ptr[r] + c0 * r);  // 0 .. cnt + c0 - 1
  const int cnt = in.row_ptr[r + 1] - in.row_ptr[r];
  int v = c * in.nbr + r, o = 0;
  const long long share = W / in.n_cta;
  const bool splittable = in.chunk_tiles > 0 && cnt > 0 &&
                          (in.mode == 2 || (in.mode == 1 && (long long)cnt + c0 > share));
  if (d == 0) {
    o = 0;
  } else if (!splittable) {
    if (2 * d >= (long long)cnt + c0) v += 1;  // nearer end of the row
    o = 0;
  } else {
    const int T = in.chunk_tiles;
    const long long tile = d > c0 ? d - c0 : 0;  // the row's own cost comes first on the axis
    o = (int)(((tile + T / 2) / T) * T);
    if (o >= cnt) { v += 1; o = 0; }
  }
  ws.bv[j] = v;
  ws.bo[j] = o;
}

// number of distinct interior offsets of row bv[j] among boundaries j, j+1, ... (bo[j] > 0)
__host__ __device__ inline int distinct_from(const PlanWs& ws, int j, int n_cta) {
  const int v = ws.bv[j];
  int m = 1, prev = ws.bo[j];
  for (int i = j + 1; i <= n_cta && ws.bv[i] == v; ++i) {
    if (ws.bo[i] != prev) { ++m; prev = ws.bo[i]; }
  }
  return m;
}

// phase 2: leaders of split rows (modes 0/1), segments per CTA
__host__ __device__ inline void plan_leaders(const PlanIn& in, const PlanWs& ws, int j) {
  int lead = 0, nseg = 0;
  if (in.mode != 2 && j <= in.n_cta && ws.bo[j] > 0) {
    const bool first = (j == 0) || ws.bv[j - 1] != ws.bv[j] || ws.bo[j - 1] == 0;
    if (first) { lead = 1; nseg = distinct_from(ws, j, in.n_cta) + 1; }
  }
  ws.lead_flag[j] = lead;
  ws.lead_nseg[j] = nseg;
  if (j < in.n_cta) {
    const int va = ws.bv[j], oa = ws.bo[j], vb = ws.bv[j + 1], ob = ws.bo[j + 1];
    const int T = in.chunk_tiles;
    int n;
    if (in.mode != 2) {
      n = (va == vb) ? (ob > oa ? 1 : 0) : 1 + (vb - va - 1) + (ob > 0 ? 1 : 0);
    } else {
      if (va == vb) {
        n = (ob - oa + T - 1) / T;
      } else {
        const int ca = row_cnt(in, va);
        n = (ca - oa + T - 1) / T;
        if (ca == 0) n = 1;
        for (int v = va + 1; v < vb; ++v) {
          const int cv = row_cnt(in, v);
          n += cv == 0 ? 1 : (cv + T - 1) / T;
        }
        n += (ob + T - 1) / T;
      }
    }
    ws.nseg_cta[j] = n;
  } else {
    ws.nseg_cta[j] = 0;
  }
}

__host__ __device__ inline void put_seg(int32_t* segs, long long idx, int row, int chunk, int t0, int t1, int nseg,
                                        int slot0, int my_idx, int ctr) {
  int32_t* s = segs + idx * 8;
  s[0] = row; s[1] = chunk; s[2] = t0; s[3] = t1; s[4] = nseg; s[5] = slot0; s[6] = my_idx; s[7] = ctr;
}

// emits the piece [a, b) of virtual row v (tile offsets inside the row); returns segments written
__host__ __device__ inline int emit_piece(const PlanIn& in, const PlanWs& ws, int32_t* segs, long long at,
                                          long long capacity, int v, int a, int b, int k_start) {
  const int r = v % in.nbr, c = v / in.nbr;
  const int rs = in.row_ptr[r], cnt = in.row_ptr[r + 1] - rs;
  if (in.mode == 2) {
    const int T = in.chunk_tiles;
    const int nseg = cnt == 0 ? 1 : (cnt + T - 1) / T;
    const int n_workers = in.woff[in.nbr];
    const int slot0 = c * n_workers + in.woff[r];
    int n = 0;
    if (cnt == 0) {
      if (at < capacity) put_seg(segs, at, r, c, rs, rs, 1, 0, 0, 0);
      return 1;
    }
    for (int t = a; t < b; t += T, ++n) {
      const int e = (t + T) < b ? (t + T) : b;
      if (at + n < capacity) put_seg(segs, at + n, r, c, rs + t, rs + e, nseg, slot0, t / T, v);
    }
    return n;
  }
  int nseg = 1, slot0 = 0, my_idx = 0, ctr = 0;
  if (a > 0 || b < cnt) {
    // find the first interior boundary (leader) of this row: k_start is a boundary index inside or
    // at the edge of the row; walk back while the previous boundary is interior to the same row
    int j = k_start;
    if (!(ws.bv[j] == v && ws.bo[j] > 0)) j = k_start + 1;  // piece starts at the row start
    while (j > 0 && ws.bv[j - 1] == v && ws.bo[j - 1] > 0) --j;
    nseg = ws.lead_nseg[j];
    slot0 = ws.slot_off[j];
    ctr = ws.ctr_off[j];
    if (a > 0) {
      int prev = -1;
      for (int i = j; i <= in.n_cta && ws.bv[i] == v && ws.bo[i] <= a; ++i)
        if (ws.bo[i] != prev) { ++my_idx; prev = ws.bo[i]; }
    }
  }
  if (at < capacity) put_seg(segs, at, r, c, rs + a, rs + b, nseg, slot0, my_idx, ctr);
  return 1;
}

// phase 4: CTA k writes its segments starting at cta_seg_ptr[k]
__host__ __device__ inline void plan_emit(const PlanIn& in, const PlanWs& ws, const int32_t* cta_seg_ptr,
                                          int32_t* segs, long long capacity, int k) {
  const int va = ws.bv[k], oa = ws.bo[k], vb = ws.bv[k + 1], ob = ws.bo[k + 1];
  long long at = cta_seg_ptr[k];
  if (va == vb) {
    if (ob > oa) at += emit_piece(in, ws, segs, at, capacity, va, oa, ob, k);
    return;
  }
  at += emit_piece(in, ws, segs, at, capacity, va, oa, row_cnt(in, va), k);
  for (int v = va + 1; v < vb; ++v) at += emit_piece(in, ws, segs, at, capacity, v, 0, row_cnt(in, v), k);
  if (ob > 0) at += emit_piece(in, ws, segs, at, capacity, vb, 0, ob, k);
}

// single-block exclusive scan, n + 1 outputs (out[n] = total); in/out may alias
__device__ void plan_scan(const int32_t* in, int32_t* out, int n) {
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
  int32_t run = part[tid] - s;
  for (int i = lo; i < hi; ++i) {
    const int32_t v = in[i];
    out[i] = run;
    run += v;
  }
  if (tid == 1023) out[n] = part[1023];
  __syncthreads();
}

__global__ void __launch_bounds__(1024) plan_kernel(PlanIn in, PlanWs ws, int32_t* segs, long long capacity,
                                                    int32_t* cta_seg_ptr, int32_t* counts) {
  const int G = in.n_cta;
  for (int j = threadIdx.x; j <= G; j += blockDim.x) plan_boundary(in, ws, j);
  __syncthreads();
  for (int j = threadIdx.x; j <= G; j += blockDim.x) plan_leaders(in, ws, j);
  __syncthreads();
  plan_scan(ws.lead_nseg, ws.slot_off, G + 1);
  plan_scan(ws.lead_flag, ws.ctr_off, G + 1);
  plan_scan(ws.nseg_cta, cta_seg_ptr, G);
  for (int k = threadIdx.x; k < G; k += blockDim.x) plan_emit(in, ws, cta_seg_ptr, segs, capacity, k);
  if (threadIdx.x == 0) {
    counts[0] = cta_seg_ptr[G];
    if (in.mode == 2) {
      counts[1] = in.n_chunks * in.woff[in.nbr];
      counts[2] = in.n_chunks * in.nbr;
    } else {
      counts[1] = ws.slot_off[G + 1];
      counts[2] = ws.ctr_off[G + 1];
    }
    counts[3] = (cta_seg_ptr[G] > capacity) ? 1 : 0;  // overflow flag
  }
}

static void host_scan(const int32_t* in, int32_t* out, int n) {
  int32_t run = 0;
  for (int i = 0; i < n; ++i) {
    const int32_t v = in[i];
    out[i] = run;
    run += v;
  }
  out[n] = run;
}

static PlanWs carve_ws(int32_t* base, int n_cta) {
  const size_t n = (size_t)n_cta + 2;
  PlanWs ws;
  ws.bv = base;
  ws.bo = base + n;
  ws.lead_nseg = base + 2 * n;
  ws.lead_flag = base + 3 * n;
  ws.slot_off = base + 4 * n;
  ws.ctr_off = base + 5 * n;
  ws.nseg_cta = base + 6 * n;
  return ws;
}

}  // namespace vb

using namespace vb;

extern "C" {

int64_t void_plan_capacity(int64_t nnz, int32_t nbr, int32_t n_chunks, int32_t n_cta, int32_t split_rows,
                           int32_t chunk_tiles) {
  if (nnz < 0 || nbr < 0 || n_chunks <= 0 || n_cta <= 0) return 0;
  int64_t per_chunk = nbr;
  if (split_rows == 2 && chunk_tiles > 0) per_chunk = nnz / chunk_tiles + nbr + 1;
  return per_chunk * n_chunks + n_cta + 1;
}

size_t void_plan_ws_bytes(int32_t nbr, int32_t n_cta) {
  (void)nbr;
  return n_cta > 0 ? 7 * ((size_t)n_cta + 2) * sizeof(int32_t) : 0;
}

static int plan_check(const int32_t* row_ptr, int32_t nbr, int32_t n_chunks, int32_t n_cta, int32_t split_rows,
                      int32_t chunk_tiles, const int32_t* woff, const int32_t* segs, const int32_t* cta_seg_ptr,
                      const int32_t* counts) {
  if (row_ptr == nullptr || segs == nullptr || cta_seg_ptr == nullptr || counts == nullptr) return VOID_ERR_BAD_ARG;
  if (nbr <= 0 || n_chunks <= 0 || n_cta <= 0 || split_rows < 0 || split_rows > 2) return VOID_ERR_BAD_ARG;
  if (split_rows > 0 && chunk_tiles <= 0) return VOID_ERR_BAD_ARG;
  if (split_rows == 2 && woff == nullptr) return VOID_ERR_BAD_ARG;
  if ((long long)nbr * n_chunks > 0x7fffffffLL) return VOID_ERR_TOO_LARGE;
  return VOID_OK;
}

int void_plan_segments(const int32_t* row_ptr, int32_t nbr, int32_t n_chunks, int32_t n_cta, int32_t split_rows,
                       int32_t chunk_tiles, int32_t row_cost, const int32_t* woff, int32_t* segs,
                       int64_t segs_capacity, int32_t* cta_seg_ptr, int32_t* counts, void* ws, size_t ws_bytes,
                       void_stream_t stream) {
  const int st = plan_check(row_ptr, nbr, n_chunks, n_cta, split_rows, chunk_tiles, woff, segs, cta_seg_ptr, counts);
  if (st != VOID_OK) return st;
  if (ws == nullptr || ws_bytes < void_plan_ws_bytes(nbr, n_cta)) return VOID_ERR_WORKSPACE;
  if (row_cost < 1) return VOID_ERR_BAD_ARG;
  PlanIn in{row_ptr, woff, nbr, n_chunks, n_cta, split_rows, chunk_tiles, row_cost};
  const PlanWs w = carve_ws(reinterpret_cast<int32_t*>(ws), n_cta);
  plan_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(in, w, segs, segs_capacity, cta_seg_ptr, counts);
  return cudaGetLastError() == cudaSuccess ? VOID_OK : VOID_ERR_CUDA;
}

// Host twin of void_plan_segments over HOST arrays: the same splitting arithmetic run as plain
// loops.  It exists so that the splitter can be tested where there is no GPU; nothing in the
// SpMM path calls it.
int void_plan_segments_host(const int32_t* row_ptr, int32_t nbr, int32_t n_chunks, int32_t n_cta,
                            int32_t split_rows, int32_t chunk_tiles, int32_t row_cost, const int32_t* woff,
                            int32_t* segs, int64_t segs_capacity, int32_t* cta_seg_ptr, int32_t* counts) {
  const int st = plan_check(row_ptr, nbr, n_chunks, n_cta, split_rows, chunk_tiles, woff, segs, cta_seg_ptr, counts);
  if (st != VOID_OK) return st;
  std::vector<int32_t> buf(7 * ((size_t)n_cta + 2), 0);
  if (row_cost < 1) return VOID_ERR_BAD_ARG;
  PlanIn in{row_ptr, woff, nbr, n_chunks, n_cta, split_rows, chunk_tiles, row_cost};
  const PlanWs w = carve_ws(buf.data(), n_cta);
  const int G = n_cta;
  for (int j = 0; j <= G; ++j) plan_boundary(in, w, j);
  for (int j = 0; j <= G; ++j) plan_leaders(in, w, j);
  host_scan(w.lead_nseg, w.slot_off, G + 1);
  host_scan(w.lead_flag, w.ctr_off, G + 1);
  host_scan(w.nseg_cta, cta_seg_ptr, G);
  for (int k = 0; k < G; ++k) plan_emit(in, w, cta_seg_ptr, segs, segs_capacity, k);
  counts[0] = cta_seg_ptr[G];
  if (split_rows == 2) {
    counts[1] = n_chunks * woff[nbr];
    counts[2] = n_chunks * nbr;
  } else {
    counts[1] = w.slot_off[G + 1];
    counts[2] = w.ctr_off[G + 1];
  }
  counts[3] = (cta_seg_ptr[G] > segs_capacity) ? 1 : 0;
  return VOID_OK;
}

}  // extern "C"
