// Block-sparse mask-map builder.
//
// Replaces the reference's per-grid-step `block_mask_fn(q_blk, k_blk)` predicates (masks.py:20-28,
// 63-81,113-139,161-177): instead of asking "does this tile pair run?" at every grid step, the map
// stores, once per (mask, shape[, batch row]), for every q tile the contiguous range of kv tiles that
// hold at least one kept pair and the contiguous sub-range whose pairs are ALL kept (the attention
// kernels skip the mask functor there); and the transposed information for every kv tile.
//
// Tile classification is closed form on tile bounds; the document mask first reduces the ids of every
// tile to (min, max).  A pair range that is only *possibly* non-empty (document ids that are not
// sorted) is listed as a partial tile, which is always safe: partial tiles evaluate the exact mask.
#include "common.cuh"

namespace flexattn {
namespace {

struct PairClass {
  bool any, all;
};

// q rows [q0,q1], keys [k0,k1] (inclusive, already clipped to the sequence lengths).
__device__ __forceinline__ PairClass classify(int kind, int q0, int q1, int k0, int k1, int window,
                                              int stride, int2 qd, int2 kd) {
  PairClass c;
  const int dmin = q0 - k1, dmax = q1 - k0;  // range of i - j over the tile pair
  switch (kind) {
    case FLEXATTN_MASK_NONE:
      c.any = true; c.all = true; break;
    case FLEXATTN_MASK_CAUSAL:
      c.any = dmax >= 0; c.all = dmin >= 0; break;
    case FLEXATTN_MASK_SLIDING_WINDOW:
      c.any = dmin < window; c.all = dmax < window; break;
    case FLEXATTN_MASK_SLIDING_WINDOW_CAUSAL:
      c.any = dmax >= 0 && dmin < window; c.all = dmin >= 0 && dmax < window; break;
    case FLEXATTN_MASK_DOCUMENT: {
      int lo = qd.x > kd.x ? qd.x : kd.x, hi = qd.y < kd.y ? qd.y : kd.y;
      c.any = dmax >= 0 && lo <= hi;
      c.all = dmin >= 0 && qd.x == qd.y && kd.x == kd.y && qd.x == kd.x;
      break;
    }
    default: {  // S2: window-causal OR (key on the stride grid AND causal)
      bool win_any = dmax >= 0 && dmin < window;
      int first = ((k0 + stride - 1) / stride) * stride;  // first strided key in the tile
      int lim = k1 < q1 ? k1 : q1;
      c.any = win_any || (first <= lim);
      c.all = dmin >= 0 && (dmax < window || stride == 1);
      break;
    }
  }
  return c;
}

__global__ void doc_minmax_kernel(const int32_t* __restrict__ doc_ids, int2* __restrict__ out, int n_t,
                                  int len) {
  // grid (n_t, B), block 128: (min,max) document id of positions [t*128, t*128+128) of batch row b
  const int t = blockIdx.x, b = blockIdx.y;
  const int pos = t * kTile + threadIdx.x;
  int lo = INT32_MAX, hi = INT32_MIN;
  if (pos < len) lo = hi = doc_ids[(size_t)b * len + pos];
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, s));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, s));
  }
  __shared__ int slo[4], shi[4];
  if ((threadIdx.x & 31) == 0) { slo[threadIdx.x >> 5] = lo; shi[threadIdx.x >> 5] = hi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 4; ++w) { lo = min(lo, slo[w]); hi = max(hi, shi[w]); }
    out[(size_t)b * n_t + t] = make_int2(lo, hi);
  }
}

// Runs of equal document ids, one CTA of 1024 threads per batch row: run_lo[p] / run_hi[p] = first / one past the
// last position of the run position p sits in (an inclusive prefix-maximum scan of the run starts and a suffix-minimum
// scan of the run ends, in chunks of 1024 with a carry), and sorted[b] = 1 when the ids never decrease.
__global__ void __launch_bounds__(1024) doc_runs_kernel(const int32_t* __restrict__ doc_ids, int32_t* __restrict__ run_lo,
                                                        int32_t* __restrict__ run_hi, int32_t* __restrict__ sorted, int len) {
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int32_t* doc = doc_ids + (size_t)b * len;
  int32_t* lo = run_lo + (size_t)b * len;
  int32_t* hi = run_hi + (size_t)b * len;
  __shared__ int warp_v[32];
  __shared__ int carry_s, unsorted_s;
  if (tid == 0) { carry_s = 0; unsorted_s = 0; }
  __syncthreads();
  for (int base = 0; base < len; base += 1024) {  // forward: latest run start at or before p
    const int p = base + tid;
    int v = -1;
    if (p < len) {
      const int d = doc[p];
      if (p == 0) v = 0;
      else {
        const int dp = doc[p - 1];
        if (d != dp) v = p;
        if (d < dp) unsorted_s = 1;
      }
    }
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, v, s);
      if (lane >= s) v = max(v, o);
    }
    if (lane == 31) warp_v[w] = v;
    __syncthreads();
    if (w == 0) {
      int x = warp_v[lane];
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, x, s);
        if (lane >= s) x = max(x, o);
      }
      warp_v[lane] = x;
    }
    __syncthreads();
    v = max(v, max(carry_s, w > 0 ? warp_v[w - 1] : -1));
    if (p < len) lo[p] = v;
    __syncthreads();
    if (tid == 1023) carry_s = v;
    __syncthreads();
  }
  if (tid == 0) carry_s = len;
  __syncthreads();
  for (int base = ((len - 1) / 1024) * 1024; base >= 0; base -= 1024) {  // backward: earliest run end after p
    const int p = base + 1023 - tid;  // thread order = descending position
    int v = 0x7fffffff;
    if (p < len && (p == len - 1 || doc[p + 1] != doc[p])) v = p + 1;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, v, s);
      if (lane >= s) v = min(v, o);
    }
    if (lane == 31) warp_v[w] = v;
    __syncthreads();
    if (w == 0) {
      int x = warp_v[lane];
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, x, s);
        if (lane >= s) x = min(x, o);
      }
      warp_v[lane] = x;
    }
    __syncthreads();
    v = min(v, min(carry_s, w > 0 ? warp_v[w - 1] : 0x7fffffff));
    if (p < len) hi[p] = v;
    __syncthreads();
    if (tid == 1023) carry_s = v;
    __syncthreads();
  }
  if (tid == 0) sorted[b] = unsorted_s ? 0 : 1;
}

__global__ void mask_map_kernel(MapHeader hdr, MapHeader* __restrict__ hdr_out, int4* __restrict__ row_map,
                                int4* __restrict__ col_map, const int2* __restrict__ docmm, int n_t) {
  if (blockIdx.x == 0 && threadIdx.x == 0) *hdr_out = hdr;
  // one thread per (map row, tile) for the row map, then for the column map
  const int n_row_entries = hdr.rows * hdr.n_qt;
  const int n_col_entries = hdr.rows * hdr.n_kt;
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < n_row_entries + n_col_entries;
       e += gridDim.x * blockDim.x) {
    const bool is_col = e >= n_row_entries;
    const int idx = is_col ? e - n_row_entries : e;
    const int n_self = is_col ? hdr.n_kt : hdr.n_qt;
    const int n_other = is_col ? hdr.n_qt : hdr.n_kt;
    const int r = idx / n_self, t = idx % n_self;
    const int len_self = is_col ? hdr.seq_k : hdr.seq_q;
    const int len_other = is_col ? hdr.seq_q : hdr.seq_k;
    const int s0 = t * kTile, s1 = min(s0 + kTile, len_self) - 1;
    const int2 none = make_int2(0, 0);
    const int2 sd = docmm ? docmm[(size_t)r * n_t + t] : none;
    int lo = -1, hi = -1, flo = -1, fhi = -1;
    bool run_open = false;
    for (int u = 0; u < n_other; ++u) {
      const int o0 = u * kTile, o1 = min(o0 + kTile, len_other) - 1;
      const int2 od = docmm ? docmm[(size_t)r * n_t + u] : none;
      PairClass c = is_col ? classify(hdr.mask_kind, o0, o1, s0, s1, hdr.window, hdr.stride, od, sd)
                           : classify(hdr.mask_kind, s0, s1, o0, o1, hdr.window, hdr.stride, sd, od);
      // a ragged tile on either side still needs its out-of-range positions masked
      if (o0 + kTile > len_other) c.all = false;
      if (c.any) {
        if (lo < 0) lo = u;
        hi = u + 1;
      }
      if (c.any && c.all) {
        if (flo < 0) { flo = u; fhi = u + 1; run_open = true; }
        else if (run_open && fhi == u) fhi = u + 1;
      } else if (flo >= 0) {
        run_open = false;
      }
    }
    if (lo < 0) { lo = hi = 0; }
    if (flo < 0) { flo = fhi = lo; }
    (is_col ? col_map : row_map)[idx] = make_int4(lo, hi, flo, fhi);
  }
}

// Work order of the q tiles of one map row: by decreasing number of kv tiles (counting sort; ties by decreasing
// tile index, so the result is deterministic).  One CTA per map row; hist has n_kt + 2 entries.
__global__ void order_kernel(const int4* __restrict__ row_map, int32_t* __restrict__ order, int4* __restrict__ order_rm,
                             int n_qt, int n_kt) {
  extern __shared__ int hist[];
  const int4* rm = row_map + (size_t)blockIdx.x * n_qt;
  int32_t* ord = order + (size_t)blockIdx.x * n_qt;
  int4* ord_rm = order_rm + (size_t)blockIdx.x * n_qt;
  for (int i = threadIdx.x; i < n_kt + 2; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (int t = threadIdx.x; t < n_qt; t += blockDim.x) atomicAdd(&hist[rm[t].y - rm[t].x], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int running = 0;
    for (int n = n_kt; n >= 0; --n) {  // exclusive offsets, largest count first
      const int c = hist[n];
      hist[n] = running;
      running += c;
    }
    for (int t = n_qt - 1; t >= 0; --t) ord[hist[rm[t].y - rm[t].x]++] = t;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_qt; i += blockDim.x) ord_rm[i] = rm[ord[i]];
}

}  // namespace

cudaError_t launch_mask_map(cudaStream_t st, const FlexAttnParams& p) {
  MapLayout L = map_layout(p.batch, p.seq_q, p.seq_k, p.mask_kind);
  char* ws = static_cast<char*>(p.workspace);
  MapHeader hdr{};
  hdr.magic = kMapMagic;
  hdr.mask_kind = p.mask_kind;
  hdr.window = p.window;
  hdr.stride = p.stride > 0 ? p.stride : 1;
  hdr.seq_q = p.seq_q;
  hdr.seq_k = p.seq_k;
  hdr.n_qt = L.n_qt;
  hdr.n_kt = L.n_kt;
  hdr.rows = L.rows;
  int2* docmm = nullptr;
  if (p.mask_kind == FLEXATTN_MASK_DOCUMENT) {
    docmm = reinterpret_cast<int2*>(ws + L.off_doc);
    const int len = p.seq_q > p.seq_k ? p.seq_q : p.seq_k;
    doc_minmax_kernel<<<dim3(L.n_t, p.batch), 128, 0, st>>>(p.doc_ids, docmm, L.n_t, len);
    doc_runs_kernel<<<p.batch, 1024, 0, st>>>(p.doc_ids, reinterpret_cast<int32_t*>(ws + L.off_run_lo),
                                              reinterpret_cast<int32_t*>(ws + L.off_run_hi),
                                              reinterpret_cast<int32_t*>(ws + L.off_sorted), len);
  }
  const int entries = L.rows * (L.n_qt + L.n_kt);
  const int blocks = (entries + 127) / 128;
  mask_map_kernel<<<blocks < 1184 ? blocks : 1184, 128, 0, st>>>(
      hdr, reinterpret_cast<MapHeader*>(ws), reinterpret_cast<int4*>(ws + L.off_row), reinterpret_cast<int4*>(ws + L.off_col), docmm, L.n_t);
  const size_t hist_bytes = sizeof(int) * (size_t)(L.n_kt + 2);
  if (hist_bytes > 48 * 1024) return cudaErrorInvalidValue;  // more than 12 286 kv tiles (1.5 M keys)
  order_kernel<<<L.rows, 256, hist_bytes, st>>>(reinterpret_cast<const int4*>(ws + L.off_row),
                                                 reinterpret_cast<int32_t*>(ws + L.off_order),
                                                 reinterpret_cast<int4*>(ws + L.off_order_rm), L.n_qt, L.n_kt);
  return cudaGetLastError();
}

}  // namespace flexattn
