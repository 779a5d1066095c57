// Work distribution of the persistent kernels: every CTA walks the same global list of (q tile, batch*head) items.
#pragma once
#include "common.cuh"

namespace flexattn {

// A CTA's walk over its work items.  The heads of a batch row are taken in groups small enough for the K and V of a
// whole group to stay in L2 (every q tile of a slice re-reads them); inside a group the items follow the mask map's
// work order of the q tiles (most kv tiles first), head index fastest.  The resulting list is dealt to the CTAs in
// rounds that alternate direction (CTA c takes entry c of an even round and entry G-1-c of an odd one), which evens
// out the work of a sorted list.  Tile order and mask-map row of the next item are fetched one item ahead.
struct ItemCursor {
  const DevParams& P;
  int total, per_row, group, full_groups;
  int round, w;      // current round and item; valid while w < total
  int4 rm, rm_next;  // mask-map rows {first kv tile, end kv tile, first full, end full} of this item and the next
  int bh_, qt_, bh_next, qt_next;
  __device__ __forceinline__ int item_of(int r) const {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    return r * G + ((r & 1) ? G - 1 - c : c);
  }
  __device__ __forceinline__ int4 fetch(int item, int& bh, int& qt) const {
    const int b = item / per_row, r = item - b * per_row;
    int gi = r / (group * P.n_qt), width = group;
    if (gi >= full_groups) {  // the last, smaller group of the batch row
      gi = full_groups;
      width = P.heads - full_groups * group;
    }
    const int r2 = r - gi * group * P.n_qt;
    const int rank = r2 / width;
    bh = b * P.heads + gi * group + (r2 - rank * width);
    const size_t row = (size_t)(P.map_rows > 1 ? b : 0) * P.n_qt;
    qt = __ldg(&P.order[row + rank]);
    return __ldg(&P.order_rm[row + rank]);  // the row-map entry of that q tile: two independent loads
  }
  // l2_budget: bytes of K + V that may be live at a time (sets how many heads form a group)
  __device__ __forceinline__ explicit ItemCursor(const DevParams& p, long long l2_budget = 48ll << 20) : P(p) {
    per_row = p.heads * p.n_qt;
    total = p.batch * per_row;
    // K + V of one slice: 2 * seq_k * head_dim * 2 bytes
    const long long slice_bytes = 4ll * p.seq_k * p.head_dim;
    group = (int)max(1ll, min((long long)p.heads, l2_budget / slice_bytes));
    full_groups = p.heads / group;
    round = 0;
    w = item_of(0);
    rm = rm_next = make_int4(0, 0, 0, 0);
    bh_ = qt_ = bh_next = qt_next = 0;
    if (w < total) rm = fetch(w, bh_, qt_);
    if (item_of(1) < total) rm_next = fetch(item_of(1), bh_next, qt_next);
  }
  __device__ __forceinline__ bool valid() const { return w < total; }
  __device__ __forceinline__ int tiles() const { return rm.y - rm.x; }
  __device__ __forceinline__ int bh() const { return bh_; }
  __device__ __forceinline__ int qt() const { return qt_; }
  __device__ __forceinline__ void next() {
    ++round;
    w = item_of(round);
    rm = rm_next;
    bh_ = bh_next;
    qt_ = qt_next;
    const int nxt = item_of(round + 1);
    if (nxt < total) rm_next = fetch(nxt, bh_next, qt_next);
  }
  // skip items without any kv tile (the producers and the MMA issuer have nothing to do for them)
  __device__ __forceinline__ void skip_empty() {
    while (valid() && tiles() <= 0) next();
  }
};

#ifndef FLEXATTN_JIT
// Number of SMs of the current device (queried once per device); -1 on error.
inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cached[dev] = n;
  }
  return cached[dev];
}
#endif  // !FLEXATTN_JIT

}  // namespace flexattn
