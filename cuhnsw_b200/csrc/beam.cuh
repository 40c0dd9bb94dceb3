// Warp-level building blocks of the graph walk: a sorted candidate/result list
// in shared memory, a lossy visited table, the ef-bounded best-first search of
// one layer and the greedy descent through the upper layers.
//
// What they replace in the reference:
//   sorted list + batch merge   PqPush/PqPop (cpp/include/cuda_heap_kernels.cuh:13-49, thread 0 only,
//                               heap in global memory), GetCand (cuda_utils_kernels.cuh:104-151) and
//                               CheckAlreadyExists (cuda_utils_kernels.cuh:50-103)
//   visited table               CheckVisited (cuda_utils_kernels.cuh:185-210)
//   beam_layer                  the expansion loops of SearchGraphKernel (cuda_search_kernels.cuh:114-139)
//                               and BuildLevelGraphKernel (cuda_build_kernels.cuh:219-248)
//   greedy_descent              GetEntryPointsKernel (cuda_search_kernels.cuh:22-66)
//
// One warp owns one query; there is no block-level synchronisation anywhere.
#pragma once
#include "common.cuh"
#include "distance.cuh"

namespace hnsw {

struct WalkCounters {
  unsigned long long evals;       // rows gathered for a distance
  unsigned long long expansions;  // adjacency rows read at the searched layer
  unsigned long long sweeps;      // adjacency rows read during greedy descent
  unsigned long long inserts;     // keys merged into the list
};

// Per-warp shared-memory state.
struct WarpList {
  unsigned long long* keys;  // ascending (distance, id); capacity `cap`
  int* spos;                 // 32 ints of scratch
  unsigned* vt;              // visited table, vsize entries (power of two), 0xffffffff = empty
  int vshift;                // 32 - log2(vsize)
  int vsize;
  int cap;
  int size;
  int cursor;  // every key before `cursor` is expanded

  __host__ __device__ static constexpr size_t smem_bytes(int cap, int vsize) {
    return (size_t)((cap + 31) / 32 * 32) * 8 + 32 * 4 + (size_t)vsize * 4;
  }
  __device__ __forceinline__ void bind(void* smem, int cap_, int vsize_) {
    keys = reinterpret_cast<unsigned long long*>(smem);
    int capr = (cap_ + 31) / 32 * 32;
    spos = reinterpret_cast<int*>(keys + capr);
    vt = reinterpret_cast<unsigned*>(spos + 32);
    cap = cap_;
    vsize = vsize_;
    vshift = 32 - (31 - __clz(vsize_));
    size = 0;
    cursor = 0;
  }
  // The table size is proportional to the list capacity, so clearing it is
  // O(nodes touched); the reference resets through a touched-slot list
  // (cuda_search_kernels.cuh:145-147).
  __device__ __forceinline__ void reset() {
    uint4* p = reinterpret_cast<uint4*>(vt);
    const uint4 e = make_uint4(~0u, ~0u, ~0u, ~0u);
    for (int i = lane_id(); i < vsize / 4; i += 32) p[i] = e;
    size = 0;
    cursor = 0;
    __syncwarp();
  }
  // Lossy set with no false positives: a hit means the id was recorded
  // earlier; a miss records it (possibly displacing another id), which can
  // only cause a repeated distance evaluation, never a different result,
  // because duplicates are rejected when merging into the list.
  __device__ __forceinline__ bool test_and_set(int id) {
    unsigned slot = ((unsigned)id * 2654435761u) >> vshift;
    unsigned a = vt[slot];
    if (a == (unsigned)id) return true;
    unsigned b = vt[slot ^ 1];
    if (b == (unsigned)id) return true;
    if (a == ~0u || b != ~0u) vt[slot] = (unsigned)id;
    else vt[slot ^ 1] = (unsigned)id;
    return false;
  }
  __device__ __forceinline__ void mark(int id) {
    if (lane_id() == 0) test_and_set(id);
    __syncwarp();
  }

  // Merges up to 32 new keys (one per lane, `active` lanes) into the list,
  // keeping the `cap` smallest.  Equivalent to inserting them one by one in any
  // order with "insert if not full or smaller than the largest, evicting the
  // largest" (cuda_utils_kernels.cuh:220-225).
  __device__ __forceinline__ void merge(unsigned long long key, bool active, WalkCounters& wc) {
    const int lane = lane_id();
    unsigned long long worst = (size >= cap) ? (keys[size - 1] & KEY_MASK) : KEY_MAX;
    bool keep = active && key < worst;
    if (!__any_sync(FULL, keep)) return;
    // position = number of list keys smaller than the new key
    int lo = 0, hi = keep ? size : 0;
    while (__any_sync(FULL, lo < hi)) {
      if (lo < hi) {
        int mid = (lo + hi) >> 1;
        if ((keys[mid] & KEY_MASK) < key) lo = mid + 1;
        else hi = mid;
      }
    }
    const int pos = lo;
    if (keep && pos < size && (keys[pos] & KEY_MASK) == key) keep = false;  // already listed
    const unsigned km = __ballot_sync(FULL, keep);
    if (km == 0) return;
    const int m = __popc(km);
    int rk = 0;
    for (unsigned mm = km; mm; mm &= mm - 1) {
      int b = __ffs(mm) - 1;
      unsigned long long kb = shfl64(key, b);
      rk += (kb < key) ? 1 : 0;
    }
    if (keep) spos[rk] = pos;
    __syncwarp();
    const int minpos = spos[0];
    for (int base = (size - 1) & ~31; size > 0 && base >= (minpos & ~31); base -= 32) {
      int i = base + lane;
      bool have = (i < size) && (i >= minpos);
      unsigned long long v = have ? keys[i] : 0ull;
      int cnt = 0;
      if (have)
        for (int j = 0; j < m; ++j) cnt += (spos[j] <= i) ? 1 : 0;
      __syncwarp();
      if (have && i + cnt < cap) keys[i + cnt] = v;
      __syncwarp();
    }
    if (keep && pos + rk < cap) keys[pos + rk] = key;
    size = min(cap, size + m);
    cursor = min(cursor, minpos);
    wc.inserts += m;
    __syncwarp();
  }

  // moves `cursor` to the first unexpanded key at or after it
  __device__ __forceinline__ void advance() {
    const int lane = lane_id();
    int c = cursor;
    while (c < size) {
      int i = c + lane;
      bool open = (i < size) && !(keys[i] & KEY_FLAG);
      unsigned m = __ballot_sync(FULL, open);
      if (m) {
        c += __ffs(m) - 1;
        break;
      }
      c += 32;
    }
    cursor = min(c, size);
  }
};

// Gathers one adjacency row chunk (32 ids per step), filters it through the
// visited table, evaluates the fresh ids and merges them.  `rows` is a
// sentinel-padded table: unused slots hold -1.
template <class Dist>
__device__ __forceinline__ void expand_row(Dist& de, WarpList& wl, const int* __restrict__ row, int stride,
                                           int self, WalkCounters& wc) {
  const int lane = lane_id();
  for (int base = 0; base < stride; base += 32) {
    int l = base + lane;
    int nid = (l < stride) ? __ldg(row + l) : -1;
    bool fresh = (nid >= 0) && (nid != self);
    if (fresh) fresh = !wl.test_and_set(nid);
    unsigned fm = __ballot_sync(FULL, fresh);
    if (fm == 0) continue;
    int n = __popc(fm);
    if (fresh) wl.spos[__popc(fm & ((1u << lane) - 1))] = nid;
    __syncwarp();
    int cid = wl.spos[lane];
    __syncwarp();
    float dist = de.eval(cid, n);
    wc.evals += n;
    wl.merge(mkkey(dist, cid), lane < n, wc);
  }
}

// ef-bounded best-first search of one layer.  The list must already hold the
// seeds; on return it holds the min(ef, reachable) closest nodes, ascending.
// Row number of node `id` in the adjacency table of `level`: layer 0 is indexed by id,
// the upper layers of a node are stored consecutively from upper_base[id].
__device__ __forceinline__ size_t row_index(const int* __restrict__ upper_base, int level, int id) {
  return level == 0 ? (size_t)id : (size_t)__ldg(upper_base + id) + (size_t)(level - 1);
}

template <class Dist>
__device__ __forceinline__ void beam_layer(Dist& de, WarpList& wl, const int* __restrict__ rows, int stride,
                                           const int* __restrict__ upper_base, int level, int self,
                                           WalkCounters& wc) {
  wl.advance();
  while (wl.cursor < wl.size) {
    unsigned long long k = wl.keys[wl.cursor];
    __syncwarp();
    if (lane_id() == 0) wl.keys[wl.cursor] = k | KEY_FLAG;
    __syncwarp();
    const int cur = key_id(k);
    wc.expansions += 1;
    expand_row(de, wl, rows + row_index(upper_base, level, cur) * stride, stride, self, wc);
    wl.advance();
  }
}

// Greedy walk through layers top..bottom+1: in each layer, evaluate every
// neighbour of the current node, move to the closest one if it is strictly
// closer (first in row order among equals), repeat until no move.
template <class Dist>
__device__ __forceinline__ void greedy_descent(Dist& de, int* scratch, const int* __restrict__ rowsU, int strideU,
                                               const int* __restrict__ upper_base, int top, int bottom_excl,
                                               int& cur, float& dcur, WalkCounters& wc) {
  const int lane = lane_id();
  for (int l = top; l > bottom_excl; --l) {
    bool moved = true;
    while (moved) {
      moved = false;
      const int* row = rowsU + ((size_t)__ldg(upper_base + cur) + (l - 1)) * strideU;
      int best_id = cur;
      float best_d = dcur;
      wc.sweeps += 1;
      for (int base = 0; base < strideU; base += 32) {
        int li = base + lane;
        int nid = (li < strideU) ? __ldg(row + li) : -1;
        bool ok = nid >= 0;
        unsigned fm = __ballot_sync(FULL, ok);
        if (fm == 0) continue;
        int n = __popc(fm);
        if (ok) scratch[__popc(fm & ((1u << lane) - 1))] = nid;
        __syncwarp();
        int cid = scratch[lane];
        __syncwarp();
        float dist = de.eval(cid, n);
        wc.evals += n;
        float dm = (lane < n) ? dist : __int_as_float(0x7f800000);
        int lm = lane;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          float od = __shfl_xor_sync(FULL, dm, off);
          int ol = __shfl_xor_sync(FULL, lm, off);
          if (od < dm || (od == dm && ol < lm)) {
            dm = od;
            lm = ol;
          }
        }
        if (dm < best_d) {
          best_d = dm;
          best_id = __shfl_sync(FULL, cid, lm);
        }
      }
      if (best_id != cur) {
        cur = best_id;
        dcur = best_d;
        moved = true;
      }
    }
  }
}

}  // namespace hnsw
