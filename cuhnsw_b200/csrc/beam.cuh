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
#include "kernels.h"

namespace hnsw {

__device__ __forceinline__ VecTable make_table(const GraphView& g) {
  return VecTable{static_cast<const unsigned char*>(g.vec), (size_t)g.vstride * (g.rows16 ? 2 : 4), (g.d + 3) / 4, g.d,
                  g.dist_type};
}

struct WalkCounters {  // per warp and launch
  unsigned evals;       // rows gathered for a distance
  unsigned expansions;  // adjacency rows read at the searched layer
  unsigned sweeps;      // adjacency rows read during greedy descent
  unsigned inserts;     // keys merged into the list
};

// Number of bits that hold every node id of an index with n nodes.
__host__ __device__ inline int id_bits(long long n) {
  int b = 1;
  while (b < 31 && (1ll << b) < n) ++b;
  return b;
}
// Bytes per visited-table entry: 2 when the tag that remains after the bucket number fits in 15 bits.
__host__ __device__ inline int visited_entry_bytes(long long n, int entries) {
  int kb = 0;
  while ((2 << kb) < entries) ++kb;  // buckets = entries / 2 = 2^kb
  int tag_bits = id_bits(n) - kb;
  return tag_bits <= 15 ? 2 : 4;
}

// Per-warp shared-memory state.
struct WarpList {
  unsigned long long* keys;  // ascending (distance, id); capacity `cap`
  int* spos;                 // 32 ints of scratch
  unsigned* vt;              // visited table: buckets of two tags (2 x 16 bit in one word, or 2 x 32 bit)
  unsigned hmask;            // 2^B - 1, B = id_bits(n)
  int tag_bits;              // low bits of the hash kept as the tag; the rest is the bucket number
  unsigned tag_mask;
  bool wide;                 // 32-bit tags
  int vbytes;
  int cap;
  int size;
  int cursor;  // every key before `cursor` is expanded
  unsigned long long worst;  // largest key of a full list, KEY_MAX while there is room

  __host__ __device__ static size_t smem_bytes(int cap, int entries, long long n) {
    return (size_t)((cap + 31) / 32 * 32) * 8 + 32 * 4 + (size_t)entries * visited_entry_bytes(n, entries);
  }
  __device__ __forceinline__ void bind(void* smem, int cap_, int entries, long long n) {
    keys = reinterpret_cast<unsigned long long*>(smem);
    int capr = (cap_ + 31) / 32 * 32;
    spos = reinterpret_cast<int*>(keys + capr);
    vt = reinterpret_cast<unsigned*>(spos + 32);
    cap = cap_;
    const int b = id_bits(n);
    int kb = 0;
    while ((2 << kb) < entries) ++kb;
    tag_bits = b - kb > 0 ? b - kb : 0;
    hmask = b >= 32 ? ~0u : ((1u << b) - 1u);
    tag_mask = (1u << tag_bits) - 1u;
    wide = tag_bits > 15;
    vbytes = entries * (wide ? 4 : 2);
    size = 0;
    cursor = 0;
    worst = KEY_MAX;
  }
  // The table size is proportional to the list capacity, so clearing it is
  // O(nodes touched); the reference resets through a touched-slot list
  // (cuda_search_kernels.cuh:145-147).
  __device__ __forceinline__ void reset() {
    uint4* p = reinterpret_cast<uint4*>(vt);
    const uint4 e = make_uint4(~0u, ~0u, ~0u, ~0u);
    for (int i = lane_id(); i < vbytes / 16; i += 32) p[i] = e;
    size = 0;
    cursor = 0;
    worst = KEY_MAX;
    __syncwarp();
  }
  // Lossy set with no false positives.  id -> h = id * odd mod 2^B is a bijection on B-bit
  // numbers, so (bucket, tag) = (high bits, low bits) of h identifies the id exactly and only
  // the tag has to be stored.  Each bucket keeps its two most recent tags; a displaced id can
  // only cause a repeated distance evaluation, never a different result, because duplicates are
  // rejected when merging into the list and a key that left the list can never re-enter.
  __device__ __forceinline__ bool test_and_set(int id) {
    const unsigned h = ((unsigned)id * 2654435761u) & hmask;
    const unsigned bucket = h >> tag_bits;
    const unsigned tag = h & tag_mask;
    if (!wide) {
      const unsigned w = vt[bucket];
      if ((w & 0xffffu) == tag || (w >> 16) == tag) return true;
      vt[bucket] = (w << 16) | tag;
      return false;
    }
    uint2* p = reinterpret_cast<uint2*>(vt) + bucket;
    const uint2 w = *p;
    if (w.x == tag || w.y == tag) return true;
    *p = make_uint2(tag, w.x);
    return false;
  }
  __device__ __forceinline__ void mark(int id) {
    if (lane_id() == 0) test_and_set(id);
    __syncwarp();
  }

  // Merges up to 32 new keys (one per lane, `active` lanes) into the list,
  // keeping the `cap` smallest.  Equivalent to inserting them one by one in any
  // order with "insert if not full or smaller than the largest, evicting the
  // largest" (cuda_utils_kernels.cuh:220-225).  Returns the smallest position a
  // newcomer took, or `cap` when nothing was inserted.
  __device__ __forceinline__ int merge(unsigned long long key, bool active, WalkCounters& wc) {
    const int lane = lane_id();
    bool keep = active && key < worst;
    const unsigned km0 = __ballot_sync(FULL, keep);
    if (km0 == 0) return cap;
    // pos = number of list keys smaller than the new key
    int pos = 0;
    bool dup = false;
    const int nch = (size + 31) >> 5;
    if (__popc(km0) <= 4 && nch <= 32) {
      // up to four newcomers: two-level search by the whole warp, one newcomer at a time
      for (unsigned mm = km0; mm; mm &= mm - 1) {
        const int b = __ffs(mm) - 1;
        const unsigned long long kb = shfl64(key, b);
        int c = 0;
        if (nch > 1) {
          const unsigned long long pv = (lane < nch) ? (keys[min(lane * 32 + 31, size - 1)] & KEY_MASK) : KEY_MAX;
          c = __popc(__ballot_sync(FULL, pv < kb));  // chunks entirely below kb (lanes >= nch hold KEY_MAX)
        }
        const int i = c * 32 + lane;
        const unsigned long long kv = (i < size) ? (keys[i] & KEY_MASK) : KEY_MAX;
        const unsigned lt = __ballot_sync(FULL, kv < kb);
        const unsigned eq = __ballot_sync(FULL, kv == kb);
        if (lane == b) {
          pos = min(c * 32 + __popc(lt), size);
          dup = eq != 0;
        }
      }
    } else if (__popc(km0) <= 4) {
      // the same for lists of more than 1024 keys: a lane stands for a span of `cs` chunks, the span that holds
      // the newcomer's place is then searched chunk by chunk
      const int cs = (nch + 31) >> 5;
      for (unsigned mm = km0; mm; mm &= mm - 1) {
        const int b = __ffs(mm) - 1;
        const unsigned long long kb = shfl64(key, b);
        const unsigned long long pv =
            (lane * cs < nch) ? (keys[min((lane + 1) * cs * 32 - 1, size - 1)] & KEY_MASK) : KEY_MAX;
        const int c = __popc(__ballot_sync(FULL, pv < kb));  // spans entirely below kb
        int below = 0;
        bool same = false;
        for (int j = 0; j < cs; ++j) {
          const int i = (c * cs + j) * 32 + lane;
          const unsigned long long kv = (i < size) ? (keys[i] & KEY_MASK) : KEY_MAX;
          const unsigned lt = __ballot_sync(FULL, kv < kb);
          same = same || __ballot_sync(FULL, kv == kb) != 0;
          below += __popc(lt);
          if (lt != 0xffffffffu) break;  // the place is in this chunk
        }
        if (lane == b) {
          pos = min(c * cs * 32 + below, size);
          dup = same;
        }
      }
    } else {
      int lo = 0, hi = keep ? size : 0;
      while (__any_sync(FULL, lo < hi)) {
        if (lo < hi) {
          int mid = (lo + hi) >> 1;
          if ((keys[mid] & KEY_MASK) < key) lo = mid + 1;
          else hi = mid;
        }
      }
      pos = lo;
      dup = keep && pos < size && (keys[pos] & KEY_MASK) == key;
    }
    if (dup) keep = false;  // already listed
    const unsigned km = __ballot_sync(FULL, keep);
    if (km == 0) return cap;
    const int m = __popc(km);
    int minpos;
    if (m == 1) {
      // the common case: one newcomer, everything from its position on moves up by one
      minpos = __shfl_sync(FULL, pos, __ffs(km) - 1);
      // windows of 64 keys, top down; both halves are read before either is written (a window's
      // targets lie above everything a lower window reads)
      for (int hi = size; hi > minpos; hi -= 64) {
        const int i = hi - 32 + lane, i2 = i - 32;
        const bool have = i >= minpos, have2 = i2 >= minpos;
        const unsigned long long v = have ? keys[i] : 0ull;
        const unsigned long long v2 = have2 ? keys[i2] : 0ull;
        __syncwarp();
        if (have && i + 1 < cap) keys[i + 1] = v;
        if (have2) keys[i2 + 1] = v2;  // i2 + 1 <= size - 32 < cap
      }
      if (keep) keys[pos] = key;  // pos < cap: either the list is not full or key < worst
    } else {
      int rk = 0;
      for (unsigned mm = km; mm; mm &= mm - 1) {
        const int b = __ffs(mm) - 1;
        const unsigned long long kb = shfl64(key, b);
        rk += (kb < key) ? 1 : 0;
      }
      if (keep) spos[rk] = pos;  // newcomer positions, ascending
      __syncwarp();
      minpos = spos[0];
      const int mypos = (lane < m) ? spos[lane] : 0x7fffffff;
      for (int hi = size; hi > minpos; hi -= 64) {
        // key i moves up by the number of newcomers placed at or before it; that number is the same for a
        // whole window of 32 unless a newcomer lands inside it.  Two windows per turn, both read before
        // either is written.
        const int i = hi - 32 + lane, i2 = i - 32;
        const bool have = i >= minpos, have2 = i2 >= minpos;
        const unsigned long long v = have ? keys[i] : 0ull;
        const unsigned long long v2 = have2 ? keys[i2] : 0ull;
        const int below2 = __popc(__ballot_sync(FULL, mypos <= hi - 64));
        const int below = __popc(__ballot_sync(FULL, mypos <= hi - 32));
        const int upto = __popc(__ballot_sync(FULL, mypos <= hi - 1));
        int cnt = below, cnt2 = below2;
        for (int j = below; j < upto; ++j) cnt += (spos[j] <= i) ? 1 : 0;
        for (int j = below2; j < below; ++j) cnt2 += (spos[j] <= i2) ? 1 : 0;
        __syncwarp();
        if (have && i + cnt < cap) keys[i + cnt] = v;
        if (have2 && i2 + cnt2 < cap) keys[i2 + cnt2] = v2;
      }
      if (keep && pos + rk < cap) keys[pos + rk] = key;
    }
    size = min(cap, size + m);
    cursor = min(cursor, minpos);
    wc.inserts += m;
    __syncwarp();
    worst = (size >= cap) ? (keys[cap - 1] & KEY_MASK) : KEY_MAX;
    return minpos;
  }

  // list = {key}
  __device__ __forceinline__ void seed(unsigned long long key) {
    if (lane_id() == 0) keys[0] = key;
    size = 1;
    cursor = 0;
    worst = cap <= 1 ? (key & KEY_MASK) : KEY_MAX;
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

// One chunk of an adjacency row (lane l holds the id in slot l, -1 = unused): filter through the
// visited table, evaluate the fresh ids, merge them.
template <class Dist>
__device__ __forceinline__ int expand_chunk(Dist& de, WarpList& wl, int nid, int self, WalkCounters& wc) {
  const int lane = lane_id();
  bool fresh = (nid >= 0) && (nid != self);
  if (fresh) fresh = !wl.test_and_set(nid);
  const unsigned fm = __ballot_sync(FULL, fresh);
  if (fm == 0) return wl.cap;
  const int n = __popc(fm);
  if (fresh) wl.spos[__popc(fm & ((1u << lane) - 1))] = nid;
  __syncwarp();
  const int cid = wl.spos[lane];
  // the shuffles inside eval() order this read before any later write of spos
  const float dist = de.eval(cid, n);
  wc.evals += n;
  return wl.merge(mkkey(dist, cid), lane < n, wc);
}

// Whole adjacency row; `rows` is a sentinel-padded table: unused slots hold -1.
template <class Dist>
__device__ __forceinline__ void expand_row(Dist& de, WarpList& wl, const int* __restrict__ row, int stride,
                                           int self, WalkCounters& wc) {
  const int lane = lane_id();
  for (int base = 0; base < stride; base += 32) {
    const int l = base + lane;
    const int nid = (l < stride) ? __ldg(row + l) : -1;
    expand_chunk(de, wl, nid, self, wc);
  }
}

// Row number of node `id` in the adjacency table of `level`: layer 0 is indexed by id,
// the upper layers of a node are stored consecutively from upper_base[id].
__device__ __forceinline__ size_t row_index(const int* __restrict__ upper_base, int level, int id) {
  return level == 0 ? (size_t)id : (size_t)__ldg(upper_base + id) + (size_t)(level - 1);
}

// ef-bounded best-first search of one layer.  The list must already hold the
// seeds; on return it holds the min(ef, reachable) closest nodes, ascending.
// While the neighbours of the current node are gathered, the first 32 slots of
// the adjacency row of the likely next node (the key after the cursor) are
// already on their way; a newcomer that overtakes it costs one ordinary load.
template <class Dist>
__device__ __forceinline__ void beam_layer(Dist& de, WarpList& wl, const int* __restrict__ rows, int stride,
                                           const int* __restrict__ upper_base, int level, int self,
                                           WalkCounters& wc) {
  const int lane = lane_id();
  int pf_node = -1, pf_val = -1;
  wl.advance();
  if (wl.cursor >= wl.size) return;
  unsigned long long k = wl.keys[wl.cursor];
  for (;;) {
    // k = keys[cursor] is the closest unexpanded key
    const unsigned long long k2 = (wl.cursor + 1 < wl.size) ? wl.keys[wl.cursor + 1] : KEY_FLAG;
    if (lane == 0) wl.keys[wl.cursor] = k | KEY_FLAG;
    __syncwarp();
    const int cur = key_id(k);
    const int* row = rows + row_index(upper_base, level, cur) * stride;
    int nid;
    if (cur == pf_node) {
      nid = pf_val;
    } else {
      nid = (lane < stride) ? __ldg(row + lane) : -1;
    }
    pf_node = -1;
    if (!(k2 & KEY_FLAG)) {
      pf_node = key_id(k2);
      const int* nrow = rows + row_index(upper_base, level, pf_node) * stride;
      pf_val = (lane < stride) ? __ldg(nrow + lane) : -1;
    }
    wc.expansions += 1;
    const int at = wl.cursor;  // position of the key being expanded; insertions at or before it move the cursor
    int first_new = expand_chunk(de, wl, nid, self, wc);
    for (int base = 32; base < stride; base += 32) {
      const int l = base + lane;
      first_new = min(first_new, expand_chunk(de, wl, (l < stride) ? __ldg(row + l) : -1, self, wc));
    }
    // next key: a newcomer placed at or before at + 1, else the old successor if it is still unexpanded,
    // else scan on
    if (first_new > at + 1 && !(k2 & KEY_FLAG)) {
      // no newcomer in front of the old successor: it sits at at + 1 unchanged
      wl.cursor = at + 1;
      k = k2;
      continue;
    }
    __syncwarp();
    wl.advance();
    if (wl.cursor >= wl.size) break;
    k = wl.keys[wl.cursor];
  }
}

// reverse_cand variant (cuda_utils_kernels.cuh:113-124 of the reference): every step expands
// the FARTHEST unexpanded key of the list; the walk ends when every key is expanded.
template <class Dist>
__device__ __forceinline__ void beam_layer_reverse(Dist& de, WarpList& wl, const int* __restrict__ rows, int stride,
                                                   const int* __restrict__ upper_base, int level, int self,
                                                   WalkCounters& wc) {
  const int lane = lane_id();
  int hi = wl.size - 1;  // every key above `hi` is expanded
  for (;;) {
    int at = -1;
    for (int base = hi & ~31; hi >= 0 && base >= 0; base -= 32) {
      const int i = base + lane;
      const bool open = (i <= hi) && !(wl.keys[i] & KEY_FLAG);
      const unsigned m = __ballot_sync(FULL, open);
      if (m) {
        at = base + 31 - __clz(m);
        break;
      }
    }
    if (at < 0) break;
    const unsigned long long k = wl.keys[at];
    __syncwarp();
    if (lane == 0) wl.keys[at] = k | KEY_FLAG;
    __syncwarp();
    const int* row = rows + row_index(upper_base, level, key_id(k)) * stride;
    wc.expansions += 1;
    int first_new = wl.cap;
    for (int base = 0; base < stride; base += 32) {
      const int l = base + lane;
      first_new = min(first_new, expand_chunk(de, wl, (l < stride) ? __ldg(row + l) : -1, self, wc));
    }
    __syncwarp();
    hi = (first_new < wl.cap) ? wl.size - 1 : at - 1;
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
