// Per-level graph construction without locks.
//
// The reference inserts all nodes of a level in one launch and serialises row
// updates with a per-node spin lock (atomicCAS on mutex[], cpp/include/
// cuda_build_kernels.cuh:197,227,261,301), so its result depends on timing.
// Here a level is inserted in deterministic batches of consecutive nodes; each
// batch runs three launches and nothing ever waits on another warp:
//
//   A  search + own-row selection against the graph as it was before the
//      batch (cuda_build_kernels.cuh:196-292 for one node); rows are staged.
//   B  staged rows are copied into the graph and every new edge (src -> dst)
//      becomes a reverse-link proposal keyed by dst; proposals are grouped by
//      a stable radix sort on dst (ascending src inside a group).
//   C  one warp per target node folds its proposals into the row one by one in
//      ascending source order, each through the reference's neighbour selection
//      with its newcomer shortcut (cuda_build_kernels.cuh:295-332).
//
// Nodes of one batch do not see each other while searching, exactly as nodes
// that are in flight together do not in the reference.
#include <cub/device/device_radix_sort.cuh>

#include "kernels.h"
#include "beam.cuh"

namespace hnsw {

constexpr int kBuildWarps = 2;
constexpr int kMaxLinks = 64;  // largest supported link budget (max_m0)

// Per-warp shared memory of the build kernels, after the Dist block and the WarpList block.
struct SelBuf {
  int* ids;       // kMaxLinks
  float* dist;    // kMaxLinks
  unsigned long long* tmp;  // kMaxLinks + 8 unsorted keys
  __host__ __device__ static constexpr size_t smem_bytes() {
    return kMaxLinks * 4 + kMaxLinks * 4 + (kMaxLinks + 8) * 8;
  }
  __device__ __forceinline__ void bind(void* p) {
    tmp = reinterpret_cast<unsigned long long*>(p);
    ids = reinterpret_cast<int*>(tmp + kMaxLinks + 8);
    dist = reinterpret_cast<float*>(ids + kMaxLinks);
  }
};

// Neighbour selection of the reference (SearchHeuristic, cuda_build_kernels.cuh:68-162).
// cands: ascending keys (distance to the row owner, id), flags ignored.  Writes
// sel.ids/sel.dist and returns the new degree.  The distance engine's query is
// overwritten.
template <class Dist>
__device__ __forceinline__ int select_neighbors(Dist& de, const unsigned long long* cands, int nc, int m,
                                                int nn_num, int save_remains, int new_comer, SelBuf& sel,
                                                WalkCounters& wc) {
  const int lane = lane_id();
  int head = 0;
  int tail = min(m, nc) - 1;
  const int max_head = tail + 1;
  bool nc_in = false;
  for (int j = 0; j < nc; ++j) {
    if (head >= m) break;
    const unsigned long long k = cands[j];
    const int cid = key_id(k);
    const float cd = key_dist(k);
    const bool freepass = head < nn_num || (new_comer >= 0 && !nc_in && cid != new_comer);
    if (freepass) {
      if (lane == 0) {
        sel.ids[head] = cid;
        sel.dist[head] = cd;
      }
      head++;
      __syncwarp();
      continue;
    }
    bool skip = false;
    de.load_query_row(cid);
    if (new_comer >= 0 && nc_in) {
      float dd = de.eval(new_comer, 1);
      dd = __shfl_sync(FULL, dd, 0);
      wc.evals += 1;
      skip = cd > dd;
    } else {
      // the accepted neighbours are tested four at a time (one distance pass), closest first: most
      // candidates are turned down by one of the first ones, and the rows of the others are then never
      // read (1.18 M x 50: build 0.208 -> 0.192 s; 8 per vote 0.201 s)
      constexpr int kVote = 4;
      for (int base = 0; base < head; base += kVote) {
        int n = min(kVote, head - base);
        int id = (lane < n) ? sel.ids[base + lane] : 0;
        float dd = de.eval(id, n);
        wc.evals += n;
        if (__any_sync(FULL, lane < n && cd > dd)) {
          skip = true;
          break;
        }
      }
    }
    if (cid == new_comer && !skip) nc_in = true;
    if (skip && tail >= head) {
      if (lane == 0) {
        sel.ids[tail] = cid;
        sel.dist[tail] = cd;
      }
      tail--;
    } else if (!skip) {
      if (lane == 0) {
        sel.ids[head] = cid;
        sel.dist[head] = cd;
      }
      head++;
    }
    __syncwarp();
  }
  __syncwarp();
  return save_remains ? max_head : head;
}

template <class Dist>
__device__ __forceinline__ void bind_warp(unsigned char* smem, int per_warp, const GraphView& g, int cap, int vsize,
                                          Dist& de, WarpList& wl, SelBuf& sel) {
  unsigned char* mine = smem + (size_t)(threadIdx.x >> 5) * per_warp;
  const VecTable tab = make_table(g);
  de.init(tab, mine);
  mine += Dist::smem_bytes(g.d);
  wl.bind(mine, cap, vsize, g.n);
  mine += WarpList::smem_bytes(cap, vsize, g.n);
  sel.bind(mine);
}

template <class Dist>
__host__ __device__ inline size_t build_smem_per_warp(int d, int cap, int vsize, long long n) {
  return (Dist::smem_bytes(d) + WarpList::smem_bytes(cap, vsize, n) + SelBuf::smem_bytes() + 15) / 16 * 16;
}

// ---------------------------------------------------------------------------
// initial rows of a level (cpp/src/cuhnsw_build.cu:113-142)
// ---------------------------------------------------------------------------
struct InitParams {
  BuildLevel L;
  int per_warp;
  unsigned long long* ticket;
};

template <class Dist>
__global__ void __launch_bounds__(kBuildWarps * 32) init_level_kernel(InitParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31;
  const BuildLevel& L = p.L;
  Dist de;
  WarpList wl;
  SelBuf sel;
  bind_warp(smem, p.per_warp, L.g, 32, 32, de, wl, sel);
  WalkCounters wc{0, 0, 0, 0};
  const int l = L.level;
  for (;;) {
    long long t = 0;
    if (lane == 0) t = (long long)atomicAdd(p.ticket, 1ull);
    t = __shfl_sync(FULL, t, 0);
    if (t >= L.n_level) break;
    const int i = L.nodes ? __ldg(L.nodes + t) : (int)t;
    int* row = L.rows + row_index(L.g.upper_base, l, i) * L.stride;
    float* drow = L.dists + row_index(L.g.upper_base, l, i) * L.stride;
    if (lane == 0) L.went[i] = 0;
    const int lv = __ldg(L.levels + i);
    if (lv > l) {
      // keep the finished row of the level above, with its stored distances
      const size_t ur = row_index(L.g.upper_base, l + 1, i) * L.g.strideU;
      const int* urow = L.g.rowsU + ur;
      const float* udist = L.distU + ur;
      for (int j = lane; j < L.stride; j += 32) {
        row[j] = (j < L.g.strideU) ? urow[j] : -1;
        drow[j] = (j < L.g.strideU) ? udist[j] : 0.0f;
      }
    } else if (l == L.g.max_level) {
      // top level: one edge to the enter point (cuhnsw_build.cu:130,137-142); the enter point itself starts empty
      float dd = 0.0f;
      if (i != L.g.enter_point) {
        de.load_query_row(i);
        dd = de.eval(L.g.enter_point, 1);
        dd = __shfl_sync(FULL, dd, 0);
      }
      for (int j = lane; j < L.stride; j += 32) {
        row[j] = (j == 0 && i != L.g.enter_point) ? L.g.enter_point : -1;
        drow[j] = (j == 0) ? dd : 0.0f;
      }
    } else {
      de.load_query_row(i);
      int cur = L.g.enter_point;
      float dcur = de.eval(cur, 1);
      dcur = __shfl_sync(FULL, dcur, 0);
      greedy_descent(de, wl.spos, L.g.rowsU, L.g.strideU, L.g.upper_base, L.g.max_level, l, cur, dcur, wc);
      for (int j = lane; j < L.stride; j += 32) {
        row[j] = (j == 0) ? cur : -1;
        drow[j] = (j == 0) ? dcur : 0.0f;
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// phase A: search + own-row selection, staged
// ---------------------------------------------------------------------------
struct BatchParams {
  BuildLevel L;
  BuildScratch S;
  long long first;
  int count;
  int per_warp;
  int cap;
  long long total;  // count * stride proposals
  int nn_num;
};

template <class Dist>
__global__ void __launch_bounds__(kBuildWarps * 32, Dist::kBuildMinCtas) build_search_kernel(BatchParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31;
  const BuildLevel& L = p.L;
  Dist de;
  WarpList wl;
  SelBuf sel;
  bind_warp(smem, p.per_warp, L.g, p.cap, L.vsize, de, wl, sel);
  // the shared-memory block is laid out for p.cap keys (at least a full row plus one, which the
  // reverse-link kernel needs); the search itself keeps ef_construction keys
  wl.cap = L.ef_construction;
  WalkCounters wc{0, 0, 0, 0};
  for (;;) {
    long long t = 0;
    if (lane == 0) t = (long long)atomicAdd(p.S.ticket, 1ull);
    t = __shfl_sync(FULL, t, 0);
    if (t >= p.count) break;
    const int s = L.nodes ? __ldg(L.nodes + p.first + t) : (int)(p.first + t);
    de.load_query_row(s);
    wl.reset();
    // seeds: the node's current row (cuda_build_kernels.cuh:203-212)
    expand_row(de, wl, L.rows + row_index(L.g.upper_base, L.level, s) * L.stride, L.stride, s, wc);
    if (L.reverse_cand) beam_layer_reverse(de, wl, L.rows, L.stride, L.g.upper_base, L.level, s, wc);
    else beam_layer(de, wl, L.rows, L.stride, L.g.upper_base, L.level, s, wc);
    int deg = select_neighbors(de, wl.keys, wl.size, L.max_m, p.nn_num, L.save_remains, -1, sel, wc);
    int* so = p.S.st_ids + (size_t)t * L.stride;
    float* sd = p.S.st_dist + (size_t)t * L.stride;
    for (int j = lane; j < L.stride; j += 32) {
      so[j] = (j < deg) ? sel.ids[j] : -1;
      sd[j] = (j < deg) ? sel.dist[j] : 0.0f;
    }
    __syncwarp();
  }
  if (p.S.stats && lane == 0) {
    atomicAdd(p.S.stats + 0, (unsigned long long)wc.evals);
    atomicAdd(p.S.stats + 1, (unsigned long long)wc.expansions);
    atomicAdd(p.S.stats + 3, (unsigned long long)wc.inserts);
  }
}

// ---------------------------------------------------------------------------
// phase B: apply staged rows, emit proposals (one thread per row slot)
// ---------------------------------------------------------------------------
__global__ void build_apply_kernel(BatchParams p) {
  const BuildLevel& L = p.L;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= p.total) return;
  const int t = (int)(idx / L.stride), j = (int)(idx % L.stride);
  const int s = L.nodes ? L.nodes[p.first + t] : (int)(p.first + t);
  const int id = p.S.st_ids[idx];
  const float dd = p.S.st_dist[idx];
  const size_t r = row_index(L.g.upper_base, L.level, s) * L.stride + j;
  L.rows[r] = id;
  L.dists[r] = dd;
  if (j == 0) L.went[s] = 1;
  // proposal: key = target node (n = "none", sorts last); value = source node and distance
  p.S.pkeys[idx] = (id >= 0) ? (unsigned)id : (unsigned)L.g.n;
  p.S.pvals[idx] = ((unsigned long long)(unsigned)s << 32) | __float_as_uint(dd);
}

// ---------------------------------------------------------------------------
// phase C: reverse links, one warp per target node
// ---------------------------------------------------------------------------
template <class Dist>
__global__ void __launch_bounds__(kBuildWarps * 32, Dist::kBuildMinCtas) build_reverse_kernel(BatchParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31;
  const BuildLevel& L = p.L;
  Dist de;
  WarpList wl;
  SelBuf sel;
  bind_warp(smem, p.per_warp, L.g, p.cap, 32, de, wl, sel);
  WalkCounters wc{0, 0, 0, 0};
  const unsigned* keys = p.S.pkeys_sorted;
  const unsigned long long* vals = p.S.pvals_sorted;
  const unsigned none = (unsigned)L.g.n;
  const long long nchunk = (p.total + 31) / 32;
  for (;;) {
    long long c = 0;
    if (lane == 0) c = (long long)atomicAdd(p.S.ticket + 1, 1ull);
    c = __shfl_sync(FULL, c, 0);
    if (c >= nchunk) break;
    const long long i = c * 32 + lane;
    const unsigned ki = (i < p.total) ? keys[i] : none;
    const unsigned kprev = (i > 0 && i < p.total) ? keys[i - 1] : none;
    const bool is_head = (ki != none) && (i == 0 || kprev != ki);
    unsigned heads = __ballot_sync(FULL, is_head);
    while (heads) {
      const int b = __ffs(heads) - 1;
      heads &= heads - 1;
      const int dst = (int)__shfl_sync(FULL, ki, b);
      const size_t r = row_index(L.g.upper_base, L.level, dst) * L.stride;
      // the row lives in shared memory while the segment is processed
      int deg = 0;
      for (int base = 0; base < L.stride; base += 32) {
        int j = base + lane;
        int id = (j < L.stride) ? L.rows[r + j] : -1;
        float dd = (j < L.stride) ? L.dists[r + j] : 0.0f;
        unsigned vm = __ballot_sync(FULL, id >= 0);
        if (id >= 0) {
          int at = deg + __popc(vm & ((1u << lane) - 1));
          sel.ids[at] = id;
          sel.dist[at] = dd;
        }
        deg += __popc(vm);
      }
      __syncwarp();
      bool went = L.went[dst] != 0;
      bool changed = false;
      for (long long pi = c * 32 + b; pi < p.total && keys[pi] == (unsigned)dst; ++pi) {
        const unsigned long long v = vals[pi];
        const int s = (int)(v >> 32);
        const float sd = __uint_as_float((unsigned)v);
        // already a neighbour? (IsNeighbor, cuda_build_kernels.cuh:10-66)
        bool present = false;
        for (int base = 0; base < deg; base += 32) {
          int j = base + lane;
          present = present || (j < deg && sel.ids[j] == s);
        }
        if (__any_sync(FULL, present)) continue;
        // candidates = {newcomer} U row \ {self}, ascending (distance, id)
        int ncand = 0;
        if (lane == 0) sel.tmp[0] = mkkey(sd, s);
        ncand = 1;
        for (int base = 0; base < deg; base += 32) {
          int j = base + lane;
          bool ok = (j < deg) && (sel.ids[j] != dst);
          unsigned om = __ballot_sync(FULL, ok);
          if (ok) sel.tmp[ncand + __popc(om & ((1u << lane) - 1))] = mkkey(sel.dist[j], sel.ids[j]);
          ncand += __popc(om);
        }
        __syncwarp();
        for (int e = lane; e < ncand; e += 32) {
          const unsigned long long ke = sel.tmp[e];
          int rank = 0;
          for (int f = 0; f < ncand; ++f) rank += (sel.tmp[f] < ke) ? 1 : 0;
          wl.keys[rank] = ke;
        }
        __syncwarp();
        if (ncand > L.ef_construction) ncand = L.ef_construction;
        const int new_comer = (!L.save_remains && went) ? s : -1;
        deg = select_neighbors(de, wl.keys, ncand, L.max_m, p.nn_num, L.save_remains, new_comer, sel, wc);
        went = true;
        changed = true;
      }
      if (changed) {
        for (int j = lane; j < L.stride; j += 32) {
          L.rows[r + j] = (j < deg) ? sel.ids[j] : -1;
          L.dists[r + j] = (j < deg) ? sel.dist[j] : 0.0f;
        }
        if (lane == 0) L.went[dst] = 1;
      }
      __syncwarp();
    }
  }
  if (p.S.stats && lane == 0) atomicAdd(p.S.stats + 0, (unsigned long long)wc.evals);
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
template <class K>
static cudaError_t grid_for(K kern, size_t smem, int threads, int sm_count, long long want, int* grid) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorInvalidConfiguration;
  long long g = (long long)per_sm * sm_count;
  if (g > want) g = want;
  if (g < 1) g = 1;
  *grid = (int)g;
  return cudaSuccess;
}

static int sort_end_bit(long long n) {
  int b = 1;
  while ((1ll << b) <= n) ++b;
  return b;
}

size_t build_sort_tmp_bytes(long long max_items) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const unsigned*)nullptr, (unsigned*)nullptr,
                                  (const unsigned long long*)nullptr, (unsigned long long*)nullptr,
                                  (int)max_items, 0, 32);
  return bytes;
}

template <class Dist>
static cudaError_t init_level_t(const BuildLevel& L, unsigned long long* ticket, int sm_count, cudaStream_t stream) {
  InitParams p{L, 0, ticket};
  size_t per_warp = build_smem_per_warp<Dist>(L.g.d, 32, 32, L.g.n);
  p.per_warp = (int)per_warp;
  size_t smem = per_warp * kBuildWarps;
  int grid = 1;
  cudaError_t e = grid_for(init_level_kernel<Dist>, smem, kBuildWarps * 32, sm_count,
                           (L.n_level + kBuildWarps - 1) / kBuildWarps, &grid);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(ticket, 0, sizeof(unsigned long long), stream);
  if (e != cudaSuccess) return e;
  init_level_kernel<Dist><<<grid, kBuildWarps * 32, smem, stream>>>(p);
  return cudaGetLastError();
}

template <class Dist>
static cudaError_t build_batch_t(const BuildLevel& L, const BuildScratch& S, long long first, int count,
                                 int sm_count, cudaStream_t stream) {
  BatchParams p;
  p.L = L;
  p.S = S;
  p.first = first;
  p.count = count;
  p.cap = L.ef_construction > kMaxLinks + 8 ? L.ef_construction : kMaxLinks + 8;
  p.total = (long long)count * L.stride;
  p.nn_num = (int)(L.max_m * (double)L.heuristic_coef);
  cudaError_t e = cudaMemsetAsync(S.ticket, 0, 2 * sizeof(unsigned long long), stream);
  if (e != cudaSuccess) return e;
  {
    size_t per_warp = build_smem_per_warp<Dist>(L.g.d, p.cap, L.vsize, L.g.n);
    p.per_warp = (int)per_warp;
    size_t smem = per_warp * kBuildWarps;
    int grid = 1;
    e = grid_for(build_search_kernel<Dist>, smem, kBuildWarps * 32, sm_count,
                 ((long long)count + kBuildWarps - 1) / kBuildWarps, &grid);
    if (e != cudaSuccess) return e;
    build_search_kernel<Dist><<<grid, kBuildWarps * 32, smem, stream>>>(p);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  {
    int threads = 256;
    long long blocks = (p.total + threads - 1) / threads;
    build_apply_kernel<<<(unsigned)blocks, threads, 0, stream>>>(p);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  {
    size_t bytes = S.sort_tmp_bytes;
    e = cub::DeviceRadixSort::SortPairs(S.sort_tmp, bytes, (const unsigned*)S.pkeys, S.pkeys_sorted,
                                        (const unsigned long long*)S.pvals, S.pvals_sorted, (int)p.total, 0,
                                        sort_end_bit(L.g.n), stream);
    if (e != cudaSuccess) return e;
  }
  {
    size_t per_warp = build_smem_per_warp<Dist>(L.g.d, p.cap, 32, L.g.n);
    p.per_warp = (int)per_warp;
    size_t smem = per_warp * kBuildWarps;
    int grid = 1;
    long long chunks = (p.total + 31) / 32;
    e = grid_for(build_reverse_kernel<Dist>, smem, kBuildWarps * 32, sm_count,
                 (chunks + kBuildWarps - 1) / kBuildWarps, &grid);
    if (e != cudaSuccess) return e;
    build_reverse_kernel<Dist><<<grid, kBuildWarps * 32, smem, stream>>>(p);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  return cudaSuccess;
}

#define HNSW_DISPATCH_ROWS(E, d, CALL)           \
  do {                                            \
    if ((d) <= 32) return CALL(typename E::D32);   \
    if ((d) <= 64) return CALL(typename E::D64);   \
    if ((d) <= 96) return CALL(typename E::D96);   \
    if ((d) <= 128) return CALL(typename E::D128); \
    return CALL(typename E::Wide);                 \
  } while (0)

template <class Row>
static cudaError_t init_level_rows(const BuildLevel& L, unsigned long long* ticket, int sm_count, cudaStream_t stream) {
#define CALL(D) init_level_t<D>(L, ticket, sm_count, stream)
  HNSW_DISPATCH_ROWS(Pick<Row>, L.g.d, CALL);
#undef CALL
}
template <class Row>
static cudaError_t build_batch_rows(const BuildLevel& L, const BuildScratch& S, long long first, int count,
                                    int sm_count, cudaStream_t stream) {
#define CALL(D) build_batch_t<D>(L, S, first, count, sm_count, stream)
  HNSW_DISPATCH_ROWS(Pick<Row>, L.g.d, CALL);
#undef CALL
}

cudaError_t launch_init_level(const BuildLevel& L, unsigned long long* ticket, int sm_count, cudaStream_t stream) {
  if (L.n_level <= 0) return cudaSuccess;
#define CALL(R) init_level_rows<R>(L, ticket, sm_count, stream)
  return HNSW_WITH_ROWS(L.g.rows16, CALL);
#undef CALL
}

cudaError_t launch_build_batch(const BuildLevel& L, const BuildScratch& S, long long first, int count,
                               int sm_count, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
#define CALL(R) build_batch_rows<R>(L, S, first, count, sm_count, stream)
  return HNSW_WITH_ROWS(L.g.rows16, CALL);
#undef CALL
}

// ---------------------------------------------------------------------------
// small utility kernels
// ---------------------------------------------------------------------------
__global__ void pad_rows_kernel(const float* src, long long src_stride, float* dst, long long n, int d, int vstride) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = n * vstride;
  for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    long long r = idx / vstride;
    int c = (int)(idx % vstride);
    dst[idx] = (c < d) ? src[r * src_stride + c] : 0.0f;
  }
}
__global__ void unpad_rows_kernel(const float* src, float* dst, long long dst_stride, long long n, int d,
                                  int vstride) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = n * d;
  for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    long long r = idx / d;
    int c = (int)(idx % d);
    dst[r * dst_stride + c] = src[r * vstride + c];
  }
}
// half rows: rounded to nearest even and stored in the paired-column layout of RowF16 (the rows were
// cleared beforehand, so the padding reads zero)
template <class H>
__device__ __forceinline__ H round16(float x);
template <>
__device__ __forceinline__ __half round16<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 round16<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
__device__ __forceinline__ float widen16(__half x) { return __half2float(x); }
__device__ __forceinline__ float widen16(__nv_bfloat16 x) { return __bfloat162float(x); }

template <class H>
__global__ void pad_rows_16_kernel(const float* src, long long src_stride, H* dst, long long n, int d, int vstride) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = n * d;
  for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    long long r = idx / d;
    int e = (int)(idx % d);
    dst[r * vstride + RowF16::position(d, e)] = round16<H>(src[r * src_stride + e]);
  }
}
template <class H>
__global__ void unpad_rows_16_kernel(const H* src, float* dst, long long dst_stride, long long n, int d,
                                     int vstride) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = n * d;
  for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    long long r = idx / d;
    int e = (int)(idx % d);
    dst[r * dst_stride + e] = widen16(src[r * vstride + RowF16::position(d, e)]);
  }
}
// The inverse of unpack_links_kernel: degree word, neighbour ids packed to the front of max_m0 slots (zeros
// after them) and the record's own number as its 64-bit label; the vector words in between are written by the
// unpad kernels.
__global__ void pack_links_kernel(const int* __restrict__ rows, int stride, long long count, long long first,
                                  int max_m0, unsigned* __restrict__ records, long long rec_words) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = count * max_m0;
  for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / max_m0;
    const int j = (int)(idx % max_m0);
    const int* row = rows + r * stride;
    unsigned* rec = records + r * rec_words;
    int before = 0, deg = 0;
    for (int k = 0; k < max_m0; ++k) {
      const int live = row[k] >= 0 ? 1 : 0;
      deg += live;
      before += k < j ? live : 0;
    }
    if (row[j] >= 0) rec[1 + before] = (unsigned)row[j];
    if (j >= deg) rec[1 + j] = 0u;
    if (j == 0) {
      rec[0] = (unsigned)deg;
      const unsigned long long label = (unsigned long long)(first + r);
      rec[rec_words - 2] = (unsigned)label;
      rec[rec_words - 1] = (unsigned)(label >> 32);
    }
  }
}
__global__ void unpack_links_kernel(const unsigned* __restrict__ records, long long rec_words, long long count,
                                    long long first, int max_m0, long long n, int* __restrict__ rows, int stride,
                                    int* __restrict__ labels, unsigned long long* bad) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = count * stride;
  for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / stride;
    const int j = (int)(idx % stride);
    const unsigned* rec = records + r * rec_words;
    const unsigned deg = rec[0] & 0xffffu;  // hnswlib keeps flags in the upper half of this word
    int id = -1;
    if (deg > (unsigned)max_m0) {
      atomicMin(bad, (unsigned long long)(first + r + 1));
    } else if ((unsigned)j < deg) {
      const unsigned v = rec[1 + j];
      bool twice = false;  // an id listed twice in one row would reach the list merge as two equal newcomers
      for (int k = 0; k < j; ++k) twice = twice || rec[1 + k] == v;
      if ((long long)v >= n || twice) atomicMin(bad, (unsigned long long)(first + r + 1));
      else id = (int)v;
    }
    rows[idx] = id;
    if (j == 0 && labels) labels[r] = (int)rec[rec_words - 2];  // low word of the 64-bit label
  }
}
__global__ void fill_i32_kernel(int* p, long long n, int v) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; idx < n; idx += (long long)gridDim.x * blockDim.x) p[idx] = v;
}

static unsigned blocks_for(long long total) {
  long long b = (total + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  if (b < 1) b = 1;
  return (unsigned)b;
}
cudaError_t launch_pad_rows(const float* src, long long src_stride, void* dst, long long n, int d, int vstride,
                            int rows16, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (rows16) {
    cudaError_t e = cudaMemsetAsync(dst, 0, (size_t)n * vstride * 2, stream);
    if (e != cudaSuccess) return e;
    if (rows16 == kRowsBF16)
      pad_rows_16_kernel<<<blocks_for(n * d), 256, 0, stream>>>(src, src_stride, static_cast<__nv_bfloat16*>(dst), n, d,
                                                                vstride);
    else
      pad_rows_16_kernel<<<blocks_for(n * d), 256, 0, stream>>>(src, src_stride, static_cast<__half*>(dst), n, d,
                                                                vstride);
  } else {
    pad_rows_kernel<<<blocks_for(n * vstride), 256, 0, stream>>>(src, src_stride, static_cast<float*>(dst), n, d,
                                                                 vstride);
  }
  return cudaGetLastError();
}
cudaError_t launch_unpack_links(const unsigned* records, long long rec_words, long long count, long long first,
                                int max_m0, long long n, int* rows, int stride, int* labels,
                                unsigned long long* bad, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  unpack_links_kernel<<<blocks_for(count * stride), 256, 0, stream>>>(records, rec_words, count, first, max_m0, n,
                                                                      rows, stride, labels, bad);
  return cudaGetLastError();
}
cudaError_t launch_unpad_rows(const void* src, float* dst, long long dst_stride, long long n, int d, int vstride,
                              int rows16, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  if (rows16 == kRowsBF16)
    unpad_rows_16_kernel<<<blocks_for(n * d), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), dst,
                                                                dst_stride, n, d, vstride);
  else if (rows16)
    unpad_rows_16_kernel<<<blocks_for(n * d), 256, 0, stream>>>(static_cast<const __half*>(src), dst, dst_stride, n,
                                                                d, vstride);
  else
    unpad_rows_kernel<<<blocks_for(n * d), 256, 0, stream>>>(static_cast<const float*>(src), dst, dst_stride, n, d,
                                                             vstride);
  return cudaGetLastError();
}
cudaError_t launch_pack_links(const int* rows, int stride, long long count, long long first, int max_m0,
                              unsigned* records, long long rec_words, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  pack_links_kernel<<<blocks_for(count * max_m0), 256, 0, stream>>>(rows, stride, count, first, max_m0, records,
                                                                    rec_words);
  return cudaGetLastError();
}
cudaError_t launch_fill_i32(int* p, long long n, int v, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  fill_i32_kernel<<<blocks_for(n), 256, 0, stream>>>(p, n, v);
  return cudaGetLastError();
}

}  // namespace hnsw
