// Batch kNN search over a device-resident graph: greedy descent through the upper layers and the
// ef_search-bounded layer-0 search in ONE launch (knn_search_kernel), or, for batches that need more
// than one wave of warps, a descent kernel, a sort of the queries by entry distance and the same search
// kernel serving the farthest entries first (entry_kernel, schedule_search).
//
// Replaces GetEntryPointsKernel + SearchGraphKernel and their host driver
// (cpp/include/cuda_search_kernels.cuh:11-165, cpp/src/cuhnsw_build.cu:210-290),
// which re-flatten and re-upload the graph on every call, launch once per
// layer and keep the heap in global memory.
#include <cub/block/block_radix_sort.cuh>
#include <cub/device/device_radix_sort.cuh>

#include "kernels.h"
#include "beam.cuh"

namespace hnsw {

constexpr int kWarpsPerCta = 2;
// batches of up to this many queries are ordered by one CTA (sort_schedule_kernel) instead of the four kernels
// of a device-wide radix sort (10 000 queries on a B200: 19 us in one launch against 27 us in four)
constexpr long long kBlockSortMax = 10240;

template <class Dist, bool kReverse>
__global__ void __launch_bounds__(kWarpsPerCta * 32, Dist::kSearchMinCtas)
knn_search_kernel(SearchParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* mine = smem + (size_t)warp * p.smem_per_warp;
  Dist de;
  const VecTable tab = make_table(p.g);
  de.init(tab, mine);
  WarpList wl;
  wl.bind(mine + Dist::smem_bytes(p.g.d), p.ef, p.vsize, p.g.n);
  WalkCounters wc{0, 0, 0, 0};

  for (;;) {
    long long qi = 0;
    if (lane == 0) qi = (long long)atomicAdd(p.ticket, 1ull);
    qi = __shfl_sync(FULL, qi, 0);
    if (qi >= p.nq) break;
    if (p.order) qi = __ldg(p.order + qi);
    de.load_query(p.queries + (size_t)qi * p.g.d);
    wl.reset();
    int cur;
    float dcur;
    if (p.entry_node) {
      cur = __ldg(p.entry_node + qi);
      dcur = __ldg(p.entry_dist + qi);
    } else {
      cur = p.g.enter_point;
      dcur = de.eval(cur, 1);
      dcur = __shfl_sync(FULL, dcur, 0);
      wc.evals += 1;
      greedy_descent(de, wl.spos, p.g.rowsU, p.g.strideU, p.g.upper_base, p.g.max_level, 0, cur, dcur, wc);
    }
    // layer 0: list = {entry}, visited = {entry} (cuda_search_kernels.cuh:108-112)
    wl.seed(mkkey(dcur, cur));
    wl.mark(cur);
    if (kReverse) beam_layer_reverse(de, wl, p.g.rows0, p.g.stride0, p.g.upper_base, 0, -1, wc);
    else beam_layer(de, wl, p.g.rows0, p.g.stride0, p.g.upper_base, 0, -1, wc);
    // ascending top-k, found = min(size, k); slots past `found` read -1 / +inf
    int found = min(wl.size, p.topk);
    for (int j = lane; j < p.topk; j += 32) {
      int id = -1;
      float dist = __int_as_float(0x7f800000);
      if (j < found) {
        unsigned long long k = wl.keys[j];
        id = key_id(k);
        dist = key_dist(k);
        if (p.labels) id = __ldg(p.labels + id);
      }
      p.out_ids[(size_t)qi * p.topk + j] = id;
      p.out_dist[(size_t)qi * p.topk + j] = dist;
    }
    if (lane == 0) p.out_found[qi] = found;
    __syncwarp();
  }
  if (p.stats && lane == 0) {
    atomicAdd(p.stats + 0, (unsigned long long)wc.evals);
    atomicAdd(p.stats + 1, (unsigned long long)wc.expansions);
    atomicAdd(p.stats + 2, (unsigned long long)wc.sweeps);
    atomicAdd(p.stats + 3, (unsigned long long)wc.inserts);
  }
}

// First stage of a scheduled search: one warp per query walks down the upper layers
// (GetEntryPointsKernel of the reference, cuda_search_kernels.cuh:11-77, all layers in one launch) and
// leaves where it ended, how far that is, and a sort key that puts the farthest entries first.
template <class Dist>
__global__ void __launch_bounds__(kWarpsPerCta * 32) entry_kernel(SearchParams p, SearchSchedule s) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int scratch[kWarpsPerCta][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long qi = (long long)blockIdx.x * kWarpsPerCta + warp;
  if (qi >= p.nq) return;
  Dist de;
  const VecTable tab = make_table(p.g);
  de.init(tab, smem + (size_t)warp * Dist::smem_bytes(p.g.d));
  WalkCounters wc{0, 0, 0, 0};
  de.load_query(p.queries + (size_t)qi * p.g.d);
  int cur = p.g.enter_point;
  float dcur = de.eval(cur, 1);
  dcur = __shfl_sync(FULL, dcur, 0);
  wc.evals += 1;
  greedy_descent(de, scratch[warp], p.g.rowsU, p.g.strideU, p.g.upper_base, p.g.max_level, 0, cur, dcur, wc);
  if (lane == 0) {
    s.entry_node[qi] = cur;
    s.entry_dist[qi] = dcur;
    // sort key: farthest entry first.  Small batches are sorted by one CTA (sort_schedule_kernel), which wants
    // the query number in the low half of the word.
    const unsigned key = ~f2ord(dcur);
    s.keys[qi] = p.nq <= kBlockSortMax ? ((key & 0xffff0000u) | (unsigned)qi) : key;
    s.index[qi] = (int)qi;
    if (p.stats) {
      atomicAdd(p.stats + 0, (unsigned long long)wc.evals);
      atomicAdd(p.stats + 2, (unsigned long long)wc.sweeps);
    }
  }
}

template <class Dist>
static cudaError_t launch_entry_t(const SearchParams& p, const SearchSchedule& s, cudaStream_t stream) {
  const size_t smem = Dist::smem_bytes(p.g.d) * kWarpsPerCta;
  auto kern = entry_kernel<Dist>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const long long grid = (p.nq + kWarpsPerCta - 1) / kWarpsPerCta;
  kern<<<(unsigned)grid, kWarpsPerCta * 32, smem, stream>>>(p, s);
  return cudaGetLastError();
}

template <class Row>
static cudaError_t launch_entry_rows(const SearchParams& p, const SearchSchedule& s, cudaStream_t stream) {
  using E = Pick<Row>;
  const int d = p.g.d;
  return d <= 32    ? launch_entry_t<typename E::D32>(p, s, stream)
         : d <= 64  ? launch_entry_t<typename E::D64>(p, s, stream)
         : d <= 96  ? launch_entry_t<typename E::D96>(p, s, stream)
         : d <= 128 ? launch_entry_t<typename E::D128>(p, s, stream)
                    : launch_entry_t<typename E::Wide>(p, s, stream);
}

// Orders up to kBlockSortMax packed words (sort key in the upper 16 bits, query number in the lower 16) with one
// CTA: a block-wide radix sort over the key bits, stable, so equal keys stay in query order.  Writes the query
// numbers in sorted order.
constexpr int kBlockSortThreads = 1024, kBlockSortItems = 10;
__global__ void __launch_bounds__(kBlockSortThreads) sort_schedule_kernel(const unsigned* __restrict__ words, int nq,
                                                                          int* __restrict__ order) {
  using Sort = cub::BlockRadixSort<unsigned, kBlockSortThreads, kBlockSortItems>;
  __shared__ typename Sort::TempStorage tmp;
  unsigned mine[kBlockSortItems];
#pragma unroll
  for (int i = 0; i < kBlockSortItems; ++i) {
    const int at = threadIdx.x * kBlockSortItems + i;
    mine[i] = at < nq ? words[at] : 0xffffffffu;
  }
  Sort(tmp).Sort(mine, 16, 32);
#pragma unroll
  for (int i = 0; i < kBlockSortItems; ++i) {
    const int at = threadIdx.x * kBlockSortItems + i;
    if (at < nq) order[at] = (int)(mine[i] & 0xffffu);
  }
}

size_t search_schedule_tmp_bytes(long long nq) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const unsigned*)nullptr, (unsigned*)nullptr, (const int*)nullptr,
                                  (int*)nullptr, (int)nq, 16, 32);
  return bytes;
}

cudaError_t schedule_search(SearchParams& p, const SearchSchedule& s, int sm_count, cudaStream_t stream) {
  (void)sm_count;
  if (p.nq > s.capacity || p.nq > 0x7fffffffll) return cudaErrorInvalidValue;  // the sort counts items in an int
#define CALL(R) launch_entry_rows<R>(p, s, stream)
  cudaError_t e = HNSW_WITH_ROWS(p.g.rows16, CALL);
#undef CALL
  if (e != cudaSuccess) return e;
  // the upper 16 bits of the key (sign, exponent, 7 bits of mantissa) order the queries finely enough
  if (p.nq <= kBlockSortMax) {
    sort_schedule_kernel<<<1, kBlockSortThreads, 0, stream>>>(s.keys, (int)p.nq, s.order);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    p.order = s.order;
    p.entry_node = s.entry_node;
    p.entry_dist = s.entry_dist;
    return cudaSuccess;
  }
  size_t bytes = s.sort_tmp_bytes;
  e = cub::DeviceRadixSort::SortPairs(s.sort_tmp, bytes, (const unsigned*)s.keys, s.keys_sorted, (const int*)s.index,
                                      s.order, (int)p.nq, 16, 32, stream);
  if (e != cudaSuccess) return e;
  p.order = s.order;
  p.entry_node = s.entry_node;
  p.entry_dist = s.entry_dist;
  return cudaSuccess;
}

template <class Dist, bool kReverse>
static cudaError_t launch_search_tr(const SearchParams& p0, int sm_count, cudaStream_t stream,
                                    const SearchSchedule* sched);

template <class Dist>
static cudaError_t launch_search_t(const SearchParams& p0, int sm_count, cudaStream_t stream,
                                   const SearchSchedule* sched) {
  return p0.reverse_cand ? launch_search_tr<Dist, true>(p0, sm_count, stream, sched)
                         : launch_search_tr<Dist, false>(p0, sm_count, stream, sched);
}

template <class Dist, bool kReverse>
static cudaError_t launch_search_tr(const SearchParams& p0, int sm_count, cudaStream_t stream,
                                    const SearchSchedule* sched) {
  SearchParams p = p0;
  size_t per_warp = Dist::smem_bytes(p.g.d) + WarpList::smem_bytes(p.ef, p.vsize, p.g.n);
  per_warp = (per_warp + 15) / 16 * 16;
  p.smem_per_warp = (int)per_warp;
  size_t smem = per_warp * kWarpsPerCta;
  auto kern = knn_search_kernel<Dist, kReverse>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kWarpsPerCta * 32, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorInvalidConfiguration;
  long long want = (p.nq + kWarpsPerCta - 1) / kWarpsPerCta;
  long long grid = (long long)per_sm * sm_count;
  if (grid > want) grid = want;
  if (grid < 1) grid = 1;
  // more queries than resident warps: start the long walks first
  if (sched && p.nq > grid * kWarpsPerCta && p.nq <= sched->capacity && p.nq <= 0x7fffffffll) {
    e = schedule_search(p, *sched, sm_count, stream);
    if (e != cudaSuccess) return e;
  }
  e = cudaMemsetAsync(p.ticket, 0, sizeof(unsigned long long), stream);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)grid, kWarpsPerCta * 32, smem, stream>>>(p);
  return cudaGetLastError();
}

size_t search_smem_per_cta(int d, int ef, int vsize, long long n) {
  size_t dq = d <= 128 ? 0 : DistLarge::smem_bytes(d);
  size_t per_warp = (dq + WarpList::smem_bytes(ef, vsize, n) + 15) / 16 * 16;
  return per_warp * kWarpsPerCta;
}

// Rows wider than 128 floats, fewer queries than warp slots: resident warps do not matter, the time of one
// step does.  Up to 7 queries per SM one CTA of four warps per query shares the distance evaluations of every
// step; up to 10 per SM one warp per query keeps 32 float4 loads in flight instead of 16.
// Measured on 1M x 960 (ef 100 / 500): 100 queries 0.85 / 3.0 ms against 1.47 / 4.3 ms with one warp per
// query, 1000 queries 1.48 / 5.9 against 1.74 / 6.0 ms, 1480 queries 1.79 / 7.2 against 2.17 / 6.8 ms.
int search_kernel_kind(int d, long long nq, int team, int reverse_cand, int sm_count) {
  if (d <= 128) return kSearchWarpSmall;
  if (!reverse_cand && (team == 1 || (team < 0 && nq <= (long long)sm_count * 7))) return kSearchTeam;
  if (nq <= (long long)sm_count * 10) return kSearchWarpDeep;
  return kSearchWarp;
}

template <class Row>
static cudaError_t launch_search_rows(const SearchParams& p, int sm_count, cudaStream_t stream,
                                      const SearchSchedule* sched) {
  using E = Pick<Row>;
  const int d = p.g.d;
  if (d <= 32) return launch_search_t<typename E::D32>(p, sm_count, stream, sched);
  if (d <= 64) return launch_search_t<typename E::D64>(p, sm_count, stream, sched);
  if (d <= 96) return launch_search_t<typename E::D96>(p, sm_count, stream, sched);
  if (d <= 128) return launch_search_t<typename E::D128>(p, sm_count, stream, sched);
  switch (search_kernel_kind(d, p.nq, p.team, p.reverse_cand, sm_count)) {
    case kSearchTeam: return launch_search_team(p, sm_count, stream, sched);
    case kSearchWarpDeep: return launch_search_t<typename E::WideDeep>(p, sm_count, stream, sched);
    default: break;
  }
  return launch_search_t<typename E::Wide>(p, sm_count, stream, sched);
}

cudaError_t launch_search(const SearchParams& p, int sm_count, cudaStream_t stream, const SearchSchedule* sched) {
  if (p.nq <= 0) return cudaSuccess;
#define CALL(R) launch_search_rows<R>(p, sm_count, stream, sched)
  return HNSW_WITH_ROWS(p.g.rows16, CALL);
#undef CALL
}

}  // namespace hnsw

// ---------------------------------------------------------------------------
// Search that allocates nothing
// ---------------------------------------------------------------------------
// Some callers must not reach cudaMalloc: a serving process that has already handed every free byte of
// device memory to its own pool allocator (a late cudaMalloc there fails or evicts), a job running under a
// fixed memory budget, or a real-time loop that cannot take the device-wide synchronisation cudaMalloc and
// cudaFree imply.  For them the staging buffers and the work ticket of the search kernel live in one
// file-scope device array of fixed size instead of grow-on-demand allocations.  Every GPU that loads this
// library carries the array (4 MiB) until the process exits.
//
// In host code the name `g_search_scratch` is only the runtime's handle of the symbol, not a device address:
// a kernel given `g_search_scratch` from the host would fault or, where the GPU can reach host memory, use the
// wrong memory.  The device address is obtained once per device with cudaGetSymbolAddress (with that device
// current) and it is that pointer that is handed to the kernel.
#include <mutex>

namespace hnsw {

constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr int kMaxDevices = 64;
static __device__ __align__(256) unsigned char g_search_scratch[kStaticScratchBytes];

static std::mutex g_scratch_mu;
static void* g_scratch_addr[kMaxDevices] = {};

static cudaError_t static_scratch_address(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_search_scratch);  // set-up: first call on this device
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_scratch_addr[dev]);
  return cudaSuccess;
}

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }

size_t search_static_capacity() { return kStaticScratchBytes; }

size_t search_static_bytes(long long nq, int d, int topk) {
  return 256 + align256((size_t)nq * d * sizeof(float)) + 2 * align256((size_t)nq * topk * 4) +
         align256((size_t)nq * sizeof(int));
}

// Host buffers in and out; the caller has checked search_static_bytes() <= search_static_capacity().
// Layout of the array: [ticket | queries | ids | distances | found].  Only the ticket has to start at zero and
// the launcher clears it on the stream; everything else is overwritten before it is read.  The array is shared
// by every call in the process on this device, so two calls that overlap on the GPU race on it.
cudaError_t search_static(const SearchParams& proto, const float* h_queries, int* h_ids, float* h_dist, int* h_found,
                          int sm_count, cudaStream_t stream) {
  unsigned char* base = nullptr;
  cudaError_t e = static_scratch_address(&base);
  if (e != cudaSuccess) return e;
  const long long nq = proto.nq;
  const size_t qbytes = (size_t)nq * proto.g.d * sizeof(float), rbytes = (size_t)nq * proto.topk * 4;
  SearchParams p = proto;
  p.ticket = reinterpret_cast<unsigned long long*>(base);
  p.stats = nullptr;
  unsigned char* at = base + 256;
  float* d_q = reinterpret_cast<float*>(at);
  at += align256(qbytes);
  p.out_ids = reinterpret_cast<int*>(at);
  at += align256(rbytes);
  p.out_dist = reinterpret_cast<float*>(at);
  at += align256(rbytes);
  p.out_found = reinterpret_cast<int*>(at);
  p.queries = d_q;
  if ((e = cudaMemcpyAsync(d_q, h_queries, qbytes, cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e;
  if ((e = launch_search(p, sm_count, stream)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(h_ids, p.out_ids, rbytes, cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(h_dist, p.out_dist, rbytes, cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
  if ((e = cudaMemcpyAsync(h_found, p.out_found, (size_t)nq * sizeof(int), cudaMemcpyDeviceToHost, stream)) !=
      cudaSuccess)
    return e;
  return cudaStreamSynchronize(stream);
}

}  // namespace hnsw
