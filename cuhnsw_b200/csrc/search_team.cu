// Batch kNN search for few queries over long rows: one CTA of kTeamWarps warps per query.
//
// With d = 960 a row is 3840 bytes and one warp needs several dependent round trips to gather the
// ~9 fresh rows of a step; with only ~1000 queries there are fewer queries than warp slots, so the
// machine idles.  Here warp 0 runs the very same walk as knn_search_kernel (greedy descent, sorted list,
// visited table) and the other warps of the CTA only help with the distances: every evaluation request is
// posted in shared memory, each warp takes every kTeamWarps-th row, two block barriers frame the step.
// The distance code and its summation order are the ones of the single-warp kernel, so results stay
// bit-identical.  (Reference counterpart: SearchGraphKernel with block_dim > 32,
// cpp/include/cuda_search_kernels.cuh:79-165, where the extra warps split every single row instead.)
#include "kernels.h"
#include "beam.cuh"

namespace hnsw {

constexpr int kTeamWarps = 4;

struct TeamMailbox {
  int n;  // rows to evaluate; -1 = the walk is over
  int ids[32];
  float dist[32];
  int pad[3];
};

// Distance engine of warp 0: same interface as DistLargeT, evaluation shared with the helper warps.
template <class Base>
struct DistTeam {
  Base base;
  TeamMailbox* mb;

  __device__ __forceinline__ void load_query(const float* qp) { base.load_query(qp); }
  __device__ __forceinline__ float eval(int id, int n) {
    const int lane = lane_id();
    if (lane < n) mb->ids[lane] = id;
    if (lane == 0) mb->n = n;
    __syncthreads();  // request visible to the helpers
    const int cnt = (n + kTeamWarps - 1) / kTeamWarps;
    const int mine = (lane < cnt) ? mb->ids[lane * kTeamWarps] : 0;
    const float d = base.eval(mine, cnt);
    if (lane < cnt) mb->dist[lane * kTeamWarps] = d;
    __syncthreads();  // all shares written
    return lane < n ? mb->dist[lane] : 0.0f;
  }
};

template <class Base>
__global__ void __launch_bounds__(kTeamWarps * 32, 16 / kTeamWarps) knn_search_team_kernel(SearchParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t qbytes = Base::smem_bytes(p.g.d);
  TeamMailbox* mb = reinterpret_cast<TeamMailbox*>(smem + qbytes);
  unsigned char* list_mem = smem + qbytes + sizeof(TeamMailbox);
  const VecTable tab = make_table(p.g);
  Base base;
  base.init(tab, smem);  // every warp reads the one query copy in shared memory

  if (warp != 0) {
    // helper: barrier, read the request, evaluate rows warp, warp + W, ..., barrier.  Exactly two barriers
    // per request and one for the final "over", mirroring warp 0.
    for (;;) {
      __syncthreads();
      const int n = mb->n;
      if (n < 0) return;
      const int cnt = n > warp ? (n - warp + kTeamWarps - 1) / kTeamWarps : 0;
      if (cnt > 0) {
        const int mine = (lane < cnt) ? mb->ids[warp + lane * kTeamWarps] : 0;
        const float d = base.eval(mine, cnt);
        if (lane < cnt) mb->dist[warp + lane * kTeamWarps] = d;
      }
      __syncthreads();
    }
  }

  DistTeam<Base> de{base, mb};
  WarpList wl;
  wl.bind(list_mem, p.ef, p.vsize, p.g.n);
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
    wl.seed(mkkey(dcur, cur));
    wl.mark(cur);
    beam_layer(de, wl, p.g.rows0, p.g.stride0, p.g.upper_base, 0, -1, wc);
    const int found = min(wl.size, p.topk);
    for (int j = lane; j < p.topk; j += 32) {
      int id = -1;
      float dist = __int_as_float(0x7f800000);
      if (j < found) {
        const unsigned long long k = wl.keys[j];
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
  // release the helpers: this is the only way out of the kernel for warp 0
  if (lane == 0) mb->n = -1;
  __syncthreads();
}

size_t search_team_smem(int d, int ef, int vsize, long long n) {
  return (DistLarge::smem_bytes(d) + sizeof(TeamMailbox) + WarpList::smem_bytes(ef, vsize, n) + 15) / 16 * 16;
}

cudaError_t launch_search_team(const SearchParams& p0, int sm_count, cudaStream_t stream,
                               const SearchSchedule* sched) {
  SearchParams p = p0;
  const size_t smem = search_team_smem(p.g.d, p.ef, p.vsize, p.g.n);
  p.smem_per_warp = (int)smem;
#define CALL(R) knn_search_team_kernel<typename Pick<R>::Team>
  auto kern = HNSW_WITH_ROWS(p.g.rows16, CALL);
#undef CALL
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kTeamWarps * 32, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorInvalidConfiguration;
  long long grid = (long long)per_sm * sm_count;
  if (grid > p.nq) grid = p.nq;
  if (grid < 1) grid = 1;
  if (sched && p.nq > grid && p.nq <= sched->capacity && p.nq <= 0x7fffffffll) {  // more queries than resident CTAs: long walks first
    e = schedule_search(p, *sched, sm_count, stream);
    if (e != cudaSuccess) return e;
  }
  e = cudaMemsetAsync(p.ticket, 0, sizeof(unsigned long long), stream);
  if (e != cudaSuccess) return e;
  kern<<<(unsigned)grid, kTeamWarps * 32, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace hnsw
