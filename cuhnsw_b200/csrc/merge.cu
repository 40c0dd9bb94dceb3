// k-way merge of per-shard top-k lists into a global top-k (base-sharded search).
// The reference has no multi-GPU path (README.md:146 of the reference); this is the exchange
// step that follows an all-gather of every shard's (distance, id) rows.
#include "kernels.h"
#include "common.cuh"

namespace hnsw {

// lists: per part nq x k ids (-1 = empty slot) and distances; part p starts at ids/dist + p * part_stride
// (part_stride = nq * k for two dense parts x nq x k blocks, 2 * nq * k for the parts x 2 x nq x k buffer one
// all-gather fills).  With `offsets`, ids are local to their shard and offsets[p] makes them global.  One
// warp per query: every candidate counts the keys smaller than its own and writes itself at that rank.
__global__ void __launch_bounds__(128) merge_topk_kernel(const int* __restrict__ ids, const float* __restrict__ dist,
                                                         long long part_stride, const int* __restrict__ offsets,
                                                         int parts, long long nq, int k, int* __restrict__ out_ids,
                                                         float* __restrict__ out_dist, int* __restrict__ out_found) {
  extern __shared__ unsigned long long skeys[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = parts * k;
  unsigned long long* mine = skeys + (size_t)warp * total;
  for (long long q = (long long)blockIdx.x * 4 + warp; q < nq; q += (long long)gridDim.x * 4) {
    for (int e = lane; e < total; e += 32) {
      int p = e / k, j = e % k;
      size_t at = (size_t)p * part_stride + (size_t)q * k + j;
      int id = ids[at];
      if (id >= 0 && offsets) id += offsets[p];
      mine[e] = id >= 0 ? mkkey(dist[at], id) : ~0ull;
    }
    __syncwarp();
    int valid = 0;
    for (int e = lane; e < total; e += 32) {
      unsigned long long ke = mine[e];
      if (ke == ~0ull) continue;
      valid++;
      int rank = 0;
      for (int f = 0; f < total; ++f) {
        unsigned long long kf = mine[f];
        rank += (kf < ke || (kf == ke && f < e)) ? 1 : 0;
      }
      if (rank < k) {
        out_ids[(size_t)q * k + rank] = key_id(ke);
        out_dist[(size_t)q * k + rank] = key_dist(ke);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) valid += __shfl_xor_sync(FULL, valid, off);
    int found = valid < k ? valid : k;
    for (int j = found + lane; j < k; j += 32) {
      out_ids[(size_t)q * k + j] = -1;
      out_dist[(size_t)q * k + j] = __int_as_float(0x7f800000);
    }
    if (lane == 0 && out_found) out_found[q] = found;
    __syncwarp();
  }
}

cudaError_t launch_merge_topk(const int* ids, const float* dist, long long part_stride, const int* offsets, int parts,
                              long long nq, int k, int* out_ids, float* out_dist, int* out_found,
                              cudaStream_t stream) {
  if (nq <= 0) return cudaSuccess;
  size_t smem = (size_t)4 * parts * k * sizeof(unsigned long long);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(merge_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  long long blocks = (nq + 3) / 4;
  if (blocks > 148 * 16) blocks = 148 * 16;
  merge_topk_kernel<<<(unsigned)blocks, 128, smem, stream>>>(ids, dist, part_stride, offsets, parts, nq, k, out_ids,
                                                             out_dist, out_found);
  return cudaGetLastError();
}

}  // namespace hnsw
