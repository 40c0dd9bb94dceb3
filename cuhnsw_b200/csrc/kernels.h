// Host-visible parameter blocks and launchers of the CUDA kernels.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace hnsw {

// Device-resident index.  All ids are global node ids on every layer.
struct GraphView {
  const void* vec;        // n x vstride elements, rows zero padded, 32-byte aligned rows
  int vstride;            // elements per row (row_stride_elements)
  int rows16;             // 0: fp32 rows; 1: IEEE half; 2: bfloat16 (round to nearest even of the input).  Distances
                          // are always the fp32 distances over the stored values
  int d;
  int dist_type;          // 0 dot (-dot), 1 l2 (squared)
  long long n;
  int* rows0;             // n x stride0, -1 padded
  int stride0;            // ints per layer-0 row (multiple of 8, >= max_m0)
  int* rowsU;             // total_upper x strideU, -1 padded
  int strideU;
  const int* upper_base;  // n: index of a node's layer-1 row in rowsU (exclusive prefix sum of levels)
  int max_level;
  int enter_point;
};

struct SearchParams {
  GraphView g;
  const float* queries;  // nq x d, unpadded
  long long nq;
  int topk;
  int ef;
  int vsize;             // visited table entries per warp (power of two)
  int reverse_cand;      // expand the farthest unexpanded key first
  int team = -1;         // rows wider than 128 floats: 1 = one CTA per query, 0 = one warp per query, -1 = by batch size
  int smem_per_warp;     // filled by the launcher
  const int* labels;     // optional id -> label map (index loaded from a file)
  int* out_ids;          // nq x topk
  float* out_dist;       // nq x topk
  int* out_found;        // nq
  unsigned long long* ticket;  // work counter (zeroed by the launcher)
  unsigned long long* stats;   // optional: evals, expansions, sweeps, inserts
  // filled by the launcher when it schedules the batch (see SearchSchedule): ticket t serves query order[t],
  // whose greedy descent through the upper layers has already ended at entry_node / entry_dist
  const int* order = nullptr;
  const int* entry_node = nullptr;
  const float* entry_dist = nullptr;
};

// Scratch for longest-first scheduling of a batch that needs more than one wave of warps.  A query's walk
// is a chain of dependent steps; a few per cent of the queries need two to three times the median number
// of steps, and when one of those starts in the last wave the whole launch waits for it.  Those queries
// are the ones whose descent through the upper layers ends far from the query, so a first kernel does
// that descent for every query, the queries are sorted by the distance it ended at (farthest first), and
// the search kernel serves them in that order, starting from the stored entry.  Results do not depend on
// the order.  All arrays hold `capacity` elements.
struct SearchSchedule {
  long long capacity;
  int* entry_node;
  float* entry_dist;
  unsigned* keys;         // sort keys: farthest entry first
  unsigned* keys_sorted;
  int* index;             // 0, 1, 2, ...
  int* order;             // query numbers, sorted
  void* sort_tmp;
  size_t sort_tmp_bytes;
};
size_t search_schedule_tmp_bytes(long long nq);

// `sched` may be null: queries are then served in input order and descend inside the search kernel.
cudaError_t launch_search(const SearchParams& p, int sm_count, cudaStream_t stream,
                          const SearchSchedule* sched = nullptr);
size_t search_smem_per_cta(int d, int ef, int vsize, long long n);
// which search kernel a batch gets: rows <= 128 floats; wide rows with many / some / few queries
enum SearchKernelKind { kSearchWarpSmall = 0, kSearchWarp = 1, kSearchWarpDeep = 2, kSearchTeam = 3 };
int search_kernel_kind(int d, long long nq, int team, int reverse_cand, int sm_count);
// d > 128 only: one CTA of four warps per query, the extra warps share the distance evaluations
cudaError_t launch_search_team(const SearchParams& p, int sm_count, cudaStream_t stream,
                               const SearchSchedule* sched = nullptr);
// first stage of a scheduled search: descent of every query + sort; fills p.order / entry_node / entry_dist
cudaError_t schedule_search(SearchParams& p, const SearchSchedule& sched, int sm_count, cudaStream_t stream);
// search whose device staging and work ticket live in a fixed file-scope device array (no allocation)
size_t search_static_capacity();
size_t search_static_bytes(long long nq, int d, int topk);
cudaError_t search_static(const SearchParams& proto, const float* h_queries, int* h_ids, float* h_dist, int* h_found,
                          int sm_count, cudaStream_t stream);

// ---- construction -------------------------------------------------------
struct BuildLevel {
  GraphView g;           // rows of the level being built are read through rows/stride below
  int level;
  int* rows;             // this level's adjacency table (rows0 or rowsU view)
  float* dists;          // stored edge distances, same shape as rows
  const float* distU;    // distance table of the upper layers (source when a row is copied down)
  int stride;            // ints per row of this level
  int max_m;             // link budget of this level (max_m0 on level 0)
  const int* levels;     // n
  const int* nodes;      // node list of the level, ascending ids (nullptr on level 0: identity)
  long long n_level;
  unsigned char* went;   // n: row has been through neighbour selection on this level
  int ef_construction;
  float heuristic_coef;
  int save_remains;
  int reverse_cand;
  int vsize;
};

struct BuildScratch {
  int* st_ids;                  // bmax x stride: staged own rows
  float* st_dist;
  unsigned* pkeys;              // bmax x stride proposal keys: target node id (n = none)
  unsigned* pkeys_sorted;
  unsigned long long* pvals;    // source node id << 32 | distance bits
  unsigned long long* pvals_sorted;
  void* sort_tmp;
  size_t sort_tmp_bytes;
  unsigned long long* ticket;   // 2 counters
  unsigned long long* stats;    // optional
};

size_t build_sort_tmp_bytes(long long max_items);
// rows of `level` for every node of the level: copy from the level above or seed with the descent result
cudaError_t launch_init_level(const BuildLevel& L, unsigned long long* ticket, int sm_count, cudaStream_t stream);
// one insertion batch: nodes [first, first + count) of the level's node list
cudaError_t launch_build_batch(const BuildLevel& L, const BuildScratch& S, long long first, int count,
                               int sm_count, cudaStream_t stream);
// elements per stored row: d rounded up to 8 floats, or whole pairs of chunk columns of halves
int row_stride_elements(int d, int rows16);
// pads n fp32 rows of d elements (row r starts at src + r * src_stride; src_stride = d for a dense matrix,
// the record length in words for rows embedded in index-file records) into n x vstride rows of floats or
// halves, and back
cudaError_t launch_pad_rows(const float* src, long long src_stride, void* dst, long long n, int d, int vstride,
                            int rows16, cudaStream_t stream);
cudaError_t launch_unpad_rows(const void* src, float* dst, long long dst_stride, long long n, int d, int vstride,
                              int rows16, cudaStream_t stream);
cudaError_t launch_fill_i32(int* p, long long n, int v, cudaStream_t stream);
// Level-0 records of an hnswlib index file, already on the device (`count` records of `rec_words` 32-bit words:
// degree word, max_m0 neighbour slots, the vector, a 64-bit label): writes the -1 padded adjacency rows and
// the labels truncated to int (cpp/src/cuhnsw_base.cu:300-324).  A degree above max_m0, a neighbour id outside
// [0, n) or an id listed twice in one row stores 1 + the smallest offending record number in *bad (which the
// caller presets to all ones).
cudaError_t launch_unpack_links(const unsigned* records, long long rec_words, long long count, long long first,
                                int max_m0, long long n, int* rows, int stride, int* labels,
                                unsigned long long* bad, cudaStream_t stream);
// The other direction, for save_index: `count` adjacency rows become the degree word, the packed neighbour
// slots and the label (= first + record number) of level-0 records laid out on the device as in the file
// (cpp/src/cuhnsw_base.cu:196-214); launch_unpad_rows with dst = records + 1 + max_m0 and dst_stride = rec_words
// fills in the vectors.
cudaError_t launch_pack_links(const int* rows, int stride, long long count, long long first, int max_m0,
                              unsigned* records, long long rec_words, cudaStream_t stream);
// merges per-shard rows (part p at ids/dist + p * part_stride, nq x k each, -1 = empty; offsets[p], when given,
// turns shard-local ids into global ones) into nq x k rows ordered by (distance, id)
cudaError_t launch_merge_topk(const int* ids, const float* dist, long long part_stride, const int* offsets, int parts,
                              long long nq, int k, int* out_ids, float* out_dist, int* out_found,
                              cudaStream_t stream);
// out[i] = canonical distance between stored rows src[i] and dst[i]
cudaError_t launch_batch_distance(const GraphView& g, const int* src, const int* dst, long long npairs, float* out,
                                  cudaStream_t stream);

// self-tests of the candidate list and the visited table (host arrays in and out; see selftest.cu)
cudaError_t selftest_list_host(int cap, const float* dist, const int* ids, const int* batch_begin, int nbatches,
                               const int* expand, unsigned long long* out_keys, int* out_size, int* out_minpos,
                               int* out_cursor);
cudaError_t selftest_visited_host(int entries, long long n, const int* ids, int count, int* seen);

}  // namespace hnsw
