/*
 * C ABI of the B200 HNSW engine (libcuhnsw_b200.so).
 *
 * Every entry point takes plain pointers and sizes, returns 0 on success and a
 * negative status otherwise (no C++ exception crosses this boundary); the text
 * of the last error of a handle is available from cuhnsw_last_error().  The
 * functions are exactly what a binding of the reference's host class needs:
 * each one names the reference method it stands for (paths inside the
 * reference project).  One handle owns one device-resident index on one GPU
 * (plus replicas on further GPUs when the option `devices` lists them);
 * calls on one handle must not overlap.
 */
#ifndef CUHNSW_B200_H_
#define CUHNSW_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cuhnsw_handle cuhnsw_handle;

enum {
  CUHNSW_OK = 0,
  CUHNSW_INVALID_ARGUMENT = -1,
  CUHNSW_IO_ERROR = -2,      /* option or index file cannot be opened / is truncated */
  CUHNSW_PARSE_ERROR = -3,   /* option file is not valid JSON / index file is inconsistent */
  CUHNSW_INVALID_OPTION = -4,/* e.g. dist_type other than "dot" or "l2" */
  CUHNSW_CUDA_ERROR = -5,    /* includes "no CUDA device": there is no CPU path */
  CUHNSW_BAD_STATE = -6,     /* call order: init -> set_data -> set_random_levels -> build_graph */
  CUHNSW_UNSUPPORTED = -7,
  CUHNSW_OUT_OF_MEMORY = -8, /* host allocation failed inside the call */
  CUHNSW_INTERNAL_ERROR = -9 /* an unexpected C++ exception was caught at the boundary */
};

/* CuHNSWBind() constructor + cuhnsw::CuHNSW::CuHNSW()  (cuhnsw/bindings.cc:20, cpp/src/cuhnsw_base.cu:13-62) */
cuhnsw_handle* cuhnsw_create(void);
/* destructor (cpp/src/cuhnsw_base.cu:65) */
void cuhnsw_destroy(cuhnsw_handle* h);
/* text of the last failure on this handle; valid until the next call on it */
const char* cuhnsw_last_error(const cuhnsw_handle* h);

/* CuHNSWBind::Init -> CuHNSW::Init(opt_path)  (cuhnsw/bindings.cc:22-24, cpp/src/cuhnsw_base.cu:67-106).
 * opt_path: JSON object with the field names of cuhnsw/proto/config.proto:9-27.
 * IO/PARSE errors correspond to the reference returning false; INVALID_OPTION to its runtime_error.
 * Keys beyond the reference's schema (all optional): device_id (GPU of the handle; default: the current device),
 * devices (array of GPU numbers: the index is built or loaded on the first and copied to the others, and
 * cuhnsw_search_knn cuts every batch into contiguous slices, one per listed GPU, searched at the same time by one
 * host thread each; results equal the single-GPU results row for row; a GPU may be listed more than once),
 * batch_max, ramp_div (insertion batch schedule), search_team, search_schedule, zero_copy (page-locked host
 * buffers are read and written in place by the search kernels), row_dtype ("f32", "f16", "bf16"). */
int cuhnsw_init(cuhnsw_handle* h, const char* opt_path);

/* CuHNSWBind::SetData -> CuHNSW::SetData  (cuhnsw/bindings.cc:26-33, cpp/src/cuhnsw_base.cu:108-128).
 * data: num_data x num_dims row-major fp32 on the host; copied, the pointer is not retained. */
int cuhnsw_set_data(cuhnsw_handle* h, const float* data, int64_t num_data, int32_t num_dims);

/* CuHNSWBind::SetRandomLevels -> CuHNSW::SetRandomLevels  (cuhnsw/bindings.cc:39-44, cpp/src/cuhnsw_base.cu:130-156).
 * levels: num_data int32, node i belongs to layers 0..levels[i]. */
int cuhnsw_set_random_levels(cuhnsw_handle* h, const int32_t* levels);

/* CuHNSWBind::BuildGraph -> CuHNSW::BuildGraph  (cuhnsw/bindings.cc:35-37, cpp/src/cuhnsw_build.cu:96-208) */
int cuhnsw_build_graph(cuhnsw_handle* h);

/* CuHNSWBind::SaveIndex / LoadIndex -> CuHNSW::SaveIndex / LoadIndex
 * (cuhnsw/bindings.cc:46-52, cpp/src/cuhnsw_base.cu:159-247, 250-365); hnswlib file layout. */
int cuhnsw_save_index(cuhnsw_handle* h, const char* fpath);
int cuhnsw_load_index(cuhnsw_handle* h, const char* fpath);

/* CuHNSWBind::SearchGraph -> CuHNSW::SearchGraph  (cuhnsw/bindings.cc:54-68, cpp/src/cuhnsw_build.cu:210-290).
 * Host buffers: qdata num_queries x num_dims; nns/distances num_queries x topk; found_cnt num_queries.
 * ef_search is raised to topk.  Distances: squared l2, or -dot.  Rows are ascending by (distance, id);
 * slots past found_cnt[i] hold -1 / +inf.  Ids are file labels when the index came from load_index. */
int cuhnsw_search_knn(cuhnsw_handle* h, const float* qdata, int64_t num_queries, int32_t topk, int32_t ef_search,
                      int32_t* nns, float* distances, int32_t* found_cnt);

/* Same search with every buffer already on the engine's GPU; enqueued on the engine's stream and not
 * waited for.  Device-resident counterpart of the kernel launch inside CuHNSW::SearchGraph
 * (cpp/src/cuhnsw_build.cu:254-274) without its per-call copies. */
int cuhnsw_search_knn_device(cuhnsw_handle* h, const float* d_qdata, int64_t num_queries, int32_t topk,
                             int32_t ef_search, int32_t* d_nns, float* d_distances, int32_t* d_found_cnt);

/* cuhnsw_search_knn without the wait at its end: the copy of the queries to the GPU, the kernels and the copies
 * of the results back are enqueued on the engine's stream (cuhnsw_set_stream) and the call returns; nns,
 * distances and found_cnt are complete once that stream has reached this point (cuhnsw_synchronize, or the
 * caller's own event).  The host buffers should be page-locked, or the copies wait for the host.  No counterpart in
 * the reference, whose SearchGraph blocks (cpp/src/cuhnsw_build.cu:210-290).
 * Searches enqueued on DIFFERENT streams (set the stream before each call; this call and cuhnsw_search_knn_device)
 * may run at the same time: every stream gets its own scratch, up to eight streams at once, a ninth waits for
 * the least recently used one.  A launch lasts as long as its longest walk, so a serving loop that rotates its
 * batches over two to four streams fills the tail of each batch with the next one.  One host thread per handle,
 * as for every other call.  cuhnsw_set_data, cuhnsw_build_graph and cuhnsw_load_index first wait for every search
 * enqueued so far; the caller may destroy a stream once its own work on it is complete.  A handle with `devices` set searches on its first device only through this call. */
int cuhnsw_search_knn_async(cuhnsw_handle* h, const float* qdata, int64_t num_queries, int32_t topk, int32_t ef_search,
                            int32_t* nns, float* distances, int32_t* found_cnt);

/* The same on a handle with `devices`: replica 0 is the first listed GPU, cuhnsw_replica_count gives their number
 * (1 without `devices`).  The stream must belong to the replica's GPU (cuhnsw_stream_create_on makes one); the
 * handle's own stream setting is left alone.  A host that rotates its batches over the replicas, several streams
 * each, keeps every GPU busy from one thread.  No counterpart in the reference (single device). */
int cuhnsw_replica_count(const cuhnsw_handle* h);
int cuhnsw_stream_create_on(cuhnsw_handle* h, int32_t replica, void** out_stream);
int cuhnsw_search_knn_async_on(cuhnsw_handle* h, int32_t replica, void* cuda_stream, const float* qdata,
                               int64_t num_queries, int32_t topk, int32_t ef_search, int32_t* nns, float* distances,
                               int32_t* found_cnt);

/* Search for callers that must not allocate.  No counterpart in the reference (its SearchGraph allocates a dozen
 * device vectors per call, cpp/src/cuhnsw_build.cu:241-249).  Same arguments and results as cuhnsw_search_knn (host
 * buffers), but once the index is in place (cuhnsw_set_data or cuhnsw_load_index has run on this handle: they
 * create the handle's few words of device counters) the call itself reaches no cudaMalloc/cudaFree or other
 * allocating routine: the device copies of the queries and results and the kernel's work ticket live in one
 * fixed 4 MiB array inside the library image, which every GPU that loads the library keeps until the process
 * exits.  Meant for processes whose device memory is
 * already owned by their own pool or capped by a budget (a late allocation would fail), and for loops that cannot
 * take the device-wide synchronisation an allocation implies.
 *  - Limit: 256 + 4*num_queries*num_dims + 8*num_queries*topk + 4*num_queries bytes (each term rounded up to
 *    256) must not exceed 4 MiB, e.g. 10 000 queries of 50 dims at topk 10; larger requests fail with
 *    CUHNSW_INVALID_ARGUMENT and a message that states both numbers.
 *  - The first call on a device looks up the array's device address (a one-time set-up per device); make that
 *    first call before any stream capture is started.
 *  - The CUDA runtime loads a kernel into device memory the first time it is launched.  Which search kernel runs
 *    depends on the row width class (<= 32, 64, 96, 128 floats, wider), row_dtype, reverse_cand and, for rows wider
 *    than 128 floats, the batch size class; the first call of each combination therefore takes that memory and
 *    belongs in the warm-up of a process that later runs with its pool full.
 *  - The array is shared by all handles and calls of the process on that device and keeps the previous call's
 *    contents; the call clears the one word that has to start at zero.  Calls that overlap on the GPU (two
 *    threads, two streams) race on it: issue them one after the other. */
int cuhnsw_search_knn_noalloc(cuhnsw_handle* h, const float* qdata, int64_t num_queries, int32_t topk,
                              int32_t ef_search, int32_t* nns, float* distances, int32_t* found_cnt);

/* out[i] = distance between stored rows src[i] and dst[i] (host arrays): squared l2 or -dot, in the engine's
 * fixed fp32 summation order.  Counterpart of BatchDistanceKernel (cpp/include/cuda_dist_kernels.cuh:143-156). */
int cuhnsw_batch_distance(cuhnsw_handle* h, const int32_t* src, const int32_t* dst, int64_t num_pairs, float* out);

/* Stream the engine launches on (a cudaStream_t passed as void*); default: the legacy default stream.
 * The reference launches on the default stream only (cpp/src/cuhnsw_build.cu:66,163,254). */
int cuhnsw_set_stream(cuhnsw_handle* h, void* cuda_stream);
/* cudaDeviceSynchronize of the reference (cpp/src/cuhnsw_build.cu:80,185,275), on the engine's stream */
int cuhnsw_synchronize(cuhnsw_handle* h);

/* For hosts without a CUDA binding of their own (the Python layer's search_knn_batches): a stream on the handle's
 * GPU to pass to cuhnsw_set_stream, and page-locked host memory for cuhnsw_search_knn_async.  No counterpart in
 * the reference.  cuhnsw_stream_create stores the stream in *out_stream; cuhnsw_stream_destroy first waits for
 * it; cuhnsw_host_alloc returns NULL when the allocation fails. */
int cuhnsw_stream_create(cuhnsw_handle* h, void** out_stream);
int cuhnsw_stream_synchronize(cuhnsw_handle* h, void* cuda_stream);
int cuhnsw_stream_destroy(cuhnsw_handle* h, void* cuda_stream);
void* cuhnsw_host_alloc(cuhnsw_handle* h, size_t bytes);
void cuhnsw_host_free(cuhnsw_handle* h, void* ptr);

/* Work counters, the counterpart of acc_visited_cnt (cpp/include/cuda_search_kernels.cuh:141-143):
 * out4 = {rows gathered for a distance, layer rows expanded, greedy sweeps, keys inserted} since the last read. */
int cuhnsw_enable_stats(cuhnsw_handle* h, int32_t on);
int cuhnsw_get_stats(cuhnsw_handle* h, uint64_t* out4);

/* out8 = {num_data, num_dims, max_level, enter_point, max_m, max_m0, upper-layer rows, SM count}
 * (the values CuHNSW::LoadIndex logs, cpp/src/cuhnsw_base.cu:286-287) */
int cuhnsw_describe(cuhnsw_handle* h, int64_t* out8);
/* Host copies of the graph, the flat form of LevelGraph (cpp/include/level_graph.hpp:23-89):
 * levels[num_data]; rows0[num_data x max_m0]; rows_upper[upper rows x max_m], -1 padded; any may be NULL. */
int cuhnsw_get_graph(cuhnsw_handle* h, int32_t* levels, int32_t* rows0, int32_t* rows_upper);
/* wall seconds of the last cuhnsw_build_graph */
double cuhnsw_last_build_seconds(const cuhnsw_handle* h);

/* Base-sharded search: merges `parts` per-shard result blocks (d_ids/d_distances: parts x num_queries x topk,
 * ids already global, -1 = empty slot) into num_queries x topk rows ordered by (distance, id); all device
 * pointers, enqueued on cuda_stream.  No counterpart in the reference, which is single-device
 * (README.md:146 there); it consumes the rows cuhnsw_search_knn_device produces on every shard. */
int cuhnsw_merge_topk_device(const int32_t* d_ids, const float* d_distances, int32_t parts, int64_t num_queries,
                             int32_t topk, int32_t* d_out_ids, float* d_out_distances, int32_t* d_out_found,
                             void* cuda_stream);

/* The same merge, reading the buffer ONE all-gather fills: d_gathered is parts x 2 x num_queries x topk int32, block
 * [p][0] the ids of shard p (local to the shard), block [p][1] the bit patterns of its distances; d_id_offsets[p]
 * (may be NULL) is added to every valid id of shard p.  Each rank's search writes its two blocks in place, the
 * collective (NCCL all-gather over NVLink) exchanges them, and this kernel reads them where they landed: no
 * repacking copy on either side.  No counterpart in the reference (single-device). */
int cuhnsw_merge_topk_gathered_device(const int32_t* d_gathered, const int32_t* d_id_offsets, int32_t parts,
                                      int64_t num_queries, int32_t topk, int32_t* d_out_ids, float* d_out_distances,
                                      int32_t* d_out_found, void* cuda_stream);

/* Self-tests of the two shared-memory structures every walk uses, for checking them against a host model
 * (host arrays in and out, runs on the current GPU, one warp).  They pin the semantics the reference spreads
 * over PushNodeToSearchPq / CheckAlreadyExists / GetCand (cpp/include/cuda_utils_kernels.cuh:50-151,212-227:
 * insert while there is room, else replace the largest key if the new one is smaller; no key twice; the next
 * key to expand is the smallest unexpanded one) and CheckVisited (:185-210: may forget, never invents).
 *
 * list_merge: batch b holds the pairs [batch_begin[b], batch_begin[b+1]) (at most 32) of distances/ids and is
 * merged in one step into a list of `capacity` keys; before it, the expand_before[b] smallest unexpanded keys
 * are marked expanded.  out_keys (capacity slots): the final list, ascending by (distance, id); a key is
 * ord(distance) << 32 | expanded << 31 | id with ord the order-preserving image of the float bits.
 * out_first_position[b]: smallest position a key of batch b took, or capacity.  out_cursor: position of the
 * smallest unexpanded key (= *out_size when there is none). */
int cuhnsw_selftest_list_merge(int32_t capacity, const float* distances, const int32_t* ids,
                               const int32_t* batch_begin, int32_t num_batches, const int32_t* expand_before,
                               uint64_t* out_keys, int32_t* out_size, int32_t* out_first_position,
                               int32_t* out_cursor);
/* visited: feeds ids[0..count) one by one to a table of `entries` slots (a power of two in 64..32768) sized
 * for an index of num_nodes nodes; out_seen[i] = 1 when the table reported ids[i] as already seen. */
int cuhnsw_selftest_visited(int32_t entries, int64_t num_nodes, const int32_t* ids, int32_t count, int32_t* out_seen);

#ifdef __cplusplus
}
#endif
#endif /* CUHNSW_B200_H_ */
