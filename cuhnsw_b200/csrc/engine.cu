#include "engine.h"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>

#include "json_min.h"

namespace hnsw {

namespace {
constexpr int kMaxLinksHost = 64;
constexpr int kMaxEf = 8192;

int round_up(int x, int m) { return (x + m - 1) / m * m; }
int next_pow2(long long x) {
  int p = 1;
  while (p < x) p <<= 1;
  return p;
}

#pragma pack(push, 1)
// Header of an hnswlib index file as the reference writes it (cpp/src/cuhnsw_base.cu:182-194).
struct FileHeader {
  uint64_t offset_level0;
  uint64_t max_elements;
  uint64_t cur_element_count;
  uint64_t size_data_per_element;
  uint64_t label_offset;
  uint64_t offset_data;
  int32_t maxlevel;
  uint32_t enterpoint_node;
  uint64_t max_m;
  uint64_t max_m0;
  uint64_t m;
  double mult;
  uint64_t ef_construction;
};
#pragma pack(pop)
static_assert(sizeof(FileHeader) == 96, "hnswlib header is 96 bytes");
}  // namespace

Engine::Engine() {}
Engine::~Engine() {
  for (SearchLane& l : lanes_)
    if (l.done) {
      if (device_ >= 0) cudaSetDevice(device_);
      cudaEventSynchronize(l.done);
      cudaEventDestroy(l.done);
    }
}

int Engine::Fail(int code, const std::string& msg) {
  err_ = msg;
  if (opt_.c_log_level >= 1) std::fprintf(stderr, "[cuhnsw_b200] error: %s\n", msg.c_str());
  return code;
}

int Engine::FailCuda(cudaError_t e, const char* what) {
  std::ostringstream os;
  os << "CUDA error in " << what << ": " << cudaGetErrorString(e);
  return Fail(kCudaError, os.str());
}

void Engine::Log(int level, const char* fmt, ...) const {
  if (opt_.c_log_level < level) return;
  va_list ap;
  va_start(ap, fmt);
  std::fprintf(stderr, "[cuhnsw_b200] ");
  std::vfprintf(stderr, fmt, ap);
  std::fprintf(stderr, "\n");
  va_end(ap);
}

#define CU(call)                                         \
  do {                                                   \
    cudaError_t e__ = (call);                            \
    if (e__ != cudaSuccess) return FailCuda(e__, #call); \
  } while (0)

int Engine::EnsureDevice() {
  if (device_ >= 0) {
    CU(cudaSetDevice(device_));
    return kOk;
  }
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return Fail(kCudaError, "no CUDA device: this library has no CPU path");
  int dev = 0;
  if (opt_.device_id >= 0) {
    dev = opt_.device_id;
    CU(cudaSetDevice(dev));
  } else {
    CU(cudaGetDevice(&dev));
  }
  cudaDeviceProp prop;
  CU(cudaGetDeviceProperties(&prop, dev));
  device_ = dev;
  sm_count_ = prop.multiProcessorCount;
  smem_optin_ = prop.sharedMemPerBlockOptin;
  CU(counters_.alloc(8));
  CU(cudaMemset(counters_.get(), 0, 8 * sizeof(unsigned long long)));
  Log(3, "device %d: %s, sm_%d%d, %d SMs, %zu B shared memory per block", dev, prop.name, prop.major, prop.minor,
      sm_count_, smem_optin_);
  return kOk;
}

int Engine::Init(const char* opt_path, int device_override) {
  if (!opt_path) return Fail(kInvalidArgument, "null option path");
  std::ifstream in(opt_path);
  if (!in.is_open()) return Fail(kIoError, std::string("cannot open option file ") + opt_path);
  std::string text((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  FlatJson js;
  if (!js.parse(text)) return Fail(kParseError, std::string("invalid option file ") + opt_path);
  Options o;
  o.seed = (int)js.number("seed", o.seed);
  o.c_log_level = (int)js.number("c_log_level", o.c_log_level);
  o.max_m = (int)js.number("max_m", o.max_m);
  o.max_m0 = (int)js.number("max_m0", o.max_m0);
  o.ef_construction = (int)js.number("ef_construction", o.ef_construction);
  o.level_mult = js.number("level_mult", o.level_mult);
  o.save_remains = js.boolean("save_remains", o.save_remains);
  o.hyper_threads = js.number("hyper_threads", o.hyper_threads);
  o.block_dim = (int)js.number("block_dim", o.block_dim);
  o.dist_type = js.string("dist_type", o.dist_type);
  o.visited_table_size = (int)js.number("visited_table_size", o.visited_table_size);
  o.visited_list_size = (int)js.number("visited_list_size", o.visited_list_size);
  o.nrz = js.boolean("nrz", o.nrz);
  o.reverse_cand = js.boolean("reverse_cand", o.reverse_cand);
  o.search_team = (int)js.number("search_team", o.search_team);
  o.search_schedule = js.boolean("search_schedule", o.search_schedule);
  o.zero_copy = js.boolean("zero_copy", o.zero_copy);
  o.row_dtype = js.string("row_dtype", o.row_dtype);
  if (o.row_dtype != "f32" && o.row_dtype != "f16" && o.row_dtype != "bf16")
    return Fail(kInvalidArgument, "row_dtype must be f32, f16 or bf16");
  // the reference's schema spells it heuristic_coef, its README heuristic_coff
  o.heuristic_coef = js.number("heuristic_coef", js.number("heuristic_coff", o.heuristic_coef));
  o.batch_max = (long long)js.number("batch_max", (double)o.batch_max);
  o.ramp_div = (long long)js.number("ramp_div", (double)o.ramp_div);
  o.device_id = (int)js.number("device_id", o.device_id);
  for (double v : js.numbers("devices")) {
    if (v < 0 || v > 1023 || v != std::floor(v)) return Fail(kInvalidOption, "devices must list CUDA device numbers");
    o.devices.push_back((int)v);
  }
  if (!o.devices.empty() && o.device_id >= 0 && o.device_id != o.devices[0])
    return Fail(kInvalidOption, "device_id and devices[0] disagree");
  if (!o.devices.empty()) o.device_id = o.devices[0];
  if (device_override >= 0) {  // a replica of a multi-GPU handle: same options, its own GPU
    o.device_id = device_override;
    o.devices.clear();
  }
  opt_.c_log_level = o.c_log_level;
  if (o.dist_type == "dot") dist_type_ = 0;
  else if (o.dist_type == "l2") dist_type_ = 1;
  else return Fail(kInvalidOption, "invalid dist type " + o.dist_type);
  if (o.max_m < 1 || o.max_m0 < 1 || o.max_m > o.max_m0 || o.max_m0 > kMaxLinksHost)
    return Fail(kInvalidOption, "need 1 <= max_m <= max_m0 <= 64");
  if (o.ef_construction < 1 || o.ef_construction > kMaxEf)
    return Fail(kInvalidOption, "need 1 <= ef_construction <= 8192");
  if (o.heuristic_coef < 0.0 || o.heuristic_coef > 1.0)
    return Fail(kInvalidOption, "need 0 <= heuristic_coef <= 1");
  if (o.block_dim < 32 || o.block_dim > 1024 || o.block_dim % 32) return Fail(kInvalidOption, "invalid block_dim");
  if (o.ramp_div < 1) o.ramp_div = 1;
  opt_ = o;
  inited_ = true;
  Log(3, "max_m: %d, max_m0: %d, save_remains: %d, ef_construction: %d, level_mult: %f, dist_type: %s", o.max_m,
      o.max_m0, (int)o.save_remains, o.ef_construction, o.level_mult, o.dist_type.c_str());
  return kOk;
}

int Engine::SetStream(void* stream) {
  stream_ = reinterpret_cast<cudaStream_t>(stream);
  return kOk;
}

int Engine::CreateStream(void** out) {
  if (!out) return Fail(kInvalidArgument, "null out_stream");
  int rc = EnsureDevice();
  if (rc) return rc;
  cudaStream_t s = nullptr;
  CU(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *out = s;
  return kOk;
}

int Engine::SyncStream(void* stream) {
  int rc = EnsureDevice();
  if (rc) return rc;
  CU(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  return kOk;
}

int Engine::DestroyStream(void* stream) {
  int rc = SyncStream(stream);
  if (rc) return rc;
  if (stream_ == reinterpret_cast<cudaStream_t>(stream)) stream_ = nullptr;  // back to the default stream
  if (stream) CU(cudaStreamDestroy(reinterpret_cast<cudaStream_t>(stream)));
  return kOk;
}

void* Engine::HostAlloc(size_t bytes) {
  if (EnsureDevice() != kOk) return nullptr;
  void* p = nullptr;
  if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}

void Engine::HostFree(void* ptr) {
  if (ptr && EnsureDevice() == kOk) cudaFreeHost(ptr);
}

int Engine::Synchronize() {
  int rc = EnsureDevice();
  if (rc) return rc;
  CU(cudaStreamSynchronize(stream_));
  return kOk;
}

int Engine::SetData(const float* data, long long num_data, int num_dims) {
  if (!inited_) return Fail(kBadState, "init() must be called first");
  if (!data && num_data > 0) return Fail(kInvalidArgument, "null data");
  if (num_data < 0 || num_dims < 1) return Fail(kInvalidArgument, "data must be a 2-d array with at least one column");
  if (num_data >= (1ll << 31) - 1) return Fail(kUnsupported, "at most 2^31 - 2 rows per index");
  int rc = AllocRows(num_data, num_dims);
  if (rc) return rc;
  // stage through a bounded device buffer and pad rows on the device
  const long long rows_per_chunk = std::max<long long>(1, (64ll << 20) / num_dims);
  DevBuf<float> raw;
  CU(raw.alloc((size_t)std::min(rows_per_chunk, std::max<long long>(n_, 1)) * num_dims));
  for (long long s = 0; s < n_; s += rows_per_chunk) {
    long long r = std::min(rows_per_chunk, n_ - s);
    CU(cudaMemcpyAsync(raw.get(), data + (size_t)s * num_dims, (size_t)r * num_dims * sizeof(float),
                       cudaMemcpyHostToDevice, stream_));
    CU(launch_pad_rows(raw.get(), num_dims, RowPtr(s), r, num_dims, vstride_, rows16_, stream_));
    CU(cudaStreamSynchronize(stream_));
  }
  has_data_ = true;
  Log(3, "copied data (%lld x %d), row stride %d %s", n_, d_, vstride_, rows16_ ? "16-bit values" : "floats");
  return kOk;
}

// Device storage of num_data rows; whatever graph the handle held is dropped.
int Engine::AllocRows(long long num_data, int num_dims) {
  int rc = EnsureDevice();
  if (rc) return rc;
  // searches still running on other streams read the rows and the graph that are replaced from here on
  if ((rc = WaitForSearches()) != kOk) return rc;
  n_ = num_data;
  d_ = num_dims;
  rows16_ = opt_.row_dtype == "f16" ? 1 : opt_.row_dtype == "bf16" ? 2 : 0;
  vstride_ = row_stride_elements(num_dims, rows16_);  // rows start on 32-byte sectors
  has_data_ = has_levels_ = has_graph_ = labelled_ = false;
  labels_h_.clear();
  labels_d_.release();
  CU(vec_.alloc(((size_t)n_ * vstride_ * (rows16_ ? 2 : 4) + 3) / 4));
  return kOk;
}

int Engine::AllocGraph() {
  stride0_ = round_up(opt_.max_m0, 8);
  strideU_ = round_up(opt_.max_m, 8);
  upper_base_h_.assign((size_t)n_, 0);
  long long acc = 0;
  for (long long i = 0; i < n_; ++i) {
    upper_base_h_[i] = (int)acc;
    acc += levels_h_[i];
    if (acc > (1ll << 30)) return Fail(kUnsupported, "too many upper-layer rows");
  }
  total_upper_ = acc;
  CU(rows0_.alloc((size_t)n_ * stride0_));
  CU(rowsU_.alloc((size_t)std::max<long long>(total_upper_, 1) * strideU_));
  CU(levels_d_.alloc((size_t)std::max<long long>(n_, 1)));
  CU(upper_base_d_.alloc((size_t)std::max<long long>(n_, 1)));
  CU(launch_fill_i32(rows0_.get(), n_ * stride0_, -1, stream_));
  CU(launch_fill_i32(rowsU_.get(), std::max<long long>(total_upper_, 1) * strideU_, -1, stream_));
  if (n_ > 0) {
    CU(cudaMemcpyAsync(levels_d_.get(), levels_h_.data(), (size_t)n_ * sizeof(int), cudaMemcpyHostToDevice, stream_));
    CU(cudaMemcpyAsync(upper_base_d_.get(), upper_base_h_.data(), (size_t)n_ * sizeof(int), cudaMemcpyHostToDevice,
                       stream_));
  }
  CU(cudaStreamSynchronize(stream_));
  return kOk;
}

// Level membership and enter point exactly as cpp/src/cuhnsw_base.cu:130-156:
// node i belongs to levels 0..levels[i]; the enter point is the first node that
// reaches the maximum level.
int Engine::SetRandomLevels(const int* levels) {
  if (!has_data_) return Fail(kBadState, "set_data() must be called first");
  if (!levels && n_ > 0) return Fail(kInvalidArgument, "null levels");
  levels_h_.assign((size_t)n_, 0);
  max_level_ = 0;
  enter_point_ = 0;
  for (long long i = 0; i < n_; ++i) {
    if (levels[i] < 0 || levels[i] > 64) return Fail(kInvalidArgument, "levels must lie in 0..64");
    levels_h_[i] = levels[i];
    if (levels[i] > max_level_) {
      max_level_ = levels[i];
      enter_point_ = (int)i;
    }
  }
  int rc = AllocGraph();
  if (rc) return rc;
  has_levels_ = true;
  has_graph_ = false;
  Log(3, "max level: %d, enter point: %d", max_level_, enter_point_);
  return kOk;
}

GraphView Engine::View() const {
  GraphView g;
  g.vec = vec_.get();
  g.vstride = vstride_;
  g.rows16 = rows16_;
  g.d = d_;
  g.dist_type = dist_type_;
  g.n = n_;
  g.rows0 = rows0_.get();
  g.stride0 = stride0_;
  g.rowsU = rowsU_.get();
  g.strideU = strideU_;
  g.upper_base = upper_base_d_.get();
  g.max_level = max_level_;
  g.enter_point = enter_point_;
  return g;
}

int Engine::ResolveVsize(int cap, long long nq, int* vsize) const {
  int v;
  if (opt_.visited_table_size > 0) {
    v = std::min(32768, std::max(64, next_pow2(opt_.visited_table_size)));
  } else {
    // Largest table that still lets the kernel keep its target number of warps resident per SM
    // (the walk is latency bound: resident warps matter more than a few repeated evaluations),
    // but never below ~4 entries per list slot, where repeats explode.
    // Wide rows and few queries: the kernels chosen there keep 4 CTAs per SM resident whatever the table
    // size, and a repeated evaluation re-reads kilobytes.  Measured on 1M x 960, 1000 queries, ef 500:
    // 3576 evaluations per query and 5.67 ms with 2048 entries, 2099 and 4.98 ms with 16384.
    const int kind = nq < 0 ? kSearchWarp
                            : search_kernel_kind(d_, nq, opt_.search_team, opt_.reverse_cand ? 1 : 0, sm_count_);
    const int warps = d_ <= 128 ? 32 : kind == kSearchTeam ? 4 : kind == kSearchWarpDeep ? 8 : 16;
    const int top = kind == kSearchTeam ? 16384 : kind == kSearchWarpDeep ? 8192 : 4096;
    const long long budget = (long long)smem_optin_ / warps - 640;
    const int floor_entries = std::min(4096, std::max(512, next_pow2(4ll * cap)));
    v = top;
    while (v > floor_entries && (long long)search_smem_per_cta(d_, cap, v, n_) / 2 > budget) v >>= 1;
  }
  while (v > 64 && search_smem_per_cta(d_, cap, v, n_) + 4096 > smem_optin_) v >>= 1;
  if (search_smem_per_cta(d_, cap, v, n_) + 4096 > smem_optin_) return kUnsupported;
  *vsize = v;
  return kOk;
}

int Engine::BuildGraph() {
  if (!has_levels_) return Fail(kBadState, "set_random_levels() must be called before build_graph()");
  int rc = EnsureDevice();
  if (rc) return rc;
  if ((rc = WaitForSearches()) != kOk) return rc;
  auto t0 = std::chrono::steady_clock::now();
  if (n_ == 0) {
    has_graph_ = true;
    return kOk;
  }
  // Insertion batch = nodes that search the same snapshot of the graph.  The reference launches
  // hyper_threads * cores / block_dim blocks, cores = SMs * 128 for this architecture
  // (cpp/src/cuhnsw_base.cu:53-57,111), each inserting one node at a time; four times that number is where
  // the build time stops falling here (1.18 M x 50: 0.311 s at 1x, 0.243 s at 2.4x, 0.226 s at 3.6x,
  // 0.217-0.224 s from 4.8x to 9.6x) and recall@10 does not move (0.954-0.956 over that range).
  long long bmax = opt_.batch_max > 0
                       ? opt_.batch_max
                       : (long long)(4.0 * opt_.hyper_threads * (double)(sm_count_ * 128 / opt_.block_dim));
  bmax = std::max<long long>(1, std::min(bmax, n_));
  const int smax = std::max(stride0_, strideU_);
  int vsize = 0;
  if (ResolveVsize(std::max(opt_.ef_construction, kMaxLinksHost + 8), -1, &vsize) != kOk)
    return Fail(kUnsupported, "ef_construction does not fit in shared memory");
  DevBuf<float> dist0, distU, st_dist;
  DevBuf<unsigned char> went;
  DevBuf<int> st_ids, nodes_d;
  DevBuf<unsigned> pkeys, pkeys_sorted;
  DevBuf<unsigned long long> pvals, pvals_sorted;
  DevBuf<unsigned char> sort_tmp;
  CU(dist0.alloc((size_t)n_ * stride0_));
  CU(distU.alloc((size_t)std::max<long long>(total_upper_, 1) * strideU_));
  CU(went.alloc((size_t)n_));
  CU(st_ids.alloc((size_t)bmax * smax));
  CU(st_dist.alloc((size_t)bmax * smax));
  CU(pkeys.alloc((size_t)bmax * smax));
  CU(pkeys_sorted.alloc((size_t)bmax * smax));
  CU(pvals.alloc((size_t)bmax * smax));
  CU(pvals_sorted.alloc((size_t)bmax * smax));
  size_t tmp_bytes = build_sort_tmp_bytes(bmax * smax);
  CU(sort_tmp.alloc(tmp_bytes + 256));
  // rows start empty on every level
  CU(launch_fill_i32(rows0_.get(), n_ * stride0_, -1, stream_));
  CU(launch_fill_i32(rowsU_.get(), std::max<long long>(total_upper_, 1) * strideU_, -1, stream_));

  std::vector<std::vector<int>> level_nodes((size_t)max_level_ + 1);
  for (long long i = 0; i < n_; ++i)
    for (int l = 1; l <= levels_h_[i]; ++l) level_nodes[l].push_back((int)i);
  size_t max_upper_nodes = max_level_ >= 1 ? level_nodes[1].size() : 0;
  CU(nodes_d.alloc(std::max<size_t>(max_upper_nodes, 1)));

  BuildScratch S;
  S.st_ids = st_ids.get();
  S.st_dist = st_dist.get();
  S.pkeys = pkeys.get();
  S.pkeys_sorted = pkeys_sorted.get();
  S.pvals = pvals.get();
  S.pvals_sorted = pvals_sorted.get();
  S.sort_tmp = sort_tmp.get();
  S.sort_tmp_bytes = tmp_bytes;
  S.ticket = counters_.get() + 1;
  S.stats = stats_on_ ? counters_.get() + 4 : nullptr;

  long long batches = 0;
  for (int l = max_level_; l >= 0; --l) {
    const long long nl = l == 0 ? n_ : (long long)level_nodes[l].size();
    const long long upper_cnt = l < max_level_ ? (long long)level_nodes[l + 1].size() : 0;
    if (l > 0) {
      // the previous level's launches still read nodes_d
      CU(cudaStreamSynchronize(stream_));
      CU(cudaMemcpyAsync(nodes_d.get(), level_nodes[l].data(), (size_t)nl * sizeof(int), cudaMemcpyHostToDevice,
                         stream_));
    } else {
      CU(cudaStreamSynchronize(stream_));
    }
    BuildLevel L;
    L.g = View();
    L.level = l;
    L.rows = l == 0 ? rows0_.get() : rowsU_.get();
    L.dists = l == 0 ? dist0.get() : distU.get();
    L.distU = distU.get();
    L.stride = l == 0 ? stride0_ : strideU_;
    L.max_m = l == 0 ? opt_.max_m0 : opt_.max_m;
    L.levels = levels_d_.get();
    L.nodes = l == 0 ? nullptr : nodes_d.get();
    L.n_level = nl;
    L.went = went.get();
    L.ef_construction = opt_.ef_construction;
    L.heuristic_coef = (float)opt_.heuristic_coef;
    L.save_remains = opt_.save_remains ? 1 : 0;
    L.reverse_cand = opt_.reverse_cand ? 1 : 0;
    L.vsize = vsize;
    CU(launch_init_level(L, counters_.get() + 3, sm_count_, stream_));
    long long p = 0;
    while (p < nl) {
      long long b = (upper_cnt + p) / opt_.ramp_div;
      b = std::max<long long>(1, std::min(b, bmax));
      b = std::min(b, nl - p);
      CU(launch_build_batch(L, S, p, (int)b, sm_count_, stream_));
      p += b;
      ++batches;
    }
    Log(3, "level %d: %lld nodes queued", l, nl);
  }
  CU(cudaStreamSynchronize(stream_));
  has_graph_ = true;
  last_build_seconds_ = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  Log(2, "built %lld nodes, %d levels, %lld batches (max %lld) in %.3f s", n_, max_level_ + 1, batches, bmax,
      last_build_seconds_);
  return kOk;
}

int Engine::SearchGraphDevice(const float* d_q, long long nq, int topk, int ef, int* d_nns, float* d_dist,
                              int* d_found) {
  if (!has_graph_) return Fail(kBadState, "no graph: call build_graph() or load_index() first");
  if (nq < 0 || topk < 1) return Fail(kInvalidArgument, "need num_queries >= 0 and topk >= 1");
  if (nq == 0) return kOk;
  if (!d_q || !d_nns || !d_dist || !d_found) return Fail(kInvalidArgument, "null buffer");
  int rc = EnsureDevice();
  if (rc) return rc;
  ef = std::max(ef, topk);  // cuhnsw/pyhnsw.py:80
  if (ef > kMaxEf) return Fail(kUnsupported, "ef_search above 8192 is not supported");
  if (n_ == 0) {
    CU(cudaMemsetAsync(d_found, 0, (size_t)nq * sizeof(int), stream_));
    CU(launch_fill_i32(d_nns, nq * topk, -1, stream_));
    CU(launch_fill_i32(reinterpret_cast<int*>(d_dist), nq * topk, 0x7f800000, stream_));  // +inf
    return kOk;
  }
  int vsize = 0;
  if (ResolveVsize(ef, nq, &vsize) != kOk) return Fail(kUnsupported, "ef_search does not fit in shared memory");
  SearchParams p;
  p.g = View();
  p.queries = d_q;
  p.nq = nq;
  p.topk = topk;
  p.ef = ef;
  p.vsize = vsize;
  p.reverse_cand = opt_.reverse_cand ? 1 : 0;
  p.team = opt_.search_team;
  p.smem_per_warp = 0;
  p.labels = labelled_ ? labels_d_.get() : nullptr;
  p.out_ids = d_nns;
  p.out_dist = d_dist;
  p.out_found = d_found;
  SearchLane* lane = nullptr;
  if ((rc = LaneFor(stream_, &lane)) != kOk) return rc;
  p.ticket = lane->ticket.get();
  p.stats = stats_on_ ? counters_.get() + 4 : nullptr;
  SearchSchedule sched;
  // the launcher schedules only batches of more than one wave of its kernel (4 CTAs to 32 warps per SM);
  // below the smallest wave there is nothing to prepare
  const bool schedule = nq > (long long)sm_count_ * 4 && opt_.search_schedule;
  if (schedule && (rc = PrepareSchedule(nq, lane, &sched)) != kOk) return rc;
  CU(launch_search(p, sm_count_, stream_, schedule ? &sched : nullptr));
  return MarkLane(lane);
}

int Engine::LaneFor(cudaStream_t stream, SearchLane** out) {
  SearchLane* pick = nullptr;
  for (SearchLane& l : lanes_)
    if (l.used && l.stream == stream) pick = &l;
  if (!pick) {
    for (SearchLane& l : lanes_)
      if (!l.used && !pick) pick = &l;
    if (!pick) {
      pick = &lanes_[0];
      for (SearchLane& l : lanes_)
        if (l.stamp < pick->stamp) pick = &l;
      if (pick->pending) CU(cudaEventSynchronize(pick->done));  // its last search is over before another stream uses it
      pick->pending = false;
    }
    if (!pick->ticket.get()) CU(pick->ticket.alloc(1));
    if (!pick->done) CU(cudaEventCreateWithFlags(&pick->done, cudaEventDisableTiming));
    pick->stream = stream;
    pick->used = true;
  }
  pick->stamp = ++lane_clock_;
  *out = pick;
  return kOk;
}

int Engine::MarkLane(SearchLane* lane) {
  CU(cudaEventRecord(lane->done, stream_));
  lane->pending = true;
  return kOk;
}

int Engine::WaitForSearches() {
  for (SearchLane& l : lanes_)
    if (l.pending) {
      CU(cudaEventSynchronize(l.done));
      l.pending = false;
    }
  return kOk;
}

int Engine::PrepareSchedule(long long nq, SearchLane* lane, SearchSchedule* s) {
  if (nq > lane->capacity) {
    const long long cap = std::max<long long>(nq, 1024);
    CU(lane->sched.reserve((size_t)cap * 6));
    CU(lane->sched_tmp.reserve(search_schedule_tmp_bytes(cap)));
    lane->capacity = cap;
  }
  unsigned* base = lane->sched.get();
  const long long c = lane->capacity;
  s->capacity = c;
  s->entry_node = reinterpret_cast<int*>(base);
  s->entry_dist = reinterpret_cast<float*>(base + c);
  s->keys = base + 2 * c;
  s->keys_sorted = base + 3 * c;
  s->index = reinterpret_cast<int*>(base + 4 * c);
  s->order = reinterpret_cast<int*>(base + 5 * c);
  s->sort_tmp = lane->sched_tmp.get();
  s->sort_tmp_bytes = lane->sched_tmp.size();
  return kOk;
}

int Engine::SearchGraph(const float* q, long long nq, int topk, int ef, int* nns, float* dist, int* found) {
  int rc = SearchGraphAsync(q, nq, topk, ef, nns, dist, found);
  if (rc) return rc;
  CU(cudaStreamSynchronize(stream_));
  return kOk;
}

int Engine::SearchGraphAsync(const float* q, long long nq, int topk, int ef, int* nns, float* dist, int* found) {
  if (!has_graph_) return Fail(kBadState, "no graph: call build_graph() or load_index() first");
  if (nq < 0 || topk < 1) return Fail(kInvalidArgument, "need num_queries >= 0 and topk >= 1");
  if (nq == 0) return kOk;
  if (!q || !nns || !dist || !found) return Fail(kInvalidArgument, "null buffer");
  int rc = EnsureDevice();
  if (rc) return rc;
  // Page-locked host buffers have a device address: the kernels then read the queries and write the results
  // in place, over PCIe while they run, instead of a copy in before the first kernel and three copies out after
  // the last.  Every query is read once or twice and every result word written once, so nothing is lost.
  if (opt_.zero_copy) {
    auto mapped = [](const void* host, void** dev) {
      cudaPointerAttributes a;
      if (cudaPointerGetAttributes(&a, host) != cudaSuccess) {
        cudaGetLastError();
        return false;
      }
      *dev = a.devicePointer;
      return a.type == cudaMemoryTypeHost && a.devicePointer != nullptr;
    };
    void *dq = nullptr, *dn = nullptr, *dd = nullptr, *df = nullptr;
    if (mapped(q, &dq) && mapped(nns, &dn) && mapped(dist, &dd) && mapped(found, &df))
      return SearchGraphDevice(static_cast<const float*>(dq), nq, topk, ef, static_cast<int*>(dn),
                               static_cast<float*>(dd), static_cast<int*>(df));
  }
  SearchLane* lane = nullptr;
  if ((rc = LaneFor(stream_, &lane)) != kOk) return rc;
  CU(lane->q.reserve((size_t)nq * d_));
  CU(lane->ids.reserve((size_t)nq * topk));
  CU(lane->dist.reserve((size_t)nq * topk));
  CU(lane->found.reserve((size_t)nq));
  CU(cudaMemcpyAsync(lane->q.get(), q, (size_t)nq * d_ * sizeof(float), cudaMemcpyHostToDevice, stream_));
  rc = SearchGraphDevice(lane->q.get(), nq, topk, ef, lane->ids.get(), lane->dist.get(), lane->found.get());
  if (rc) return rc;
  CU(cudaMemcpyAsync(nns, lane->ids.get(), (size_t)nq * topk * sizeof(int), cudaMemcpyDeviceToHost, stream_));
  CU(cudaMemcpyAsync(dist, lane->dist.get(), (size_t)nq * topk * sizeof(float), cudaMemcpyDeviceToHost, stream_));
  CU(cudaMemcpyAsync(found, lane->found.get(), (size_t)nq * sizeof(int), cudaMemcpyDeviceToHost, stream_));
  return MarkLane(lane);  // the staging buffers are in use until the copies are through
}

int Engine::SearchGraphStatic(const float* q, long long nq, int topk, int ef, int* nns, float* dist, int* found) {
  if (!has_graph_) return Fail(kBadState, "no graph: call build_graph() or load_index() first");
  if (nq < 0 || topk < 1) return Fail(kInvalidArgument, "need num_queries >= 0 and topk >= 1");
  if (nq == 0) return kOk;
  if (!q || !nns || !dist || !found) return Fail(kInvalidArgument, "null buffer");
  int rc = EnsureDevice();
  if (rc) return rc;
  ef = std::max(ef, topk);
  if (ef > kMaxEf) return Fail(kUnsupported, "ef_search above 8192 is not supported");
  const size_t need = search_static_bytes(nq, d_, topk), cap = search_static_capacity();
  if (need > cap) {
    std::ostringstream os;
    os << "search without allocation: " << nq << " queries x " << d_ << " dims, topk " << topk << " need " << need
       << " bytes of fixed device scratch, the limit is " << cap << "; split the batch or use cuhnsw_search_knn";
    return Fail(kInvalidArgument, os.str());
  }
  if (n_ == 0) {
    for (long long i = 0; i < nq; ++i) found[i] = 0;
    for (long long i = 0; i < nq * topk; ++i) {
      nns[i] = -1;
      dist[i] = INFINITY;
    }
    return kOk;
  }
  int vsize = 0;
  if (ResolveVsize(ef, nq, &vsize) != kOk) return Fail(kUnsupported, "ef_search does not fit in shared memory");
  SearchParams p;
  p.g = View();
  p.queries = nullptr;
  p.nq = nq;
  p.topk = topk;
  p.ef = ef;
  p.vsize = vsize;
  p.reverse_cand = opt_.reverse_cand ? 1 : 0;
  p.team = opt_.search_team;
  p.smem_per_warp = 0;
  p.labels = labelled_ ? labels_d_.get() : nullptr;
  p.out_ids = nullptr;
  p.out_dist = nullptr;
  p.out_found = nullptr;
  p.ticket = nullptr;
  p.stats = nullptr;
  CU(search_static(p, q, nns, dist, found, sm_count_, stream_));
  return kOk;
}

int Engine::BatchDistance(const int* src, const int* dst, long long npairs, float* out) {
  if (!has_data_) return Fail(kBadState, "set_data() must be called first");
  if (npairs < 0 || (npairs > 0 && (!src || !dst || !out))) return Fail(kInvalidArgument, "bad pair list");
  for (long long i = 0; i < npairs; ++i)
    if (src[i] < 0 || src[i] >= n_ || dst[i] < 0 || dst[i] >= n_) return Fail(kInvalidArgument, "row id out of range");
  int rc = EnsureDevice();
  if (rc) return rc;
  if (npairs == 0) return kOk;
  DevBuf<int> s, t;
  DevBuf<float> o;
  CU(s.alloc((size_t)npairs));
  CU(t.alloc((size_t)npairs));
  CU(o.alloc((size_t)npairs));
  CU(cudaMemcpyAsync(s.get(), src, (size_t)npairs * sizeof(int), cudaMemcpyHostToDevice, stream_));
  CU(cudaMemcpyAsync(t.get(), dst, (size_t)npairs * sizeof(int), cudaMemcpyHostToDevice, stream_));
  GraphView g = View();
  CU(launch_batch_distance(g, s.get(), t.get(), npairs, o.get(), stream_));
  CU(cudaMemcpyAsync(out, o.get(), (size_t)npairs * sizeof(float), cudaMemcpyDeviceToHost, stream_));
  CU(cudaStreamSynchronize(stream_));
  return kOk;
}

int Engine::EnableStats(int on) {
  int rc = EnsureDevice();
  if (rc) return rc;
  stats_on_ = on != 0;
  CU(cudaMemsetAsync(counters_.get() + 4, 0, 4 * sizeof(unsigned long long), stream_));
  return kOk;
}

int Engine::GetStats(unsigned long long* out4) {
  int rc = EnsureDevice();
  if (rc) return rc;
  CU(cudaStreamSynchronize(stream_));
  CU(cudaMemcpy(out4, counters_.get() + 4, 4 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
  CU(cudaMemset(counters_.get() + 4, 0, 4 * sizeof(unsigned long long)));
  return kOk;
}

int Engine::Describe(long long* out8) {
  out8[0] = n_;
  out8[1] = d_;
  out8[2] = max_level_;
  out8[3] = enter_point_;
  out8[4] = opt_.max_m;
  out8[5] = opt_.max_m0;
  out8[6] = total_upper_;
  out8[7] = sm_count_;
  return kOk;
}

int Engine::GetGraph(int* levels, int* rows0, int* rows_upper) {
  if (!has_levels_ && !has_graph_) return Fail(kBadState, "no graph");
  int rc = EnsureDevice();
  if (rc) return rc;
  CU(cudaStreamSynchronize(stream_));
  if (levels) std::memcpy(levels, levels_h_.data(), (size_t)n_ * sizeof(int));
  if (rows0 && n_ > 0)
    CU(cudaMemcpy2D(rows0, (size_t)opt_.max_m0 * sizeof(int), rows0_.get(), (size_t)stride0_ * sizeof(int),
                    (size_t)opt_.max_m0 * sizeof(int), (size_t)n_, cudaMemcpyDeviceToHost));
  if (rows_upper && total_upper_ > 0)
    CU(cudaMemcpy2D(rows_upper, (size_t)opt_.max_m * sizeof(int), rowsU_.get(), (size_t)strideU_ * sizeof(int),
                    (size_t)opt_.max_m * sizeof(int), (size_t)total_upper_, cudaMemcpyDeviceToHost));
  return kOk;
}

// ---------------------------------------------------------------------------
// hnswlib-compatible file (layout: cpp/src/cuhnsw_base.cu:159-247 / 250-365)
// ---------------------------------------------------------------------------
int Engine::SaveIndex(const char* path) {
  if (!has_graph_) return Fail(kBadState, "no graph to save");
  if (!path) return Fail(kInvalidArgument, "null path");
  int rc = EnsureDevice();
  if (rc) return rc;
  CU(cudaStreamSynchronize(stream_));
  std::FILE* f = std::fopen(path, "wb");
  if (!f) return Fail(kIoError, std::string("cannot open ") + path + " for writing");
  // closes the file on every way out; a file that was not written to the end is removed
  struct Guard {
    std::FILE* f;
    const char* path;
    bool done = false;
    ~Guard() {
      if (f) std::fclose(f);
      if (!done) std::remove(path);
    }
  } guard{f, path};
  const int m = opt_.max_m, m0 = opt_.max_m0;
  const size_t rec = 4 + 4 * (size_t)m0 + 4 * (size_t)d_ + 8;
  FileHeader h;
  h.offset_level0 = 0;
  h.max_elements = (uint64_t)n_;
  h.cur_element_count = (uint64_t)n_;
  h.size_data_per_element = rec;
  h.label_offset = 4 + 4 * (size_t)m0 + 4 * (size_t)d_;
  h.offset_data = 4 + 4 * (size_t)m0;
  h.maxlevel = max_level_;
  h.enterpoint_node = (uint32_t)enter_point_;
  h.max_m = (uint64_t)m;
  h.max_m0 = (uint64_t)m0;
  h.m = (uint64_t)m;
  h.mult = opt_.level_mult;
  h.ef_construction = (uint64_t)opt_.ef_construction;
  bool ok = std::fwrite(&h, sizeof(h), 1, f) == 1;
  // Level-0 records are put together on the device, 32 MB at a time, exactly as they lie in the file: one
  // kernel packs the adjacency rows into degree word + neighbour slots and writes the labels, another moves
  // the vectors out of their padded (fp32 or 16-bit) rows; the host only writes the chunk out.  Labels of a
  // loaded index are 64-bit values the device does not hold: the host patches those in.
  const long long rec_words = (long long)(rec / 4);
  const long long chunk = std::max<long long>(1, (32ll << 20) / (long long)rec);
  const size_t chunk_rows = (size_t)std::min(chunk, std::max<long long>(n_, 1));
  DevBuf<unsigned> packed;
  CU(packed.alloc(chunk_rows * (size_t)rec_words));
  std::vector<unsigned char> out(chunk_rows * rec);
  for (long long s = 0; s < n_ && ok; s += chunk) {
    const long long r = std::min(chunk, n_ - s);
    CU(launch_pack_links(rows0_.get() + (size_t)s * stride0_, stride0_, r, s, m0, packed.get(), rec_words, stream_));
    CU(launch_unpad_rows(RowPtr(s), reinterpret_cast<float*>(packed.get()) + 1 + m0, rec_words, r, d_, vstride_,
                         rows16_, stream_));
    CU(cudaMemcpyAsync(out.data(), packed.get(), (size_t)r * rec, cudaMemcpyDeviceToHost, stream_));
    CU(cudaStreamSynchronize(stream_));
    if (labelled_)
      for (long long i = 0; i < r; ++i) {
        const uint64_t label = (uint64_t)labels_h_[(size_t)(s + i)];
        std::memcpy(out.data() + (size_t)(i + 1) * rec - 8, &label, 8);
      }
    ok = std::fwrite(out.data(), rec, (size_t)r, f) == (size_t)r;
  }
  // upper-layer link lists: a length word per node, then its rows; gathered into the same buffer and written
  // whenever it fills
  std::vector<int> upper((size_t)std::max<long long>(total_upper_, 1) * strideU_);
  if (total_upper_ > 0)
    CU(cudaMemcpy(upper.data(), rowsU_.get(), (size_t)total_upper_ * strideU_ * sizeof(int), cudaMemcpyDeviceToHost));
  const size_t per_link = 4 + 4 * (size_t)m;
  size_t fill = 0;
  auto flush = [&]() {
    if (fill && ok) ok = std::fwrite(out.data(), 1, fill, f) == fill;
    fill = 0;
  };
  out.resize(std::max<size_t>(out.size(), 4 + per_link * (size_t)(max_level_ + 1)));
  for (long long i = 0; i < n_ && ok; ++i) {
    const int lv = levels_h_[(size_t)i];
    const uint32_t nbytes = (uint32_t)(per_link * (size_t)lv);
    if (fill + 4 + nbytes > out.size()) flush();
    unsigned char* o = out.data() + fill;
    std::memcpy(o, &nbytes, 4);
    std::memset(o + 4, 0, nbytes);
    for (int l = 0; l < lv; ++l) {
      const int* row = upper.data() + ((size_t)upper_base_h_[(size_t)i] + l) * strideU_;
      unsigned char* ol = o + 4 + per_link * (size_t)l;
      uint32_t deg = 0;
      for (int j = 0; j < m; ++j)
        if (row[j] >= 0) {
          const uint32_t id = (uint32_t)row[j];
          std::memcpy(ol + 4 + 4 * (size_t)deg, &id, 4);
          ++deg;
        }
      std::memcpy(ol, &deg, 4);
    }
    fill += 4 + nbytes;
  }
  flush();
  guard.f = nullptr;
  ok = (std::fclose(f) == 0) && ok;
  if (!ok) return Fail(kIoError, std::string("short write to ") + path);
  guard.done = true;
  Log(3, "saved index to %s", path);
  return kOk;
}

int Engine::LoadIndex(const char* path) {
  if (!inited_) return Fail(kBadState, "init() must be called first");
  if (!path) return Fail(kInvalidArgument, "null path");
  std::FILE* f = std::fopen(path, "rb");
  if (!f) return Fail(kIoError, std::string("cannot open ") + path);
  struct Closer {
    std::FILE* f;
    ~Closer() { std::fclose(f); }
  } closer{f};
  std::fseek(f, 0, SEEK_END);
  const long long fsize = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  FileHeader h;
  if (fsize < (long long)sizeof(h) || std::fread(&h, sizeof(h), 1, f) != 1)
    return Fail(kIoError, "index file is shorter than its header");
  if (h.max_m0 < 1 || h.max_m0 > (uint64_t)kMaxLinksHost || h.max_m < 1 || h.max_m > h.max_m0)
    return Fail(kUnsupported, "index file: need 1 <= maxM <= maxM0 <= 64");
  if (h.offset_data != 4 + 4 * h.max_m0 || h.label_offset < h.offset_data || (h.label_offset - h.offset_data) % 4 ||
      h.size_data_per_element != h.label_offset + 8)
    return Fail(kParseError, "index file: inconsistent record layout");
  // sizes are checked by division, so that a crafted header cannot overflow the products
  if (h.size_data_per_element > (uint64_t)fsize || h.cur_element_count >= (1ull << 31) - 1)
    return Fail(kParseError, "index file: bad element count or dimension");
  const long long n = (long long)h.cur_element_count;
  const int d = (int)((h.label_offset - h.offset_data) / 4);
  const size_t rec = (size_t)h.size_data_per_element;
  if (d < 1) return Fail(kParseError, "index file: bad element count or dimension");
  if (n > (fsize - (long long)sizeof(h)) / (long long)rec) return Fail(kIoError, "index file: truncated level-0 block");
  if (n > 0 && (h.enterpoint_node >= (uint64_t)n || h.maxlevel < 0 || h.maxlevel > 64))
    return Fail(kParseError, "index file: bad enter point or level");
  const int m = (int)h.max_m, m0 = (int)h.max_m0;
  // options that the file overrides (cpp/src/cuhnsw_base.cu:279-285)
  opt_.max_m = m;
  opt_.max_m0 = m0;
  opt_.ef_construction = (int)std::min<uint64_t>(h.ef_construction, kMaxEf);
  opt_.level_mult = h.mult;

  // Level-0 block: a chunk of records goes to the device as it lies in the file and is taken apart
  // there (vectors into padded rows, neighbour slots into -1 padded adjacency rows, labels); the host
  // keeps only the 64-bit labels, which a later save_index writes back unchanged.
  int rc = AllocRows(n, d);
  if (rc) return rc;
  stride0_ = round_up(m0, 8);
  strideU_ = round_up(m, 8);
  CU(rows0_.alloc((size_t)std::max<long long>(n, 1) * stride0_));
  CU(labels_d_.alloc((size_t)std::max<long long>(n, 1)));
  std::vector<long long> labels((size_t)n);
  const long long rec_words = (long long)(rec / 4);
  {
    const long long chunk = std::max<long long>(1, (32ll << 20) / (long long)rec);
    const size_t rows_in_chunk = (size_t)std::min(chunk, std::max<long long>(n, 1));
    std::vector<unsigned char> buf(rows_in_chunk * rec);
    DevBuf<unsigned> raw;
    DevBuf<unsigned long long> bad;
    CU(raw.alloc(rows_in_chunk * (size_t)rec_words));
    CU(bad.alloc(1));
    CU(cudaMemsetAsync(bad.get(), 0xff, sizeof(unsigned long long), stream_));
    for (long long s = 0; s < n; s += chunk) {
      const long long r = std::min(chunk, n - s);
      if (std::fread(buf.data(), rec, (size_t)r, f) != (size_t)r) return Fail(kIoError, "index file: short read");
      CU(cudaMemcpyAsync(raw.get(), buf.data(), (size_t)r * rec, cudaMemcpyHostToDevice, stream_));
      CU(launch_unpack_links(raw.get(), rec_words, r, s, m0, n, rows0_.get() + (size_t)s * stride0_, stride0_,
                             labels_d_.get() + s, bad.get(), stream_));
      CU(launch_pad_rows(reinterpret_cast<const float*>(raw.get() + 1 + m0), rec_words, RowPtr(s), r, d, vstride_,
                         rows16_, stream_));
      for (long long i = 0; i < r; ++i) {
        uint64_t label;
        std::memcpy(&label, buf.data() + (size_t)(i + 1) * rec - 8, 8);
        labels[(size_t)(s + i)] = (long long)label;
      }
      CU(cudaStreamSynchronize(stream_));  // buf and raw are reused by the next chunk
    }
    unsigned long long first_bad = 0;
    CU(cudaMemcpy(&first_bad, bad.get(), sizeof(first_bad), cudaMemcpyDeviceToHost));
    if (first_bad != ~0ull) {
      std::ostringstream os;
      os << "index file: record " << (first_bad - 1)
         << " has a degree above maxM0, a neighbour id out of range or a neighbour listed twice";
      return Fail(kParseError, os.str());
    }
  }
  has_data_ = true;
  // Upper layers: per node a byte count and that many bytes of (degree, maxM slots) lists.  Only the
  // nodes above level 0 carry any (one in maxM0 or so), so their rows are collected on the host in
  // the flat layout and uploaded once.
  const size_t per_link = 4 + 4 * (size_t)m;
  levels_h_.assign((size_t)n, 0);
  std::vector<int> rowsU;
  std::vector<unsigned char> lbuf;
  for (long long i = 0; i < n; ++i) {
    uint32_t nbytes;
    if (std::fread(&nbytes, 4, 1, f) != 1) return Fail(kIoError, "index file: truncated link lists");
    if (nbytes % per_link || nbytes / per_link > 64) return Fail(kParseError, "index file: bad link list size");
    const int lv = (int)(nbytes / per_link);
    if (lv > h.maxlevel) return Fail(kParseError, "index file: a node lies above the file's top level");
    levels_h_[(size_t)i] = lv;
    if (!nbytes) continue;
    lbuf.resize(nbytes);
    if (std::fread(lbuf.data(), 1, nbytes, f) != nbytes) return Fail(kIoError, "index file: truncated link lists");
    for (int l = 0; l < lv; ++l) {
      const unsigned char* o = lbuf.data() + per_link * (size_t)l;
      uint32_t deg;
      std::memcpy(&deg, o, 4);
      deg &= 0xffffu;
      if (deg > (uint32_t)m) return Fail(kParseError, "index file: degree above maxM");
      const size_t at = rowsU.size();
      rowsU.resize(at + (size_t)strideU_, -1);
      for (uint32_t j = 0; j < deg; ++j) {
        uint32_t id;
        std::memcpy(&id, o + 4 + 4 * (size_t)j, 4);
        if (id >= (uint64_t)n) return Fail(kParseError, "index file: bad upper-layer neighbour");
        for (uint32_t k = 0; k < j; ++k)
          if (rowsU[at + k] == (int)id) return Fail(kParseError, "index file: upper-layer neighbour listed twice");
        rowsU[at + j] = (int)id;
      }
    }
  }
  max_level_ = h.maxlevel;
  enter_point_ = n > 0 ? (int)h.enterpoint_node : 0;
  if (n > 0 && levels_h_[(size_t)enter_point_] < max_level_)
    return Fail(kParseError, "index file: enter point does not reach the top level");
  // a neighbour on layer l must itself reach layer l (its row there is read during the descent)
  {
    size_t at = 0;
    for (long long i = 0; i < n; ++i)
      for (int l = 1; l <= levels_h_[(size_t)i]; ++l, at += (size_t)strideU_)
        for (int j = 0; j < m && rowsU[at + j] >= 0; ++j)
          if (levels_h_[(size_t)rowsU[at + j]] < l) return Fail(kParseError, "index file: bad upper-layer neighbour");
  }
  upper_base_h_.assign((size_t)n, 0);
  long long acc = 0;
  for (long long i = 0; i < n; ++i) {
    upper_base_h_[(size_t)i] = (int)acc;
    acc += levels_h_[(size_t)i];
    if (acc > (1ll << 30)) return Fail(kUnsupported, "too many upper-layer rows");
  }
  total_upper_ = acc;
  CU(rowsU_.alloc((size_t)std::max<long long>(total_upper_, 1) * strideU_));
  CU(levels_d_.alloc((size_t)std::max<long long>(n, 1)));
  CU(upper_base_d_.alloc((size_t)std::max<long long>(n, 1)));
  if (total_upper_ > 0)
    CU(cudaMemcpy(rowsU_.get(), rowsU.data(), (size_t)total_upper_ * strideU_ * sizeof(int), cudaMemcpyHostToDevice));
  else
    CU(launch_fill_i32(rowsU_.get(), strideU_, -1, stream_));
  if (n > 0) {
    CU(cudaMemcpy(levels_d_.get(), levels_h_.data(), (size_t)n * sizeof(int), cudaMemcpyHostToDevice));
    CU(cudaMemcpy(upper_base_d_.get(), upper_base_h_.data(), (size_t)n * sizeof(int), cudaMemcpyHostToDevice));
  }
  CU(cudaStreamSynchronize(stream_));
  labels_h_.swap(labels);
  labelled_ = true;
  has_levels_ = true;
  has_graph_ = true;
  Log(3, "loaded %s: num_data %lld, num_dims %d, max_m %d, max_m0 %d, enter_point %d, max_level %d", path, n_, d_, m,
      m0, enter_point_, max_level_);
  return kOk;
}

// Replica of another engine's index on this engine's GPU: same rows, graph and labels, copied device to
// device.  The two engines must have been initialised from the same options.
int Engine::CloneFrom(const Engine& src) {
  if (!inited_) return Fail(kBadState, "init() must be called first");
  if (!src.has_graph_) return Fail(kBadState, "nothing to replicate: the source has no graph");
  opt_.max_m = src.opt_.max_m;
  opt_.max_m0 = src.opt_.max_m0;
  opt_.ef_construction = src.opt_.ef_construction;
  opt_.level_mult = src.opt_.level_mult;
  int rc = AllocRows(src.n_, src.d_);
  if (rc) return rc;
  if (rows16_ != src.rows16_) return Fail(kBadState, "replica and source store rows in different types");
  stride0_ = src.stride0_;
  strideU_ = src.strideU_;
  max_level_ = src.max_level_;
  enter_point_ = src.enter_point_;
  total_upper_ = src.total_upper_;
  levels_h_ = src.levels_h_;
  upper_base_h_ = src.upper_base_h_;
  labels_h_ = src.labels_h_;
  auto copy = [&](void* dst, const void* from, size_t bytes) {
    return bytes ? cudaMemcpyPeer(dst, device_, from, src.device_, bytes) : cudaSuccess;
  };
  const size_t one = (size_t)std::max<long long>(n_, 1);
  CU(rows0_.alloc(one * stride0_));
  CU(rowsU_.alloc((size_t)std::max<long long>(total_upper_, 1) * strideU_));
  CU(levels_d_.alloc(one));
  CU(upper_base_d_.alloc(one));
  CU(copy(vec_.get(), src.vec_.get(), vec_.size() * sizeof(float)));
  CU(copy(rows0_.get(), src.rows0_.get(), rows0_.size() * sizeof(int)));
  CU(copy(rowsU_.get(), src.rowsU_.get(), rowsU_.size() * sizeof(int)));
  CU(copy(levels_d_.get(), src.levels_d_.get(), levels_d_.size() * sizeof(int)));
  CU(copy(upper_base_d_.get(), src.upper_base_d_.get(), upper_base_d_.size() * sizeof(int)));
  if (src.labelled_) {
    CU(labels_d_.alloc(one));
    CU(copy(labels_d_.get(), src.labels_d_.get(), labels_d_.size() * sizeof(int)));
  }
  CU(cudaDeviceSynchronize());
  labelled_ = src.labelled_;
  has_data_ = has_levels_ = has_graph_ = true;
  return kOk;
}

}  // namespace hnsw
