// One handle, several GPUs: a replica of the index on every GPU listed in the option `devices`, and
// host-buffer searches split over them.
//
// The reference is single-device by construction (it takes the current device once,
// cpp/src/cuhnsw_build.cu:15-23, and lists multi-device support as an open task).  Queries are independent
// units of work, so the split needs no collective: the batch is cut into contiguous slices, one per GPU,
// each slice is searched by that GPU's replica on a host thread of its own, and the slices land in the
// caller's output arrays side by side.  The result equals the single-GPU result row for row.
//
// The graph is built (or loaded) once, on the first GPU of the list, and copied to the others device to
// device: the build's shared mutable state does not partition.
#pragma once
#include <condition_variable>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "engine.h"

namespace hnsw {

// A host thread that runs one task at a time.  wait() returns when the task has ended; a task never
// blocks on another worker, so wait() cannot hang on anything but the task itself.
class Worker {
 public:
  Worker() : thread_([this] { Loop(); }) {}
  ~Worker() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      quit_ = true;
    }
    cv_.notify_all();
    thread_.join();
  }
  void Submit(std::function<void()> task) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      task_ = std::move(task);
      busy_ = true;
    }
    cv_.notify_all();
  }
  void Wait() {
    std::unique_lock<std::mutex> lock(mu_);
    cv_.wait(lock, [this] { return !busy_; });
  }

 private:
  void Loop() {
    std::unique_lock<std::mutex> lock(mu_);
    for (;;) {
      cv_.wait(lock, [this] { return quit_ || busy_; });
      if (quit_) return;
      std::function<void()> task = std::move(task_);
      lock.unlock();
      try {
        task();
      } catch (...) {
        // tasks report through their own status slot; nothing may escape a thread
      }
      lock.lock();
      busy_ = false;
      cv_.notify_all();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::function<void()> task_;
  bool busy_ = false, quit_ = false;
  std::thread thread_;  // declared last: it starts in the constructor and uses the members above
};

class ReplicaSet {
 public:
  // Reads `devices` from the primary's options; with two or more entries creates one more engine per
  // further GPU from the same option file.  Call after a successful Init of the primary.
  int Configure(const Engine& primary, const char* opt_path, std::string* err) {
    extra_.clear();
    workers_.clear();
    stale_ = true;
    const std::vector<int>& devs = primary.options().devices;
    for (size_t i = 1; i < devs.size(); ++i) {
      auto e = std::make_unique<Engine>();
      const int rc = e->Init(opt_path, devs[i]);
      if (rc != kOk) {
        *err = "device " + std::to_string(devs[i]) + ": " + e->last_error();
        extra_.clear();
        return rc;
      }
      extra_.push_back(std::move(e));
    }
    for (size_t i = 0; i < extra_.size(); ++i) workers_.push_back(std::make_unique<Worker>());
    return kOk;
  }
  bool active() const { return !extra_.empty(); }
  int count() const { return 1 + (int)extra_.size(); }
  // Replica `index` (0 = the primary) with an up-to-date copy of the index, or nullptr with *rc and *err set.
  Engine* Fresh(Engine& primary, int index, int* rc, std::string* err) {
    *rc = kOk;
    if (index < 0 || index >= count()) {
      *rc = kInvalidArgument;
      *err = "no replica " + std::to_string(index) + ": the handle has " + std::to_string(count());
      return nullptr;
    }
    if (index == 0) return &primary;
    if (stale_ && (*rc = Sync(primary, err)) != kOk) return nullptr;
    return extra_[(size_t)index - 1].get();
  }
  // the primary's index changed (set_data, build_graph, load_index): replicas are copied again before the next search
  void Invalidate() { stale_ = true; }

  // Copies the primary's index to every other GPU (all copies run at the same time).
  int Sync(const Engine& primary, std::string* err) {
    std::vector<int> rc(extra_.size(), kOk);
    for (size_t i = 0; i < extra_.size(); ++i)
      workers_[i]->Submit([&, i] { rc[i] = extra_[i]->CloneFrom(primary); });
    for (auto& w : workers_) w->Wait();
    for (size_t i = 0; i < extra_.size(); ++i)
      if (rc[i] != kOk) {
        *err = "replica on device " + std::to_string(primary.options().devices[i + 1]) + ": " + extra_[i]->last_error();
        return rc[i];
      }
    stale_ = false;
    return kOk;
  }

  // Contiguous, balanced slices: GPU g of G gets queries [g*q/G + min(g, q%G), ...).
  static void Slice(long long total, int parts, int part, long long* lo, long long* hi) {
    const long long base = total / parts, rem = total % parts;
    *lo = part * base + (part < rem ? part : rem);
    *hi = *lo + base + (part < rem ? 1 : 0);
  }

  // Host buffers in and out, like Engine::SearchGraph.  The caller's thread searches the first slice on the
  // primary; every worker's status is collected before returning, so a failure on one GPU comes back as
  // an error code with that GPU's message, after all the others have finished.
  int Search(Engine& primary, const float* q, long long nq, int topk, int ef, int* nns, float* dist, int* found,
             std::string* err) {
    if (stale_) {
      const int rc = Sync(primary, err);
      if (rc != kOk) return rc;
    }
    const int parts = 1 + (int)extra_.size();
    const int d = primary.num_dims();
    std::vector<int> rc(extra_.size(), kOk);
    for (size_t i = 0; i < extra_.size(); ++i) {
      long long lo, hi;
      Slice(nq, parts, (int)i + 1, &lo, &hi);
      workers_[i]->Submit([&, i, lo, hi] {
        rc[i] = hi > lo ? extra_[i]->SearchGraph(q + (size_t)lo * d, hi - lo, topk, ef, nns + (size_t)lo * topk,
                                                 dist + (size_t)lo * topk, found + lo)
                        : kOk;
      });
    }
    long long lo, hi;
    Slice(nq, parts, 0, &lo, &hi);
    int first = hi > lo || nq == 0 ? primary.SearchGraph(q, hi - lo, topk, ef, nns, dist, found) : kOk;
    for (auto& w : workers_) w->Wait();
    if (first != kOk) {
      *err = primary.last_error();
      return first;
    }
    for (size_t i = 0; i < extra_.size(); ++i)
      if (rc[i] != kOk) {
        *err = "device " + std::to_string(primary.options().devices[i + 1]) + ": " + extra_[i]->last_error();
        return rc[i];
      }
    return kOk;
  }

 private:
  std::vector<std::unique_ptr<Engine>> extra_;
  std::vector<std::unique_ptr<Worker>> workers_;
  bool stale_ = true;
};

}  // namespace hnsw
