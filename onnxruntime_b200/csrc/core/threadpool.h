// A small fixed-size thread pool: the host-side concurrency of the runtime.
//
// Two uses, as in the reference (include/onnxruntime/core/platform/threadpool.h:144-285,
// onnxruntime/core/common/threadpool.cc): the session's inter-op pool runs independent nodes of a graph at the same
// time (ExecutionMode::ORT_PARALLEL), and ParallelFor splits one loop over the workers.  The pool is deliberately
// plain: one locked deque, workers that sleep on a condition variable, and a caller that helps drain the queue while it
// waits, so a ParallelFor issued from inside a worker cannot dead-lock.  Intra-op math of the CPU kernels stays with
// ATen's own pool, whose size the session sets from intra_op_num_threads.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <string>
#include <mutex>
#include <thread>
#include <vector>

namespace ortb {

class ThreadPool {
 public:
  // `threads` workers are started; 0 means every task runs in the calling thread
  explicit ThreadPool(int threads, const std::string& name = "ortb200");
  ~ThreadPool();
  ThreadPool(const ThreadPool&) = delete;
  ThreadPool& operator=(const ThreadPool&) = delete;

  int NumThreads() const { return static_cast<int>(workers_.size()); }
  // Queue one task.  With no workers it runs before Schedule returns.
  void Schedule(std::function<void()> fn);
  // fn(begin, end) over [0, total) in blocks of at least `min_block`; returns when every block is done.  The first
  // exception thrown by a block is re-thrown here.
  void ParallelFor(int64_t total, int64_t min_block, const std::function<void(int64_t, int64_t)>& fn);
  // Runs queued tasks in the calling thread until `done` returns true (used by waiters so that they do useful work).
  void HelpUntil(const std::function<bool()>& done);
  // tasks executed so far, per worker index (workers 0..n-1, callers that helped are counted at index n)
  std::vector<int64_t> TaskCounts() const;

 private:
  void WorkerLoop(int index);
  bool RunOne(int index);

  std::vector<std::thread> workers_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::function<void()>> queue_;
  std::vector<int64_t> counts_;
  bool stop_ = false;
};

}  // namespace ortb
