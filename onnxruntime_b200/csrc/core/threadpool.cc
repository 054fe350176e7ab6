#include "threadpool.h"

#include <exception>
#include <string>

namespace ortb {

ThreadPool::ThreadPool(int threads, const std::string& /*name*/) {
  if (threads < 0) threads = 0;
  counts_.assign(static_cast<size_t>(threads) + 1, 0);
  workers_.reserve(static_cast<size_t>(threads));
  for (int i = 0; i < threads; ++i) workers_.emplace_back([this, i] { WorkerLoop(i); });
}

ThreadPool::~ThreadPool() {
  {
    std::lock_guard<std::mutex> lk(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  for (auto& t : workers_)
    if (t.joinable()) t.join();
}

void ThreadPool::Schedule(std::function<void()> fn) {
  if (workers_.empty()) {
    fn();
    std::lock_guard<std::mutex> lk(mu_);
    ++counts_.back();
    return;
  }
  {
    std::lock_guard<std::mutex> lk(mu_);
    queue_.push_back(std::move(fn));
  }
  cv_.notify_one();
}

bool ThreadPool::RunOne(int index) {
  std::function<void()> fn;
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (queue_.empty()) return false;
    fn = std::move(queue_.front());
    queue_.pop_front();
    ++counts_[static_cast<size_t>(index)];
  }
  fn();
  return true;
}

void ThreadPool::WorkerLoop(int index) {
  for (;;) {
    std::function<void()> fn;
    {
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [this] { return stop_ || !queue_.empty(); });
      if (queue_.empty()) return;  // stop_ and nothing left to do
      fn = std::move(queue_.front());
      queue_.pop_front();
      ++counts_[static_cast<size_t>(index)];
    }
    fn();
  }
}

void ThreadPool::HelpUntil(const std::function<bool()>& done) {
  const int helper = static_cast<int>(workers_.size());
  while (!done()) {
    if (!RunOne(helper)) std::this_thread::yield();
  }
}

void ThreadPool::ParallelFor(int64_t total, int64_t min_block, const std::function<void(int64_t, int64_t)>& fn) {
  if (total <= 0) return;
  if (min_block < 1) min_block = 1;
  const int64_t lanes = static_cast<int64_t>(workers_.size()) + 1;
  int64_t blocks = (total + min_block - 1) / min_block;
  if (blocks > lanes) blocks = lanes;
  if (blocks <= 1) {
    fn(0, total);
    return;
  }
  const int64_t per = (total + blocks - 1) / blocks;
  std::atomic<int64_t> remaining{blocks};
  std::exception_ptr first_error;
  std::mutex err_mu;
  auto run_block = [&](int64_t b) {
    const int64_t lo = b * per, hi = lo + per < total ? lo + per : total;
    try {
      if (lo < hi) fn(lo, hi);
    } catch (...) {
      std::lock_guard<std::mutex> lk(err_mu);
      if (!first_error) first_error = std::current_exception();
    }
    remaining.fetch_sub(1, std::memory_order_acq_rel);
  };
  for (int64_t b = 1; b < blocks; ++b) Schedule([&run_block, b] { run_block(b); });
  run_block(0);
  HelpUntil([&] { return remaining.load(std::memory_order_acquire) == 0; });
  if (first_error) std::rethrow_exception(first_error);
}

std::vector<int64_t> ThreadPool::TaskCounts() const {
  std::lock_guard<std::mutex> lk(mu_);
  return counts_;
}

}  // namespace ortb
