// Fixed-size worker pool returning futures; what Prefetch and OrderedPrefetch
// run their look-ahead on (role of mlx/data/core/ThreadPool.h:21-115).
// An exception thrown by a task is delivered by future::get().
#pragma once

#include <condition_variable>
#include <functional>
#include <future>
#include <mutex>
#include <queue>
#include <thread>
#include <vector>

namespace mlx {
namespace data {
namespace core {

class ThreadPool {
 public:
  explicit ThreadPool(size_t threads) {
    if (threads == 0) {
      threads = 1;
    }
    for (size_t i = 0; i < threads; i++) {
      workers_.emplace_back([this] { run(); });
    }
  }

  template <class F>
  auto enqueue(F&& f) -> std::future<decltype(f())> {
    using R = decltype(f());
    auto task = std::make_shared<std::packaged_task<R()>>(std::forward<F>(f));
    std::future<R> fut = task->get_future();
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stopping_) {
        throw std::runtime_error("ThreadPool: enqueue on a stopped pool");
      }
      tasks_.emplace([task] { (*task)(); });
    }
    cv_.notify_one();
    return fut;
  }

  ~ThreadPool() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stopping_ = true;
    }
    cv_.notify_all();
    for (auto& w : workers_) {
      w.join();
    }
  }

 private:
  void run() {
    for (;;) {
      std::function<void()> job;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stopping_ || !tasks_.empty(); });
        if (tasks_.empty()) {
          return;  // stopping and drained
        }
        job = std::move(tasks_.front());
        tasks_.pop();
      }
      job();
    }
  }

  std::vector<std::thread> workers_;
  std::queue<std::function<void()>> tasks_;
  std::mutex mu_;
  std::condition_variable cv_;
  bool stopping_ = false;
};

} // namespace core
} // namespace data
} // namespace mlx
