// Single-queue worker pool behind async_preprocess / async_push_pull: tasks run in submission order
// on `n` threads (the table uses n = 1, so asynchronous calls keep program order).
// Same role as the reference's ThreadPool (csrc/utils/thread_pool.h:16-50).
#pragma once
#include <condition_variable>
#include <deque>
#include <functional>
#include <future>
#include <mutex>
#include <thread>
#include <vector>

namespace hetuCTR {

class ThreadPool {
 public:
  explicit ThreadPool(size_t n) {
    for (size_t i = 0; i < n; i++) workers_.emplace_back([this] { run(); });
  }
  ~ThreadPool() {
    {
      std::lock_guard<std::mutex> g(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto &t : workers_) t.join();
  }
  std::future<void> Enqueue(std::function<void()> fn) {
    std::packaged_task<void()> task(std::move(fn));
    std::future<void> f = task.get_future();
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stop_) throw std::runtime_error("enqueue on stopped ThreadPool");
      queue_.emplace_back(std::move(task));
    }
    cv_.notify_one();
    return f;
  }

 private:
  void run() {
    for (;;) {
      std::packaged_task<void()> task;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [this] { return stop_ || !queue_.empty(); });
        if (queue_.empty()) return;
        task = std::move(queue_.front());
        queue_.pop_front();
      }
      task();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::packaged_task<void()>> queue_;
  std::vector<std::thread> workers_;
  bool stop_ = false;
};

}  // namespace hetuCTR
