// A small process-wide pool of host threads for the host half of the pipeline-gather schedule
// (the reference takes these from the execution context's thread pool,
// cuda_ops/pipeline_gather.cuh:188-262).  One parallel_for runs at a time; the calling thread works
// alongside the pool.  Size: NVE_B200_HOST_WORKERS, else the hardware concurrency, at most 32.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <exception>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace nve_b200 {

class HostWorkers {
 public:
  static HostWorkers& instance() {
    static HostWorkers pool;
    return pool;
  }

  // Threads that work on a parallel_for, the caller included.
  int size() const { return static_cast<int>(threads_.size()) + 1; }

  // Runs fn(0) .. fn(tasks - 1), each exactly once, and returns when all are done.  The first
  // exception a task throws is rethrown here after the others have finished.
  void parallel_for(int64_t tasks, const std::function<void(int64_t)>& fn) {
    if (tasks <= 0) return;
    std::lock_guard<std::mutex> one_job(job_mu_);
    {
      std::lock_guard<std::mutex> lock(mu_);
      fn_ = &fn;
      tasks_ = tasks;
      next_.store(0);
      busy_ = static_cast<int>(threads_.size());
      error_ = nullptr;
      generation_++;
    }
    wake_.notify_all();
    drain();
    std::unique_lock<std::mutex> lock(mu_);
    idle_.wait(lock, [&] { return busy_ == 0; });
    fn_ = nullptr;
    if (error_) std::rethrow_exception(error_);
  }

  HostWorkers(const HostWorkers&) = delete;
  HostWorkers& operator=(const HostWorkers&) = delete;

 private:
  HostWorkers() {
    int n = static_cast<int>(std::thread::hardware_concurrency());
    if (const char* env = std::getenv("NVE_B200_HOST_WORKERS")) n = std::atoi(env);
    if (n < 1) n = 1;
    if (n > 32) n = 32;
    for (int i = 0; i + 1 < n; i++) threads_.emplace_back([this] { loop(); });
  }

  ~HostWorkers() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      stop_ = true;
    }
    wake_.notify_all();
    for (auto& t : threads_) t.join();
  }

  void drain() {
    for (;;) {
      const int64_t t = next_.fetch_add(1);
      if (t >= tasks_) return;
      try {
        (*fn_)(t);
      } catch (...) {
        std::lock_guard<std::mutex> lock(mu_);
        if (!error_) error_ = std::current_exception();
      }
    }
  }

  void loop() {
    uint64_t seen = 0;
    for (;;) {
      {
        std::unique_lock<std::mutex> lock(mu_);
        wake_.wait(lock, [&] { return stop_ || generation_ != seen; });
        if (stop_) return;
        seen = generation_;
      }
      drain();
      {
        std::lock_guard<std::mutex> lock(mu_);
        busy_--;
      }
      idle_.notify_all();
    }
  }

  std::vector<std::thread> threads_;
  std::mutex job_mu_;
  std::mutex mu_;
  std::condition_variable wake_, idle_;
  const std::function<void(int64_t)>* fn_ = nullptr;
  int64_t tasks_ = 0;
  std::atomic<int64_t> next_{0};
  int busy_ = 0;
  uint64_t generation_ = 0;
  bool stop_ = false;
  std::exception_ptr error_;
};

}  // namespace nve_b200
