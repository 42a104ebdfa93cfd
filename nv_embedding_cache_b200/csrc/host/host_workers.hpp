// Pools of host threads for the host half of the pipeline-gather schedule (the reference takes
// these from the execution context's thread pool, cuda_ops/pipeline_gather.cuh:188-262).  One
// parallel_for runs at a time per pool; the calling thread works alongside the pool's threads.
// The process-wide default pool has NVE_B200_HOST_WORKERS threads, else what
// nve_configure_default_thread_pool asked for, else the hardware concurrency, at most 32; a pool
// made through nve_thread_pool_create has the number of workers its configuration names and is used
// by the execution contexts created with it.
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
    static HostWorkers pool(default_size(/*lock=*/true));
    return pool;
  }

  // `workers` threads besides the caller of parallel_for.
  explicit HostWorkers(int workers) {
    for (int i = 0; i < workers; i++) threads_.emplace_back([this] { loop(); });
  }

  // Size of the default pool.  configure_default() may change it until the pool exists.
  static bool configure_default(int workers) {
    std::lock_guard<std::mutex> lock(config_mu());
    if (default_locked()) return false;
    configured_workers() = workers;
    return true;
  }

  // Worker threads of this pool (the reference's num_workers).
  int workers() const { return static_cast<int>(threads_.size()); }

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

  ~HostWorkers() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      stop_ = true;
    }
    wake_.notify_all();
    for (auto& t : threads_) t.join();
  }

 private:
  static std::mutex& config_mu() {
    static std::mutex m;
    return m;
  }
  static int& configured_workers() {
    static int n = -1;
    return n;
  }
  static bool& default_locked() {
    static bool locked = false;
    return locked;
  }
  // threads of the default pool besides the caller
  static int default_size(bool lock) {
    std::lock_guard<std::mutex> guard(config_mu());
    if (lock) default_locked() = true;
    int n = static_cast<int>(std::thread::hardware_concurrency());
    if (configured_workers() >= 0) n = configured_workers() + 1;
    if (const char* env = std::getenv("NVE_B200_HOST_WORKERS")) n = std::atoi(env);
    if (n < 1) n = 1;
    if (n > 32) n = 32;
    return n - 1;
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
