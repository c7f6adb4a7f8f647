// Thread and synchronisation primitives of the native runtime.
//
// Capability parity with the reference's L0 thread utilities:
//   Semaphore      tips/core/common/semaphore.h:11-29   (EINTR-safe counting semaphore)
//   RWLock+guards  tips/core/common/rwlock.h:8-43
//   ManagedThread  tips/core/common/managed_thread.h:11-64  (persistent thread, Start/Join)
//   ThreadGroup    tips/core/common/thread_group.h:15-107   (N workers + barrier + ParallelRunRange)
//   ThreadPool     tips/core/common/thread_pool.h:9-61      (task queue; the reference's
//                  version never sets its parallelism, this one does)
// Implemented on the C++17 standard library only.
#pragma once

#include <atomic>
#include <condition_variable>
#include <functional>
#include <future>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <thread>
#include <vector>

#include "core/channel.h"
#include "core/logging.h"

namespace tips {

class Semaphore {
 public:
  explicit Semaphore(int initial = 0) : count_(initial) {}
  TIPS_DISALLOW_COPY_AND_ASSIGN(Semaphore);

  void Post(int n = 1) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      count_ += n;
    }
    if (n == 1)
      cv_.notify_one();
    else
      cv_.notify_all();
  }

  void Wait() {
    std::unique_lock<std::mutex> lock(mu_);
    cv_.wait(lock, [&] { return count_ > 0; });
    --count_;
  }

  bool TryWait() {
    std::lock_guard<std::mutex> lock(mu_);
    if (count_ <= 0) return false;
    --count_;
    return true;
  }

  bool WaitFor(int64_t timeout_ms) {
    std::unique_lock<std::mutex> lock(mu_);
    if (!cv_.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return count_ > 0; })) return false;
    --count_;
    return true;
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  int count_;
};

class RWLock {
 public:
  void LockRead() { mu_.lock_shared(); }
  void UnlockRead() { mu_.unlock_shared(); }
  void LockWrite() { mu_.lock(); }
  void UnlockWrite() { mu_.unlock(); }

 private:
  std::shared_mutex mu_;
};

class RWLockReadGuard {
 public:
  explicit RWLockReadGuard(RWLock& lock) : lock_(lock) { lock_.LockRead(); }
  ~RWLockReadGuard() { lock_.UnlockRead(); }
  TIPS_DISALLOW_COPY_AND_ASSIGN(RWLockReadGuard);

 private:
  RWLock& lock_;
};

class RWLockWriteGuard {
 public:
  explicit RWLockWriteGuard(RWLock& lock) : lock_(lock) { lock_.LockWrite(); }
  ~RWLockWriteGuard() { lock_.UnlockWrite(); }
  TIPS_DISALLOW_COPY_AND_ASSIGN(RWLockWriteGuard);

 private:
  RWLock& lock_;
};

// Reusable barrier for a fixed number of participants.
class Barrier {
 public:
  explicit Barrier(int n = 1) : n_(n) {}
  void Reset(int n) {
    std::lock_guard<std::mutex> lock(mu_);
    n_       = n;
    waiting_ = 0;
  }
  void Wait() {
    std::unique_lock<std::mutex> lock(mu_);
    uint64_t gen = generation_;
    if (++waiting_ == n_) {
      waiting_ = 0;
      ++generation_;
      lock.unlock();
      cv_.notify_all();
      return;
    }
    cv_.wait(lock, [&] { return generation_ != gen; });
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  int n_;
  int waiting_{0};
  uint64_t generation_{0};
};

// A persistent OS thread that runs one task at a time: Start(task) hands the
// task over, Join() waits for that task to finish; the thread itself lives
// until the object is destroyed.
class alignas(64) ManagedThread {
 public:
  ManagedThread();
  ~ManagedThread();
  TIPS_DISALLOW_COPY_AND_ASSIGN(ManagedThread);

  bool active() const { return active_.load(); }
  void Start(std::function<void()> task);
  void Join();

 private:
  void Loop();

  std::function<void()> task_;
  Semaphore start_sem_;
  Semaphore finish_sem_;
  std::atomic<bool> active_{false};
  std::atomic<bool> terminate_{false};
  std::thread thread_;
};

// N managed threads that run the same function together and can synchronise on
// a group barrier; thread_id() gives the index of the calling worker.
class ThreadGroup {
 public:
  explicit ThreadGroup(int num_threads = 0);
  ~ThreadGroup();
  TIPS_DISALLOW_COPY_AND_ASSIGN(ThreadGroup);

  void SetThreadNum(int num_threads);
  int parallel_num() const { return static_cast<int>(threads_.size()); }

  // Run `func(thread_id)` on every worker and wait for all of them.
  void Run(const std::function<void(int)>& func);
  void Start(const std::function<void(int)>& func);
  void Join();

  // Barrier across the workers of the group; call from inside `func`.
  void BarrierWait() { barrier_.Wait(); }

  // Index of the calling thread inside its group, -1 outside.
  static int thread_id();

 private:
  std::vector<std::unique_ptr<ManagedThread>> threads_;
  Barrier barrier_;
  bool running_{false};
};

// Splits [0, n) into parallel_num contiguous ranges and calls
// func(thread_id, begin, end) on each worker.
void ParallelRunRange(ThreadGroup& group, size_t n, const std::function<void(int, size_t, size_t)>& func);

// Task-queue thread pool with futures.
class ThreadPool {
 public:
  explicit ThreadPool(int num_threads);
  ~ThreadPool();
  TIPS_DISALLOW_COPY_AND_ASSIGN(ThreadPool);

  int parallel_num() const { return static_cast<int>(workers_.size()); }

  template <typename F>
  auto Submit(F&& f) -> std::future<decltype(f())> {
    using R   = decltype(f());
    auto task = std::make_shared<std::packaged_task<R()>>(std::forward<F>(f));
    std::future<R> fut = task->get_future();
    bool ok            = tasks_.WriteMove([task] { (*task)(); });
    TIPS_CHECK(ok) << "ThreadPool is shut down";
    return fut;
  }

  void Shutdown();

 private:
  Channel<std::function<void()>> tasks_;
  std::vector<std::thread> workers_;
};

}  // namespace tips
