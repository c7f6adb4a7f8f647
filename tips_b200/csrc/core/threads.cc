#include "core/threads.h"

namespace tips {

ManagedThread::ManagedThread() : thread_([this] { Loop(); }) {}

ManagedThread::~ManagedThread() {
  if (active_.load()) Join();
  terminate_ = true;
  start_sem_.Post();
  if (thread_.joinable()) thread_.join();
}

void ManagedThread::Start(std::function<void()> task) {
  TIPS_CHECK(!active_.load()) << "ManagedThread already runs a task";
  task_   = std::move(task);
  active_ = true;
  start_sem_.Post();
}

void ManagedThread::Join() {
  TIPS_CHECK(active_.load()) << "ManagedThread::Join without Start";
  finish_sem_.Wait();
  active_ = false;
}

void ManagedThread::Loop() {
  while (true) {
    start_sem_.Wait();
    if (terminate_.load()) return;
    try {
      task_();
    } catch (const std::exception& e) {
      fprintf(stderr, "ManagedThread task threw: %s\n", e.what());
    }
    finish_sem_.Post();
  }
}

namespace {
thread_local int tl_thread_id = -1;
}

int ThreadGroup::thread_id() { return tl_thread_id; }

ThreadGroup::ThreadGroup(int num_threads) { SetThreadNum(num_threads); }

ThreadGroup::~ThreadGroup() {
  if (running_) Join();
}

void ThreadGroup::SetThreadNum(int num_threads) {
  TIPS_CHECK(!running_) << "cannot resize a running ThreadGroup";
  TIPS_CHECK_GE(num_threads, 0);
  threads_.clear();
  for (int i = 0; i < num_threads; ++i) threads_.emplace_back(new ManagedThread);
  barrier_.Reset(num_threads > 0 ? num_threads : 1);
}

void ThreadGroup::Start(const std::function<void(int)>& func) {
  TIPS_CHECK(!running_);
  running_ = true;
  for (int i = 0; i < parallel_num(); ++i) {
    threads_[i]->Start([func, i] {
      tl_thread_id = i;
      func(i);
      tl_thread_id = -1;
    });
  }
}

void ThreadGroup::Join() {
  TIPS_CHECK(running_);
  for (auto& t : threads_) t->Join();
  running_ = false;
}

void ThreadGroup::Run(const std::function<void(int)>& func) {
  Start(func);
  Join();
}

void ParallelRunRange(ThreadGroup& group, size_t n, const std::function<void(int, size_t, size_t)>& func) {
  const int p = group.parallel_num();
  TIPS_CHECK_GT(p, 0);
  group.Run([&](int tid) {
    size_t begin = n * tid / p;
    size_t end   = n * (tid + 1) / p;
    func(tid, begin, end);
  });
}

ThreadPool::ThreadPool(int num_threads) {
  TIPS_CHECK_GT(num_threads, 0);
  for (int i = 0; i < num_threads; ++i) {
    workers_.emplace_back([this] {
      std::function<void()> task;
      while (tasks_.Read(&task)) task();
    });
  }
}

void ThreadPool::Shutdown() {
  tasks_.Close();
  for (auto& w : workers_)
    if (w.joinable()) w.join();
  workers_.clear();
}

ThreadPool::~ThreadPool() { Shutdown(); }

}  // namespace tips
