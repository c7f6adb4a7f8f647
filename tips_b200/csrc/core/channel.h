// Blocking multi-producer / multi-consumer queue with open/close semantics.
//
// Same contract as the reference's Channel<T> (tips/core/common/channel.h:13-158):
// Read() blocks until an element arrives and returns false only when the channel
// is closed AND drained; Write()/WriteMove() return false once the channel has
// been closed; a capacity of 0 means unbounded.  It carries the coordinator's
// request queue, the per-shard task queues of the parameter server and the
// ordered execution queue of the collective engine.
#pragma once

#include <condition_variable>
#include <cstddef>
#include <deque>
#include <memory>
#include <mutex>
#include <utility>

namespace tips {

template <typename T>
class Channel {
 public:
  explicit Channel(size_t capacity = 0) : capacity_(capacity) {}
  Channel(const Channel&) = delete;
  Channel& operator=(const Channel&) = delete;

  void Open() {
    std::lock_guard<std::mutex> lock(mu_);
    closed_ = false;
  }

  void Close() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      closed_ = true;
    }
    not_empty_.notify_all();
    not_full_.notify_all();
  }

  bool closed() const {
    std::lock_guard<std::mutex> lock(mu_);
    return closed_;
  }

  size_t size() const {
    std::lock_guard<std::mutex> lock(mu_);
    return items_.size();
  }

  bool empty() const { return size() == 0; }
  size_t capacity() const { return capacity_; }

  void SetCapacity(size_t capacity) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      capacity_ = capacity;
    }
    not_full_.notify_all();
  }

  // Copies `value` in. Returns false if the channel is closed.
  bool Write(const T& value) {
    T copy(value);
    return WriteMove(std::move(copy));
  }

  bool WriteMove(T&& value) {
    std::unique_lock<std::mutex> lock(mu_);
    not_full_.wait(lock, [&] { return closed_ || capacity_ == 0 || items_.size() < capacity_; });
    if (closed_) return false;
    items_.emplace_back(std::move(value));
    lock.unlock();
    not_empty_.notify_one();
    return true;
  }

  // Blocks until an element is available. False means closed and drained.
  bool Read(T* out) {
    std::unique_lock<std::mutex> lock(mu_);
    not_empty_.wait(lock, [&] { return closed_ || !items_.empty(); });
    if (items_.empty()) return false;
    *out = std::move(items_.front());
    items_.pop_front();
    lock.unlock();
    not_full_.notify_one();
    return true;
  }

  // Waits at most `timeout_ms`. Returns 1 on success, 0 on timeout, -1 when
  // closed and drained.
  int ReadFor(T* out, int64_t timeout_ms) {
    std::unique_lock<std::mutex> lock(mu_);
    bool ok = not_empty_.wait_for(lock, std::chrono::milliseconds(timeout_ms),
                                  [&] { return closed_ || !items_.empty(); });
    if (!items_.empty()) {
      *out = std::move(items_.front());
      items_.pop_front();
      lock.unlock();
      not_full_.notify_one();
      return 1;
    }
    return ok ? -1 : 0;
  }

  // Non-blocking read.
  bool TryRead(T* out) {
    std::unique_lock<std::mutex> lock(mu_);
    if (items_.empty()) return false;
    *out = std::move(items_.front());
    items_.pop_front();
    lock.unlock();
    not_full_.notify_one();
    return true;
  }

 private:
  mutable std::mutex mu_;
  std::condition_variable not_empty_;
  std::condition_variable not_full_;
  std::deque<T> items_;
  size_t capacity_;
  bool closed_{false};
};

template <typename T>
std::shared_ptr<Channel<T>> MakeChannel(size_t capacity = 0) {
  return std::make_shared<Channel<T>>(capacity);
}

}  // namespace tips
