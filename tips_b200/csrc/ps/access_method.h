// Server-side access methods: how a row is created and read on pull and how a
// pushed gradient changes it.  This is the plug-in point for server-side
// optimizers.
//
// Capability parity with the reference: PullAccessMethod{InitParam, GetPullValue,
// ApplyPullValue} / PushAccessMethod{ApplyPushValue} and the agents that bind a
// method to a table (tips/core/ps/access_method.h:15-143); SparseTablePullAccess
// (a new row is zero-initialised, sparse_access_method.h:10-39);
// SparseTableSgdPushAccess (sparse_access_method.h:41-61).  The reference's SGD
// rule overwrites the row with lr*grad; here SGD is w -= lr*g, Adagrad is added,
// and the literal rule is kept as LiteralReferencePushAccess for comparisons.
// WorkerParamCache (tips/core/ps/param.h:12-44) is the worker-side cache of
// pulled parameters and pending gradients.
#pragma once

#include <cmath>
#include <memory>
#include <unordered_map>

#include "core/datatype.h"
#include "core/threads.h"
#include "ps/table.h"

namespace tips {
namespace ps {

class PullAccessMethod {
 public:
  virtual ~PullAccessMethod() = default;
  // Fills a freshly created row for `key`.
  virtual void InitParam(uint64_t key, Datatype dtype, size_t length, AnyVec* row) = 0;
  // Produces the value sent to the worker from the stored row (may borrow it).
  virtual void GetPullValue(uint64_t key, const AnyVec& row, AnyVec* out) = 0;
  // Worker side: stores a pulled value into the worker's copy.
  virtual void ApplyPullValue(uint64_t key, AnyVec* local, const AnyVec& pulled) { local->CopyFrom(pulled); }
};

class PushAccessMethod {
 public:
  virtual ~PushAccessMethod() = default;
  // Applies the pushed value (a gradient) to the stored row. Runs on the shard's thread.
  virtual void ApplyPushValue(uint64_t key, AnyVec* row, const AnyVec& push_value) = 0;
};

class SparseTablePullAccess : public PullAccessMethod {
 public:
  void InitParam(uint64_t, Datatype dtype, size_t length, AnyVec* row) override { row->Resize(dtype, length); }
  void GetPullValue(uint64_t, const AnyVec& row, AnyVec* out) override { out->ShadowCopyFrom(row); }
};

class SparseTableSgdPushAccess : public PushAccessMethod {
 public:
  explicit SparseTableSgdPushAccess(double lr) : lr_(lr) {}
  void ApplyPushValue(uint64_t, AnyVec* row, const AnyVec& grad) override { AnyVec::Axpy(-lr_, grad, row); }

 private:
  double lr_;
};

class AdagradPushAccess : public PushAccessMethod {
 public:
  AdagradPushAccess(double lr, double eps = 1e-8) : lr_(lr), eps_(eps) {}
  void ApplyPushValue(uint64_t key, AnyVec* row, const AnyVec& grad) override {
    // The accumulators live in striped maps: a key is only ever touched by the thread of its shard, so a
    // stripe's lock is held for the lookup alone and shard threads rarely meet on one.
    Stripe& stripe = stripes_[(key * 0x9E3779B97F4A7C15ull) >> (64 - kStripeBits)];
    AnyVec* state;
    {
      std::lock_guard<std::mutex> lock(stripe.mu);
      AnyVec& s = stripe.state[key];
      if (s.size() != row->size()) s.Resize(Datatype::kFp64, row->size());
      state = &s;
    }
    const size_t n = row->size();
    double* acc    = reinterpret_cast<double*>(state->buffer());
    if (row->dtype() == Datatype::kFp32 && grad.dtype() == Datatype::kFp32 && grad.size() >= n) {
      float* w       = reinterpret_cast<float*>(row->buffer());
      const float* g = reinterpret_cast<const float*>(grad.buffer());
      for (size_t i = 0; i < n; ++i) {
        const double gi = g[i];
        const double si = acc[i] + gi * gi;
        acc[i]          = si;
        w[i]            = static_cast<float>(static_cast<double>(w[i]) - lr_ * gi / (std::sqrt(si) + eps_));
      }
      return;
    }
    for (size_t i = 0; i < n; ++i) {
      const double g = grad.GetAsDouble(i);
      const double s = acc[i] + g * g;
      acc[i]         = s;
      row->SetFromDouble(i, row->GetAsDouble(i) - lr_ * g / (std::sqrt(s) + eps_));
    }
  }

 private:
  static constexpr int kStripeBits = 6;
  struct Stripe {
    std::mutex mu;
    std::unordered_map<uint64_t, AnyVec> state;
  };
  double lr_, eps_;
  Stripe stripes_[1 << kStripeBits];
};

// param = lr * grad, exactly what the reference's SGD access method computes.
class LiteralReferencePushAccess : public PushAccessMethod {
 public:
  explicit LiteralReferencePushAccess(double lr) : lr_(lr) {}
  void ApplyPushValue(uint64_t, AnyVec* row, const AnyVec& grad) override { AnyVec::Mul(grad, lr_, row); }

 private:
  double lr_;
};

// Binds a pull method to a table: find the row, or create + initialise it first.
class PullAccessAgent {
 public:
  PullAccessAgent(SparseTable* table, std::shared_ptr<PullAccessMethod> method)
      : table_(table), method_(std::move(method)) {}
  void GetPullValue(uint64_t key, Datatype dtype, size_t length, AnyVec* out) {
    bool created = false;
    AnyVec* row  = table_->FindOrCreate(key, &created);  // a new row is initialised where it is stored
    if (created) method_->InitParam(key, dtype, length, row);
    method_->GetPullValue(key, *row, out);
  }
  PullAccessMethod* method() { return method_.get(); }

 private:
  SparseTable* table_;
  std::shared_ptr<PullAccessMethod> method_;
};

class PushAccessAgent {
 public:
  PushAccessAgent(SparseTable* table, std::shared_ptr<PushAccessMethod> method)
      : table_(table), method_(std::move(method)) {}
  // False when the key has never been pulled (the row does not exist).
  bool ApplyPushValue(uint64_t key, const AnyVec& push_value) {
    AnyVec* row = table_->Find(key);
    if (!row) return false;
    method_->ApplyPushValue(key, row, push_value);
    return true;
  }

 private:
  SparseTable* table_;
  std::shared_ptr<PushAccessMethod> method_;
};

// Worker-side cache: parameters pulled for the current step and gradients waiting to be pushed.
class WorkerParamCache {
 public:
  void SetParam(uint64_t key, const AnyVec& v) {
    RWLockWriteGuard g(lock_);
    params_[key].CopyFrom(v);
  }
  bool GetParam(uint64_t key, AnyVec* out) {
    RWLockReadGuard g(lock_);
    auto it = params_.find(key);
    if (it == params_.end()) return false;
    out->ShadowCopyFrom(it->second);
    return true;
  }
  void AccumulateGrad(uint64_t key, const AnyVec& g) {
    RWLockWriteGuard guard(lock_);
    AnyVec& acc = grads_[key];
    if (acc.size() != g.size()) acc.Resize(g.dtype(), g.size());
    AnyVec::Add(acc, g, &acc);
  }
  std::unordered_map<uint64_t, AnyVec> TakeGrads() {
    RWLockWriteGuard guard(lock_);
    std::unordered_map<uint64_t, AnyVec> out;
    out.swap(grads_);
    return out;
  }
  size_t num_params() {
    RWLockReadGuard g(lock_);
    return params_.size();
  }
  void Clear() {
    RWLockWriteGuard g(lock_);
    params_.clear();
    grads_.clear();
  }

 private:
  RWLock lock_;
  std::unordered_map<uint64_t, AnyVec> params_;
  std::unordered_map<uint64_t, AnyVec> grads_;
};

}  // namespace ps
}  // namespace tips
