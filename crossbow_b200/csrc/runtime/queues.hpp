// Lock-free building blocks of the host runtime.
//
//   ThetaQueue   fixed set of slots, each FREE / BUSY / SKIP(disabled), handed out round-robin; grows by one slot
//                (auto-tuner adds a replica) and shrinks by disabling the last one.  Same role as
//                clib-multigpu/thetaqueue.c:13-209, but every wait is bounded and reports failure instead of spinning
//                for ever.
//   SpscQueue    wait-free single-producer single-consumer ring (waitfreequeue.c:17-90).
//   MpmcQueue    bounded multi-producer multi-consumer ring (Vyukov) used where the reference has a mutex-guarded
//                queue (threadsafequeue.c).
#pragma once
#include <atomic>
#include <mutex>
#include <deque>
#include <chrono>
#include <cstdint>
#include <memory>
#include <thread>
#include <vector>

namespace xb {

inline void cpu_relax(unsigned spins) {
  if (spins < 64) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  } else if (spins < 256) {
    std::this_thread::yield();
  } else {
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

using Clock = std::chrono::steady_clock;
inline double seconds_since(Clock::time_point t0) { return std::chrono::duration<double>(Clock::now() - t0).count(); }

class ThetaQueue {
 public:
  enum State : int { FREE = 0, BUSY = 1, SKIP = 2 };
  static constexpr int kMaxSlots = 256;

  explicit ThetaQueue(int n) : size_(n), cursor_(0) {
    for (int i = 0; i < kMaxSlots; ++i) slots_[i].state.store(i < n ? FREE : SKIP, std::memory_order_relaxed);
  }
  int size() const { return size_.load(std::memory_order_acquire); }
  int enabled() const {
    int c = 0;
    for (int i = 0; i < size(); ++i) c += slots_[i].state.load(std::memory_order_acquire) != SKIP;
    return c;
  }
  // Try to take slot i.
  bool try_acquire(int i) {
    int expect = FREE;
    return slots_[i].state.compare_exchange_strong(expect, BUSY, std::memory_order_acq_rel);
  }
  // Next enabled slot in round-robin order for which accept(i) holds, waiting up to timeout_s for it to become free.
  // Returns -1 on timeout.
  template <class Accept>
  int next(Accept accept, double timeout_s) {
    auto t0 = Clock::now();
    unsigned spins = 0;
    for (;;) {
      int n = size();
      for (int probe = 0; probe < n; ++probe) {
        int i = (int)(cursor_.load(std::memory_order_relaxed) % (uint64_t)n);
        int st = slots_[i].state.load(std::memory_order_acquire);
        if (st == SKIP || !accept(i)) { cursor_.fetch_add(1, std::memory_order_relaxed); continue; }
        // strict round robin: wait for THIS slot rather than skipping ahead (keeps replicas evenly loaded)
        if (try_acquire(i)) { cursor_.fetch_add(1, std::memory_order_relaxed); return i; }
        break;
      }
      cpu_relax(++spins);
      if ((spins & 63) == 0 && seconds_since(t0) > timeout_s) return -1;
    }
  }
  void release(int i) { slots_[i].state.store(FREE, std::memory_order_release); }
  int state(int i) const { return slots_[i].state.load(std::memory_order_acquire); }
  // One more enabled slot, born BUSY (the caller releases it once the new replica is ready): the lowest slot that was
  // disabled by shrink() if there is one, else a new slot at the end.  Returns its index or -1.
  int expand() {
    int n = size();
    for (int i = 0; i < n; ++i) {
      int expect = SKIP;
      if (slots_[i].state.compare_exchange_strong(expect, BUSY, std::memory_order_acq_rel)) return i;
    }
    if (n >= kMaxSlots) return -1;
    slots_[n].state.store(BUSY, std::memory_order_release);
    size_.store(n + 1, std::memory_order_release);
    return n;
  }
  // Disable the last enabled slot (must be FREE or it is waited for). Returns its index or -1.
  int shrink(double timeout_s) {
    for (int i = size() - 1; i >= 0; --i) {
      if (slots_[i].state.load(std::memory_order_acquire) == SKIP) continue;
      auto t0 = Clock::now();
      unsigned spins = 0;
      for (;;) {
        int expect = FREE;
        if (slots_[i].state.compare_exchange_strong(expect, SKIP, std::memory_order_acq_rel)) return i;
        cpu_relax(++spins);
        if (seconds_since(t0) > timeout_s) return -1;
      }
    }
    return -1;
  }

 private:
  struct alignas(64) Slot { std::atomic<int> state; };
  Slot slots_[kMaxSlots];
  std::atomic<int> size_;
  std::atomic<uint64_t> cursor_;
};

template <class T>
class SpscQueue {
 public:
  explicit SpscQueue(size_t capacity_pow2 = 1024) : mask_(capacity_pow2 - 1), buf_(capacity_pow2), head_(0), tail_(0) {}
  bool push(const T& v) {
    size_t t = tail_.load(std::memory_order_relaxed);
    if (t - head_.load(std::memory_order_acquire) > mask_) return false;
    buf_[t & mask_] = v;
    tail_.store(t + 1, std::memory_order_release);
    return true;
  }
  bool pop(T& v) {
    size_t h = head_.load(std::memory_order_relaxed);
    if (h == tail_.load(std::memory_order_acquire)) return false;
    v = buf_[h & mask_];
    head_.store(h + 1, std::memory_order_release);
    return true;
  }
  size_t size() const { return tail_.load(std::memory_order_acquire) - head_.load(std::memory_order_acquire); }

 private:
  size_t mask_;
  std::vector<T> buf_;
  alignas(64) std::atomic<size_t> head_;
  alignas(64) std::atomic<size_t> tail_;
};

template <class T>
class MpmcQueue {
 public:
  explicit MpmcQueue(size_t capacity_pow2 = 1024) : mask_(capacity_pow2 - 1), cells_(new Cell[capacity_pow2]), enq_(0), deq_(0) {
    for (size_t i = 0; i <= mask_; ++i) cells_[i].seq.store(i, std::memory_order_relaxed);
  }
  bool push(const T& v) {
    size_t pos = enq_.load(std::memory_order_relaxed);
    for (;;) {
      Cell& c = cells_[pos & mask_];
      size_t seq = c.seq.load(std::memory_order_acquire);
      intptr_t dif = (intptr_t)seq - (intptr_t)pos;
      if (dif == 0) {
        if (enq_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) { c.value = v; c.seq.store(pos + 1, std::memory_order_release); return true; }
      } else if (dif < 0) return false;
      else pos = enq_.load(std::memory_order_relaxed);
    }
  }
  bool pop(T& v) {
    size_t pos = deq_.load(std::memory_order_relaxed);
    for (;;) {
      Cell& c = cells_[pos & mask_];
      size_t seq = c.seq.load(std::memory_order_acquire);
      intptr_t dif = (intptr_t)seq - (intptr_t)(pos + 1);
      if (dif == 0) {
        if (deq_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) { v = c.value; c.seq.store(pos + mask_ + 1, std::memory_order_release); return true; }
      } else if (dif < 0) return false;
      else pos = deq_.load(std::memory_order_relaxed);
    }
  }

 private:
  struct Cell { std::atomic<size_t> seq; T value; };
  size_t mask_;
  std::unique_ptr<Cell[]> cells_;
  alignas(64) std::atomic<size_t> enq_;
  alignas(64) std::atomic<size_t> deq_;
};

// Task queue with a scheduling policy (task/TaskQueue.java:42-76, task/TaskWindow.java:185-227).
//   FIFO: a processor takes the oldest task.
//   HLS (hybrid latency scheduling): processor p (0 = CPU, 1 = GPU) walks the queue in order and takes the first task whose
//        graph it runs at least as fast as the other processor (throughput matrix[p][graph] >= matrix[other][graph]), or
//        any task once the work it has skipped would have kept the OTHER processor busy for longer than this task takes
//        here: skip cost = sum over skipped tasks of 1 / matrix[other][graph] >= 1 / matrix[p][graph].
//   NONE: never hands out a task (the reference's NULL policy).
// Tasks may carry the replica they are bound to and the oldest clock they accept (-1 / 0 = any), the reference's
// select() filter.  The native scheduler uses it between the dispatcher and its task handlers when scheduling is queued
// (--direct-scheduling false); a task costs microseconds to hand over against hundreds to run, so a mutex is enough.
class PolicyTaskQueue {
 public:
  enum Policy { HLS = 0, FIFO = 1, NONE = 2 };
  struct Task { long long id; int graph; int replica; long long clock; };
  explicit PolicyTaskQueue(int policy) : policy_(policy) {}
  void set_policy(int policy) { std::lock_guard<std::mutex> g(mu_); policy_ = policy; }
  void push(long long id, int graph, int replica, long long clock) {
    std::lock_guard<std::mutex> g(mu_);
    q_.push_back(Task{id, graph, replica, clock});
  }
  // matrix: [2][graphs] tasks per second; returns the task id or -1
  long long poll(int p, const int* matrix, int graphs, int replica, long long clock) {
    std::lock_guard<std::mutex> g(mu_);
    if (policy_ == NONE) return -1;
    const int other = (p + 1) % 2;
    double skip_cost = 0.0;
    for (auto it = q_.begin(); it != q_.end(); ++it) {
      const bool selectable = (it->replica < 0 || replica < 0 || it->replica == replica) && it->clock <= clock;
      const int gid = (it->graph >= 0 && it->graph < graphs) ? it->graph : 0;
      const double mine = matrix ? (double)matrix[p * graphs + gid] : 1.0, theirs = matrix ? (double)matrix[other * graphs + gid] : 1.0;
      if (selectable && (policy_ == FIFO || mine >= theirs || (mine > 0 && skip_cost >= 1.0 / mine))) {
        long long id = it->id;
        q_.erase(it);
        return id;
      }
      if (policy_ == HLS && theirs > 0) skip_cost += 1.0 / theirs;
    }
    return -1;
  }
  int size() { std::lock_guard<std::mutex> g(mu_); return (int)q_.size(); }

 private:
  int policy_;
  std::mutex mu_;
  std::deque<Task> q_;
};

}  // namespace xb
