// Host runtime: work clock, replica pool, task scheduler, handler threads, result ring, collector, watchdog.
//
// The reference spreads this over a Java dispatcher, a lock-free Java task queue, native task-handler and
// callback-handler thread pools, an off-heap result-slot ring and a Java result-collector thread
// (ExecutionContext.java:257-283, dispatcher/TaskDispatcher.java, clib-multigpu/taskhandler.c, callbackhandler.c,
// resulthandler.c:44-76, result/ResultCollector.java:40-70, modelmanager.c:147-245).  Here it is one C++ object driven
// through a C ABI.  The device (or a fake) is reached only through four function pointers, so the very same code
// runs against the CUDA learners, against the CPU oracle, and against a fake executor in host-only tests (the fake is
// not part of this library: csrc/selftest/fake_exec.cpp).
//
// Threads:   caller of rt_train  = dispatcher (numbers tasks, picks replicas, enqueues synchronisation)
//            task handlers       (optional) issue the submission so the dispatcher can run ahead
//            callback handlers   wait for a task's completion, publish its result slot, free the replica
//            collector           drains result slots in task order, aggregates loss / accuracy, stops on target loss
//            watchdog            aborts the run if a task does not complete within the deadline
// Every wait is bounded; a failure is reported through rt_error instead of exit(1).
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include <pthread.h>
#include <sched.h>

#include "queues.hpp"

#define RT_API extern "C" __attribute__((visibility("default")))

namespace xb {

struct Executor {
  // enqueue one task on learner `learner`; must not block on the device
  int (*submit)(void* ctx, int learner, const void* examples, const void* labels, uint64_t task, int phase);
  // block until that learner's task is complete, return its loss / accuracy
  int (*wait)(void* ctx, int learner, float* loss, float* accuracy);
  // enqueue a synchronisation over the learners flagged in `mask[0..n)`
  int (*synchronise)(void* ctx, uint64_t clock, const unsigned char* mask, int n, int copy);
  // batch source: host addresses of task `task`'s examples and labels (may be null: executor has its own data)
  int (*batch)(void* ctx, uint64_t task, int phase, const void** examples, const void** labels);
  void* ctx;
  // optional external batch source (data-set pipeline): returns a slot id >= 0 that is handed back through release
  // once the task has completed, or < 0 on failure
  int (*take)(void* dctx, uint64_t task, int phase, const void** examples, const void** labels);
  void (*release)(void* dctx, int slot);
  void* dctx;
  // optional (run-ahead): block until task `task` of that learner is complete.  A learner may then hold several tasks in
  // flight, so "the learner's task" of `wait` is no longer unique.
  int (*wait_task)(void* ctx, int learner, uint64_t task, float* loss, float* accuracy);
};

// 64-byte result slot, same state machine as the reference's ring (0 free -> 1 being written -> 2 ready -> 3 consumed -> 0)
struct alignas(64) ResultSlot {
  std::atomic<int> state;
  int learner;
  uint64_t task;
  float loss, accuracy;
  int phase;
  int status;
  double t_submit, t_done;
};

struct TaskItem { uint64_t task; int learner; int phase; const void* ex; const void* lab; int slot; };

enum SyncModel { BSP = 0, SSP = 1, ASP = 2 };

class Runtime {
 public:
  Runtime(int learners, int wpc, int slack, int sync_model, int result_slots, int task_handlers, int callback_handlers,
          double task_timeout_s)
      : theta_(learners), wpc_(wpc), slack_(slack), sync_model_(sync_model), nslots_(result_slots), slots_(new ResultSlot[result_slots]),
        n_task_handlers_(task_handlers), n_callback_handlers_(callback_handlers < 1 ? 1 : callback_handlers), timeout_(task_timeout_s),
        cb_q_(4096) {
    for (int i = 0; i < nslots_; ++i) slots_[i].state.store(0);
    for (int i = 0; i < ThetaQueue::kMaxSlots; ++i) { replica_clock_[i].store(0); replica_updates_[i].store(0); busy_since_[i].store(0.0); inflight_[i].store(0); }
    memset(&exec_, 0, sizeof(exec_));
    t_origin_ = Clock::now();
    start_threads();
  }
  ~Runtime() { stop_threads(); delete[] slots_; }

  void set_executor(const Executor& e) {
    auto t = exec_.take; auto r = exec_.release; auto d = exec_.dctx; auto w = exec_.wait_task;
    exec_ = e; exec_.take = t; exec_.release = r; exec_.dctx = d;
    if (!exec_.wait_task) exec_.wait_task = w;
  }
  // Run-ahead: a replica goes back to the free list as soon as its task has been handed to the device, until `depth` of
  // its tasks are in flight.  The device orders them (one stream per learner; a learner's next task waits for the
  // synchronisation event), so the host no longer sits between the end of one task and the start of the next.
  void set_run_ahead(int depth, decltype(Executor::wait_task) wait_task) {
    depth_ = (depth > 1 && wait_task) ? (depth > 4 ? 4 : depth) : 1;
    exec_.wait_task = wait_task;
  }
  void set_data_source(decltype(Executor::take) take, decltype(Executor::release) release, void* dctx) { exec_.take = take; exec_.release = release; exec_.dctx = dctx; }
  void set_policy(int policy) { policy_q_.set_policy(policy); }
  void set_target_loss(float t) { target_loss_ = t; }
  void set_affinity(int first_core) { first_core_ = first_core; }

  int learners() const { return theta_.enabled(); }
  uint64_t clock() const { return clock_.load(); }
  uint64_t tasks_issued() const { return next_task_.load(); }
  uint64_t tasks_completed() const { return completed_.load(); }
  const char* error() const { return error_.c_str(); }
  bool failed() const { return failed_.load(); }

  // ---- training loop (dispatcher) ----
  // Issues `ntasks` training tasks; returns the number issued (less if stopped early), negative on failure.
  long long train(long long ntasks, int phase) {
    if (!exec_.submit) return fail("no executor set");
    stop_.store(false);
    long long issued = 0;
    while (issued < ntasks && !stop_.load() && !failed_.load()) {
      uint64_t task = next_task_.fetch_add(1);
      const int64_t bound = (int64_t)clock_.load() - slack_ - 1;     // oldest model a task may use
      int learner = theta_.next([&](int i) { return (int64_t)replica_clock_[i].load(std::memory_order_acquire) >= bound; }, timeout_);
      if (learner < 0) return fail("no replica became free within the task deadline (a task or a synchronisation is stuck)");
      busy_since_[learner].store(now());
      const void *ex = nullptr, *lab = nullptr;
      int slot = -1;
      if (exec_.take) {
        slot = exec_.take(exec_.dctx, task, phase, &ex, &lab);
        if (slot < 0) return fail("data set could not provide a batch within the deadline");
      } else if (exec_.batch && exec_.batch(exec_.ctx, task, phase, &ex, &lab) != 0) return fail("data set could not provide a batch");
      TaskItem it{task, learner, phase, ex, lab, slot};
      if (n_task_handlers_ > 0) {
        // queued scheduling (ExecutionContext.java:272-277 with --direct-scheduling false): the task waits in the policy
        // queue until a task handler takes it according to --scheduling-policy
        auto t0 = Clock::now(); unsigned spins = 0;
        while (policy_q_.size() >= kPending) { cpu_relax(++spins); if (failed_.load() || seconds_since(t0) > timeout_) return fail("task queue stayed full"); }
        pending_[task % kPending] = it;
        policy_q_.push((long long)task, phase, -1, 0);
      } else {
        if (!issue(it)) return -1;
      }
      ++issued;
      if (phase == 0) {
        if (++inner_ >= wpc_) {
          inner_ = 0;
          if (!synchronise()) return -1;
        }
      }
    }
    return issued;
  }

  // Wait until every issued task has been collected. Returns 0, or -1 on failure / timeout.
  int drain(double timeout_s) {
    auto t0 = Clock::now();
    unsigned spins = 0;
    while (collected_.load() < next_task_.load()) {
      if (failed_.load()) return -1;
      cpu_relax(++spins);
      if (seconds_since(t0) > timeout_s) { fail("drain timed out"); return -1; }
    }
    return failed_.load() ? -1 : 0;      // (a failure whose task was collected before this call is still a failure)
  }

  void request_stop() { stop_.store(true); }

  // ---- replicas (auto-tuner) ----
  int add_learner() {
    int i = theta_.expand();
    if (i < 0) return -1;
    replica_clock_[i].store(clock_.load());
    theta_.release(i);
    return i;
  }
  int remove_learner() { return theta_.shrink(timeout_); }

  // ---- results ----
  struct Totals { double loss_sum, acc_sum; uint64_t n; float last_loss, last_acc; };
  Totals totals(bool reset) {
    std::lock_guard<std::mutex> g(tot_mu_);
    Totals t = tot_;
    if (reset) { tot_.loss_sum = tot_.acc_sum = 0; tot_.n = 0; }
    return t;
  }
  // copy up to n most recent (task, loss, acc) records
  int history(uint64_t* tasks, float* loss, float* acc, int n) {
    std::lock_guard<std::mutex> g(tot_mu_);
    const uint64_t have = hist_seq_ < kHistory ? hist_seq_ : kHistory;
    const int m = have < (uint64_t)n ? (int)have : n;
    for (int i = 0; i < m; ++i) { const auto& h = hist_[(hist_seq_ - m + i) % kHistory]; tasks[i] = h.task; loss[i] = h.loss; acc[i] = h.acc; }
    return m;
  }
  // Incremental read for a monitor that follows a run: records number `from`, `from` + 1, ... (every collected result has
  // a sequence number, counted from 0 over the life of the runtime), up to n of them.  `*first` receives the number of
  // the first record returned: larger than `from` when the reader fell more than the ring's capacity behind.
  int history_since(uint64_t from, uint64_t* first, uint64_t* tasks, float* loss, float* acc, int n) {
    std::lock_guard<std::mutex> g(tot_mu_);
    const uint64_t oldest = hist_seq_ > kHistory ? hist_seq_ - kHistory : 0;
    if (from < oldest) from = oldest;
    *first = from;
    int m = 0;
    for (uint64_t q = from; q < hist_seq_ && m < n; ++q, ++m) { const auto& h = hist_[q % kHistory]; tasks[m] = h.task; loss[m] = h.loss; acc[m] = h.acc; }
    hist_read_.store(from + (uint64_t)m, std::memory_order_release);
    return m;
  }
  // A follower (the monitor that displays results while a run is in progress) promises to keep calling history_since: the
  // collector then never overwrites a record the follower has not read yet - it waits for the reader instead, as the
  // reference's collector finishes displaying a result before it frees the slot (result/ResultCollector.java:40-70).
  void follow(bool on) { followed_.store(on, std::memory_order_release); }
  uint64_t history_count() { std::lock_guard<std::mutex> g(tot_mu_); return hist_seq_; }

 private:
  double now() const { return seconds_since(t_origin_); }
  long long fail(const char* why) {
    // the message is in place before anyone can see the flag (a reader of failed() may ask for error() at once)
    std::lock_guard<std::mutex> g(err_mu_);
    if (!failed_.load()) { error_ = why; failed_.store(true); }
    return -1;
  }
  template <class Q>
  bool push_bounded(Q& q, const TaskItem& it) {
    auto t0 = Clock::now();
    unsigned spins = 0;
    while (!q.push(it)) {
      cpu_relax(++spins);
      if (seconds_since(t0) > timeout_) return false;
    }
    return true;
  }
  bool issue(const TaskItem& it) {
    int e = exec_.submit(exec_.ctx, it.learner, it.ex, it.lab, it.task, it.phase);
    if (e != 0) { char b[96]; snprintf(b, sizeof b, "task submission failed with code %d", e); fail(b); return false; }
    if (!push_bounded(cb_q_, it)) { fail("callback queue stayed full"); return false; }
    if (depth_ > 1 && inflight_[it.learner].fetch_add(1) + 1 < depth_) theta_.release(it.learner);
    return true;
  }
  // Called by the dispatcher after the wpc-th task of a clock has been handed over.
  bool synchronise() {
    if (n_task_handlers_ > 0) {          // submissions must be on the device queues before the synchronisation is
      auto t0 = Clock::now(); unsigned spins = 0;
      while (handed_.load() < next_task_.load()) { cpu_relax(++spins); if (failed_.load() || seconds_since(t0) > timeout_) { fail("task handlers stalled"); return false; } }
    }
    const int n = theta_.size();
    std::vector<unsigned char> mask(n, 0);
    int count = 0;
    for (int i = 0; i < n; ++i) {
      int st = theta_.state(i);
      if (st == ThetaQueue::SKIP) continue;
      // BSP: every replica takes part (ordering is enforced on the device by events, a replica that is still
      // running simply makes the synchronisation wait there).  SSP / ASP: only replicas that are idle right now.
      if (sync_model_ == BSP || st == ThetaQueue::FREE) { mask[i] = 1; ++count; }
    }
    uint64_t c = clock_.load() + 1;
    if (count > 0 && exec_.synchronise) {
      int e = exec_.synchronise(exec_.ctx, c, mask.data(), n, 0);
      if (e != 0) { char b[96]; snprintf(b, sizeof b, "synchronisation failed with code %d", e); fail(b); return false; }
    }
    for (int i = 0; i < n; ++i) if (mask[i]) { replica_clock_[i].store(c, std::memory_order_release); replica_updates_[i].store(0); }
    clock_.store(c);
    return true;
  }

  void start_threads() {
    running_.store(true);
    for (int i = 0; i < n_task_handlers_; ++i) threads_.emplace_back([this, i] { pin(i + 1); task_loop(); });
    for (int i = 0; i < n_callback_handlers_; ++i) threads_.emplace_back([this, i] { pin(n_task_handlers_ + i + 1); callback_loop(); });
    threads_.emplace_back([this] { collector_loop(); });
    threads_.emplace_back([this] { watchdog_loop(); });
  }
  void stop_threads() {
    running_.store(false);
    for (auto& t : threads_) if (t.joinable()) t.join();
    threads_.clear();
  }
  void pin(int idx) {
    if (first_core_ < 0) return;
    cpu_set_t set; CPU_ZERO(&set);
    int ncpu = (int)std::thread::hardware_concurrency();
    if (ncpu <= 0) return;
    CPU_SET((first_core_ + idx) % ncpu, &set);
    pthread_setaffinity_np(pthread_self(), sizeof(set), &set);
  }
  void task_loop() {
    unsigned spins = 0;
    while (running_.load()) {
      // this process drives one GPU: it polls as processor 1 of the policy's two (0 = CPU workers, 1 = GPU worker)
      const long long id = policy_q_.poll(1, nullptr, 1, -1, (long long)1 << 62);
      if (id >= 0) { spins = 0; TaskItem it = pending_[(uint64_t)id % kPending]; if (!failed_.load()) issue(it); handed_.fetch_add(1); }
      else cpu_relax(++spins);
    }
  }
  void callback_loop() {
    unsigned spins = 0;
    TaskItem it;
    while (running_.load()) {
      if (!cb_q_.pop(it)) { cpu_relax(++spins); continue; }
      spins = 0;
      if (n_task_handlers_ == 0) handed_.fetch_add(1);
      float loss = NAN, acc = NAN;
      int e = failed_.load() ? -1
              : (depth_ > 1 ? exec_.wait_task(exec_.ctx, it.learner, it.task, &loss, &acc) : exec_.wait(exec_.ctx, it.learner, &loss, &acc));
      if (e != 0 && !failed_.load()) { char b[96]; snprintf(b, sizeof b, "task %llu failed on learner %d with code %d", (unsigned long long)it.task, it.learner, e); fail(b); }
      if (it.slot >= 0 && exec_.release) exec_.release(exec_.dctx, it.slot);      // the batch has been consumed
      // publish the result slot: 0 -> 1, fill, 1 -> 2
      ResultSlot& s = slots_[it.task % (uint64_t)nslots_];
      unsigned sp = 0; int expect = 0;
      auto t0 = Clock::now();
      while (!s.state.compare_exchange_weak(expect, 1)) { expect = 0; cpu_relax(++sp); if (seconds_since(t0) > timeout_) { fail("result ring stayed full"); break; } }
      s.learner = it.learner; s.task = it.task; s.loss = loss; s.accuracy = acc; s.phase = it.phase; s.status = e; s.t_done = now();
      s.state.store(2, std::memory_order_release);
      replica_updates_[it.learner].fetch_add(1);
      busy_since_[it.learner].store(0.0);
      // (run-ahead: the replica was already released at submission unless it was then at its in-flight limit)
      if (depth_ <= 1 || inflight_[it.learner].fetch_sub(1) - 1 == depth_ - 1) theta_.release(it.learner);
      completed_.fetch_add(1);
    }
  }
  void collector_loop() {
    unsigned spins = 0;
    while (running_.load()) {
      uint64_t next = collected_.load();
      ResultSlot& s = slots_[next % (uint64_t)nslots_];
      if (s.state.load(std::memory_order_acquire) != 2 || s.task != next) { cpu_relax(++spins); continue; }
      spins = 0;
      s.state.store(3);
      bool full = false;
      {
        std::lock_guard<std::mutex> g(tot_mu_);
        if (s.phase == 0 && std::isfinite(s.loss)) { tot_.loss_sum += s.loss; tot_.acc_sum += s.accuracy; tot_.n += 1; tot_.last_loss = s.loss; tot_.last_acc = s.accuracy; }
        else if (s.phase != 0 && std::isfinite(s.accuracy)) { tot_.loss_sum += s.loss; tot_.acc_sum += s.accuracy; tot_.n += 1; }
        hist_[hist_seq_ % kHistory] = {s.task, s.loss, s.accuracy};
        ++hist_seq_;
        full = followed_.load(std::memory_order_acquire) && hist_seq_ - hist_read_.load(std::memory_order_acquire) >= kHistory;
      }
      if (s.phase == 0 && target_loss_ > 0 && s.loss <= target_loss_) stop_.store(true);
      s.state.store(0, std::memory_order_release);
      collected_.fetch_add(1);
      // the ring is full of records the follower has not read: let it catch up before the next one is written
      for (unsigned sp = 0; full && running_.load() && followed_.load(std::memory_order_acquire); ) {
        { std::lock_guard<std::mutex> g(tot_mu_); full = hist_seq_ - hist_read_.load(std::memory_order_acquire) >= kHistory; }
        if (full) cpu_relax(++sp);
      }
    }
  }
  void watchdog_loop() {
    while (running_.load()) {
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
      double t = now();
      for (int i = 0; i < theta_.size(); ++i) {
        double b = busy_since_[i].load();
        if (b > 0.0 && t - b > timeout_ && theta_.state(i) == ThetaQueue::BUSY) {
          char msg[128]; snprintf(msg, sizeof msg, "watchdog: learner %d has been busy for %.1f s (deadline %.1f s)", i, t - b, timeout_);
          fail(msg);
        }
      }
    }
  }

  ThetaQueue theta_;
  int wpc_, slack_, sync_model_;
  int inner_ = 0;
  int nslots_;
  ResultSlot* slots_;
  int n_task_handlers_, n_callback_handlers_;
  double timeout_;
  int first_core_ = -1;
  Executor exec_;
  static constexpr uint64_t kPending = 4096;
  MpmcQueue<TaskItem> cb_q_;
  PolicyTaskQueue policy_q_{PolicyTaskQueue::FIFO};   // dispatcher -> task handlers, ordered by --scheduling-policy
  std::vector<TaskItem> pending_ = std::vector<TaskItem>(kPending);   // the queued tasks' payloads, by task number
  std::atomic<uint64_t> next_task_{0}, completed_{0}, collected_{0}, handed_{0}, clock_{0};
  std::atomic<uint64_t> replica_clock_[ThetaQueue::kMaxSlots];
  std::atomic<uint64_t> replica_updates_[ThetaQueue::kMaxSlots];
  std::atomic<double> busy_since_[ThetaQueue::kMaxSlots];
  std::atomic<int> inflight_[ThetaQueue::kMaxSlots];
  int depth_ = 1;
  std::atomic<bool> running_{false}, stop_{false}, failed_{false};
  std::string error_;
  std::mutex err_mu_;
  float target_loss_ = -1.f;
  std::vector<std::thread> threads_;
  std::mutex tot_mu_;
  Totals tot_{0, 0, 0, NAN, NAN};
  struct Hist { uint64_t task; float loss, acc; };
  static constexpr uint64_t kHistory = 1 << 16;       // ring of the most recent results (a monitor reads it incrementally)
  std::vector<Hist> hist_ = std::vector<Hist>(kHistory);
  uint64_t hist_seq_ = 0;                             // results collected so far = sequence number of the next record
  std::atomic<uint64_t> hist_read_{0};                // first record the follower has not read
  std::atomic<bool> followed_{false};
  Clock::time_point t_origin_;
};

}  // namespace xb

using namespace xb;

RT_API void* rt_create(int learners, int wpc, int slack, int sync_model, int result_slots, int task_handlers, int callback_handlers, double task_timeout_s) {
  if (learners < 1 || learners > ThetaQueue::kMaxSlots || wpc < 1 || result_slots < 2) return nullptr;
  return new Runtime(learners, wpc, slack, sync_model, result_slots, task_handlers, callback_handlers, task_timeout_s);
}
RT_API void rt_destroy(void* r) { delete (Runtime*)r; }
RT_API void rt_set_executor(void* r, void* submit, void* wait, void* synchronise, void* batch, void* ctx) {
  Executor e; memset(&e, 0, sizeof(e));
  e.submit = (decltype(e.submit))submit; e.wait = (decltype(e.wait))wait; e.synchronise = (decltype(e.synchronise))synchronise;
  e.batch = (decltype(e.batch))batch; e.ctx = ctx;
  ((Runtime*)r)->set_executor(e);
}
RT_API void rt_set_data_source(void* r, void* take, void* release, void* dctx) {
  ((Runtime*)r)->set_data_source((decltype(Executor::take))take, (decltype(Executor::release))release, dctx);
}
RT_API void rt_set_run_ahead(void* r, int depth, void* wait_task) { ((Runtime*)r)->set_run_ahead(depth, (decltype(Executor::wait_task))wait_task); }
RT_API void rt_set_scheduling_policy(void* r, int policy) { ((Runtime*)r)->set_policy(policy); }
RT_API void rt_set_target_loss(void* r, float t) { ((Runtime*)r)->set_target_loss(t); }
RT_API void rt_set_affinity(void* r, int first_core) { ((Runtime*)r)->set_affinity(first_core); }
RT_API long long rt_train(void* r, long long ntasks, int phase) { return ((Runtime*)r)->train(ntasks, phase); }
RT_API int rt_drain(void* r, double timeout_s) { return ((Runtime*)r)->drain(timeout_s); }
RT_API void rt_stop(void* r) { ((Runtime*)r)->request_stop(); }
RT_API int rt_add_learner(void* r) { return ((Runtime*)r)->add_learner(); }
RT_API int rt_remove_learner(void* r) { return ((Runtime*)r)->remove_learner(); }
RT_API int rt_learners(void* r) { return ((Runtime*)r)->learners(); }
RT_API unsigned long long rt_clock(void* r) { return ((Runtime*)r)->clock(); }
RT_API unsigned long long rt_tasks_issued(void* r) { return ((Runtime*)r)->tasks_issued(); }
RT_API unsigned long long rt_tasks_completed(void* r) { return ((Runtime*)r)->tasks_completed(); }
RT_API int rt_failed(void* r) { return ((Runtime*)r)->failed() ? 1 : 0; }
RT_API const char* rt_error(void* r) { return ((Runtime*)r)->error(); }
RT_API void rt_totals(void* r, int reset, double* loss_sum, double* acc_sum, unsigned long long* n, float* last_loss, float* last_acc) {
  auto t = ((Runtime*)r)->totals(reset != 0);
  *loss_sum = t.loss_sum; *acc_sum = t.acc_sum; *n = t.n; *last_loss = t.last_loss; *last_acc = t.last_acc;
}
RT_API int rt_history(void* r, unsigned long long* tasks, float* loss, float* acc, int n) {
  return ((Runtime*)r)->history((uint64_t*)tasks, loss, acc, n);
}
RT_API int rt_history_since(void* r, unsigned long long from, unsigned long long* first, unsigned long long* tasks, float* loss, float* acc, int n) {
  return ((Runtime*)r)->history_since(from, (uint64_t*)first, (uint64_t*)tasks, loss, acc, n);
}
RT_API unsigned long long rt_history_count(void* r) { return ((Runtime*)r)->history_count(); }
RT_API void rt_history_follow(void* r, int on) { ((Runtime*)r)->follow(on != 0); }

// ---- theta queue, exposed for tests and for Python-side pools ---------------------------------------------------------
// ---- micro-benchmarks of the queues (src/test/java/.../microbenchmarks/{queues,slots}) -------------------------------------
// Million items per second through one bounded MPMC queue with the given number of producer and consumer threads.
RT_API double rt_bench_mpmc(int producers, int consumers, long long items) {
  if (producers < 1 || consumers < 1 || items < 1) return 0.0;
  MpmcQueue<TaskItem> q(4096);
  std::atomic<long long> produced{0}, consumed{0};
  auto t0 = Clock::now();
  std::vector<std::thread> th;
  for (int p = 0; p < producers; ++p)
    th.emplace_back([&] {
      unsigned spins = 0;
      for (;;) {
        long long i = produced.fetch_add(1);
        if (i >= items) break;
        TaskItem it{(uint64_t)i, 0, 0, nullptr, nullptr, -1};
        while (!q.push(it)) cpu_relax(++spins);
      }
    });
  for (int c = 0; c < consumers; ++c)
    th.emplace_back([&] {
      unsigned spins = 0;
      TaskItem it;
      while (consumed.load() < items) {
        if (q.pop(it)) consumed.fetch_add(1);
        else cpu_relax(++spins);
      }
    });
  for (auto& t : th) t.join();
  return (double)items / seconds_since(t0) / 1e6;
}
// Million next() + release() pairs per second on a replica pool of `slots` entries (one thread).
RT_API double rt_bench_theta(int slots, long long rounds) {
  if (slots < 1 || slots > ThetaQueue::kMaxSlots || rounds < 1) return 0.0;
  ThetaQueue q(slots);
  auto t0 = Clock::now();
  for (long long i = 0; i < rounds; ++i) {
    int s = q.next([](int) { return true; }, 1.0);
    if (s < 0) return 0.0;
    q.release(s);
  }
  return (double)rounds / seconds_since(t0) / 1e6;
}
RT_API void* rt_taskq_create(int policy) { return new PolicyTaskQueue(policy); }
RT_API void rt_taskq_destroy(void* q) { delete (PolicyTaskQueue*)q; }
RT_API void rt_taskq_push(void* q, long long id, int graph, int replica, long long clock) { ((PolicyTaskQueue*)q)->push(id, graph, replica, clock); }
RT_API long long rt_taskq_poll(void* q, int p, const int* matrix, int graphs, int replica, long long clock) {
  return ((PolicyTaskQueue*)q)->poll(p, matrix, graphs, replica, clock);
}
RT_API int rt_taskq_size(void* q) { return ((PolicyTaskQueue*)q)->size(); }
RT_API void* rt_theta_create(int n) { return new ThetaQueue(n); }
RT_API void rt_theta_destroy(void* q) { delete (ThetaQueue*)q; }
RT_API int rt_theta_next(void* q, double timeout_s) { return ((ThetaQueue*)q)->next([](int) { return true; }, timeout_s); }
RT_API void rt_theta_release(void* q, int i) { ((ThetaQueue*)q)->release(i); }
RT_API int rt_theta_expand(void* q) { return ((ThetaQueue*)q)->expand(); }
RT_API int rt_theta_shrink(void* q, double timeout_s) { return ((ThetaQueue*)q)->shrink(timeout_s); }
RT_API int rt_theta_size(void* q) { return ((ThetaQueue*)q)->size(); }
RT_API int rt_theta_enabled(void* q) { return ((ThetaQueue*)q)->enabled(); }

// ---- CPU affinity (clib-multigpu/CPU.c:26-83) -------------------------------------------------------------------------
RT_API int rt_cpu_bind(int core) {
  cpu_set_t set; CPU_ZERO(&set); CPU_SET(core, &set);
  return sched_setaffinity(0, sizeof(set), &set);
}
RT_API int rt_cpu_unbind() {
  cpu_set_t set; CPU_ZERO(&set);
  int n = (int)std::thread::hardware_concurrency();
  for (int i = 0; i < n; ++i) CPU_SET(i, &set);
  return sched_setaffinity(0, sizeof(set), &set);
}
RT_API int rt_cpu_id() { return sched_getcpu(); }
RT_API int rt_cpu_count() { return (int)std::thread::hardware_concurrency(); }
