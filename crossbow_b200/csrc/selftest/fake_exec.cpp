// Fake executor for host-only tests of the runtime: completes every task after a fixed delay, can make one task fail
// and one task stall, and counts synchronisations.  It is NOT part of the runtime library: it is built into a test
// library of its own (and into the sanitizer self-test) and reaches the runtime through the same function-pointer table
// the CUDA executor uses.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#define FAKE_API extern "C" __attribute__((visibility("default")))

namespace {

struct FakeExec {
  int learners;
  std::atomic<int> task_us;
  std::atomic<int> fail_task{-1};        // task id whose wait returns an error
  std::atomic<int> hang_task{-1};        // task id whose wait does not return within the deadline
  std::atomic<uint64_t> syncs{0}, submits{0};
  std::vector<std::atomic<uint64_t>> current;
  std::vector<unsigned char> last_mask;
  std::mutex mu;
  FakeExec(int n, int us) : learners(n), task_us(us), current(256) { for (auto& c : current) c.store(0); }
};

int fake_submit(void* c, int learner, const void*, const void*, uint64_t task, int) {
  auto* f = (FakeExec*)c; f->current[learner].store(task); f->submits.fetch_add(1); return 0;
}
int finish(FakeExec* f, int learner, uint64_t task, float* loss, float* acc) {
  if ((int)task == f->hang_task.load()) std::this_thread::sleep_for(std::chrono::milliseconds(1500));
  else if (f->task_us.load() > 0) std::this_thread::sleep_for(std::chrono::microseconds(f->task_us.load()));
  if ((int)task == f->fail_task.load()) return 77;
  *loss = 1.0f / (1.0f + (float)task); *acc = (float)learner;
  return 0;
}
int fake_wait(void* c, int learner, float* loss, float* acc) {
  auto* f = (FakeExec*)c;
  return finish(f, learner, f->current[learner].load(), loss, acc);
}
int fake_wait_task(void* c, int learner, uint64_t task, float* loss, float* acc) { return finish((FakeExec*)c, learner, task, loss, acc); }
int fake_sync(void* c, uint64_t, const unsigned char* mask, int n, int) {
  auto* f = (FakeExec*)c; f->syncs.fetch_add(1);
  std::lock_guard<std::mutex> g(f->mu); f->last_mask.assign(mask, mask + n); return 0;
}

}  // namespace

FAKE_API void* rt_fake_create(int learners, int task_us) { return new FakeExec(learners, task_us); }
FAKE_API void rt_fake_destroy(void* f) { delete (FakeExec*)f; }
// addresses for rt_set_executor / rt_set_run_ahead: submit, wait, synchronise, wait_task
FAKE_API void rt_fake_table(void** submit, void** wait, void** synchronise, void** wait_task) {
  *submit = (void*)fake_submit; *wait = (void*)fake_wait; *synchronise = (void*)fake_sync; *wait_task = (void*)fake_wait_task;
}
FAKE_API void rt_fake_set_task_us(void* f, int us) { ((FakeExec*)f)->task_us.store(us); }
FAKE_API void rt_fake_inject(void* f, int fail_task, int hang_task) { ((FakeExec*)f)->fail_task.store(fail_task); ((FakeExec*)f)->hang_task.store(hang_task); }
FAKE_API unsigned long long rt_fake_syncs(void* f) { return ((FakeExec*)f)->syncs.load(); }
FAKE_API int rt_fake_last_mask(void* f, unsigned char* out, int n) {
  auto* fe = (FakeExec*)f; std::lock_guard<std::mutex> g(fe->mu);
  int m = (int)fe->last_mask.size() < n ? (int)fe->last_mask.size() : n;
  memcpy(out, fe->last_mask.data(), m); return m;
}
