// Stand-alone driver of the host runtime against its fake executor, meant to be built with -fsanitize=thread or
// -fsanitize=address (the reference has no such check: scripts/run.sh:19,162-163 only offers cuda-memcheck).
// Scenarios: plain dispatch with task and callback handler threads, run-ahead, replica add / remove between runs, an
// injected task failure.  Prints SELFTEST_OK and exits 0 when every scenario behaved; sanitizer reports go to stderr.
#include <cstdio>
#include <cstdlib>
#include <cstring>

extern "C" {
void* rt_create(int learners, int wpc, int slack, int sync_model, int result_slots, int task_handlers, int callback_handlers, double task_timeout_s);
void rt_destroy(void* r);
long long rt_train(void* r, long long ntasks, int phase);
int rt_drain(void* r, double timeout_s);
int rt_add_learner(void* r);
int rt_remove_learner(void* r);
int rt_learners(void* r);
unsigned long long rt_clock(void* r);
unsigned long long rt_tasks_completed(void* r);
int rt_failed(void* r);
const char* rt_error(void* r);
int rt_history(void* r, unsigned long long* tasks, float* loss, float* acc, int n);
int rt_history_since(void* r, unsigned long long from, unsigned long long* first, unsigned long long* tasks, float* loss, float* acc, int n);
void rt_set_executor(void* r, void* submit, void* wait, void* synchronise, void* batch, void* ctx);
void rt_set_run_ahead(void* r, int depth, void* wait_task);
void* rt_fake_create(int learners, int task_us);
void rt_fake_destroy(void* f);
void rt_fake_table(void** submit, void** wait, void** synchronise, void** wait_task);
void rt_fake_inject(void* f, int fail_task, int hang_task);
unsigned long long rt_fake_syncs(void* f);
int rec_jpeg_decode(const void* data, long long size, unsigned char* rgb_out, long long capacity, int* w, int* h);
}
#include <thread>
#include <vector>

static void rt_fake_attach(void* rt, void* fake) {
  void *sub, *wait, *sync, *wt;
  rt_fake_table(&sub, &wait, &sync, &wt);
  rt_set_executor(rt, sub, wait, sync, nullptr, fake);
}
static void rt_fake_run_ahead(void* rt, int depth) {
  void *sub, *wait, *sync, *wt;
  rt_fake_table(&sub, &wait, &sync, &wt);
  rt_set_run_ahead(rt, depth, wt);
}

#define CHECK(cond)                                                                  \
  do {                                                                               \
    if (!(cond)) { fprintf(stderr, "selftest: %s failed at line %d\n", #cond, __LINE__); return 1; } \
  } while (0)

static int scenario(int handlers, int depth) {
  void* rt = rt_create(4, 4, 0, 0, 256, handlers, 2, 5.0);
  CHECK(rt != nullptr);
  void* fake = rt_fake_create(16, 50);
  rt_fake_attach(rt, fake);
  if (depth > 1) rt_fake_run_ahead(rt, depth);
  CHECK(rt_train(rt, 400, 0) == 400);
  CHECK(rt_drain(rt, 20.0) == 0);
  CHECK(rt_tasks_completed(rt) == 400 && rt_clock(rt) == 100 && rt_fake_syncs(fake) == 100);
  unsigned long long tasks[512]; float loss[512], acc[512];
  int n = rt_history(rt, tasks, loss, acc, 512);
  CHECK(n == 400);
  for (int i = 0; i < n; ++i) CHECK(tasks[i] == (unsigned long long)i);
  {
    unsigned long long first = 0, t2[16]; float l2[16], a2[16];
    CHECK(rt_history_since(rt, 390, &first, t2, l2, a2, 16) == 10 && first == 390 && t2[9] == 399);
  }
  if (depth > 1) for (int i = 0; i < n; ++i) CHECK(loss[i] > 0.999f / (1.0f + (float)i) && loss[i] < 1.001f / (1.0f + (float)i));
  // replicas come and go between runs (auto-tuner)
  CHECK(rt_add_learner(rt) == 4 && rt_learners(rt) == 5);
  CHECK(rt_train(rt, 40, 0) == 40 && rt_drain(rt, 20.0) == 0);
  CHECK(rt_remove_learner(rt) == 4 && rt_learners(rt) == 4);
  CHECK(rt_train(rt, 40, 0) == 40 && rt_drain(rt, 20.0) == 0);
  CHECK(rt_tasks_completed(rt) == 480 && !rt_failed(rt));
  // a failing task is reported, not fatal
  rt_fake_inject(fake, 485, -1);
  rt_train(rt, 16, 0);
  CHECK(rt_drain(rt, 20.0) != 0 && rt_failed(rt) && strstr(rt_error(rt), "task 485 failed") != nullptr);
  rt_destroy(rt);
  rt_fake_destroy(fake);
  return 0;
}

// The JPEG decoder reads untrusted files: every truncation of a small file and a few thousand random corruptions of it
// must end in an error code or an image, without touching memory outside its buffers (AddressSanitizer) and without a
// data race between decode workers (ThreadSanitizer: the inverse-DCT table is initialised on first use).
static int jpeg_scenario(const char* path) {
  FILE* f = fopen(path, "rb");
  CHECK(f != nullptr);
  std::vector<unsigned char> file(1 << 20);
  size_t n = fread(file.data(), 1, file.size(), f);
  fclose(f);
  CHECK(n > 100);
  file.resize(n);
  std::vector<std::thread> workers;
  std::vector<int> good(4, 0);
  for (int t = 0; t < 4; ++t)
    workers.emplace_back([&, t] {
      std::vector<unsigned char> rgb(1 << 22);
      int w = 0, h = 0;
      if (rec_jpeg_decode(file.data(), (long long)file.size(), rgb.data(), (long long)rgb.size(), &w, &h) == 0 && w > 0 && h > 0) good[t] = 1;
      unsigned long long s = 0x9E3779B97F4A7C15ull * (t + 1);
      auto rnd = [&] { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; };
      for (size_t cut = 2 + t; cut < file.size(); cut += 4) {                       // truncations (exact-size heap copies)
        std::vector<unsigned char> part(file.begin(), file.begin() + cut);
        rec_jpeg_decode(part.data(), (long long)part.size(), rgb.data(), (long long)rgb.size(), &w, &h);
      }
      for (int i = 0; i < 1500; ++i) {                                              // corruptions
        std::vector<unsigned char> bad(file);
        const int flips = 1 + (int)(rnd() % 6);
        for (int j = 0; j < flips; ++j) bad[2 + rnd() % (bad.size() - 2)] = (unsigned char)rnd();
        rec_jpeg_decode(bad.data(), (long long)bad.size(), rgb.data(), (long long)rgb.size(), &w, &h);
      }
    });
  for (auto& th : workers) th.join();
  for (int g : good) CHECK(g == 1);
  return 0;
}

int main(int argc, char** argv) {
  for (int a = 1; a < argc; ++a)
    if (jpeg_scenario(argv[a])) return 1;
  for (int handlers = 0; handlers <= 2; handlers += 2)
    for (int depth = 1; depth <= 2; ++depth)
      if (scenario(handlers, depth)) return 1;
  printf("SELFTEST_OK\n");
  return 0;
}
