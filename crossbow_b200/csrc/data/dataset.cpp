// Data-set pipeline of the host runtime.
//
//   Metadata     text "key : value" description of a data set (data/DatasetMetadata.java:259-345; sample
//                data/imagenet/imagenet-train.metadata): prefixes of the partition files, partition count, element
//                count, batch size, shapes, types, per-batch padding.
//   Writer       cuts a stream of (example, label) tuples into partition files "<prefix>.<n>" (n from 1) holding whole
//                batches, each batch padded to a multiple of the page size so that a batch can be pinned / registered on
//                its own, and repeats the first tuples to fill the last batch (preprocess/DatasetFileWriter.java:90-142,
//                DatasetMetadata.java:396-458).
//   Basic        memory-maps every partition and keeps a sliding WINDOW of partitions resident: a file-handler thread
//                locks (mlock + madvise, plus an optional registration hook, e.g. cudaHostRegister) the partitions that
//                enter the window and releases those that leave it (clib-multigpu/dataset.c:27-103, datasetfile.c,
//                datasetfilehandler.c:16-102).  A task is then just two addresses inside the mappings.
//   Light        fixed ring of page-aligned slots (one batch each) filled by copier threads from the mapped files;
//                per-slot state machine 0 free -> 1 reserved -> 2 being filled -> 3 ready -> 4 in use -> 0
//                (lightweightdataset*.c).  Tasks that straddle two partitions or wrap around are handled by the
//                precomputed task table.
// All waits are bounded and report failure through the return value.
#include <atomic>
#include <algorithm>
#include <cerrno>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <map>
#include <mutex>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

#include "../runtime/queues.hpp"

#define RT_API extern "C" __attribute__((visibility("default")))

namespace xb {

static size_t page_size() { static size_t p = (size_t)sysconf(_SC_PAGESIZE); return p; }
static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Meta {
  std::string examples, labels;
  long long partitions = 0, elements = 0, batch = 1;
  std::vector<long long> example_shape, label_shape;
  std::string example_type = "float", label_type = "int";
  long long example_pad = 0, label_pad = 0;     // bytes of padding after every batch
  long long batches_per_partition = 0;          // 0: derive from file size
  long long example_bytes() const { long long n = 4; for (auto d : example_shape) n *= d; return n; }
  long long label_bytes() const { long long n = 4; for (auto d : label_shape) n *= d; return n; }
  long long batch_example_bytes() const { return batch * example_bytes() + example_pad; }
  long long batch_label_bytes() const { return batch * label_bytes() + label_pad; }
  long long batches() const { return elements / batch; }
};

static std::string trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
  return a == std::string::npos ? "" : s.substr(a, b - a + 1);
}
static std::vector<long long> parse_shape(const std::string& v) {
  std::vector<long long> out; std::string num;
  for (char c : v) { if (isdigit((unsigned char)c)) num += c; else if (!num.empty()) { out.push_back(atoll(num.c_str())); num.clear(); } }
  if (!num.empty()) out.push_back(atoll(num.c_str()));
  return out;
}
static bool meta_load(const char* path, Meta& m) {
  FILE* f = fopen(path, "r");
  if (!f) return false;
  char line[4096];
  while (fgets(line, sizeof line, f)) {
    std::string s = trim(line);
    if (s.empty() || s[0] == '#') continue;
    size_t c = s.find(':');
    if (c == std::string::npos) continue;
    std::string k = trim(s.substr(0, c)), v = trim(s.substr(c + 1));
    if (k == "examples") m.examples = v; else if (k == "labels") m.labels = v;
    else if (k == "partitions") m.partitions = atoll(v.c_str()); else if (k == "elements") m.elements = atoll(v.c_str());
    else if (k == "batch size") m.batch = atoll(v.c_str()); else if (k == "example shape") m.example_shape = parse_shape(v);
    else if (k == "label shape") m.label_shape = parse_shape(v); else if (k == "example type") m.example_type = v;
    else if (k == "label type") m.label_type = v; else if (k == "example pad") m.example_pad = atoll(v.c_str());
    else if (k == "label pad") m.label_pad = atoll(v.c_str()); else if (k == "batches per partition") m.batches_per_partition = atoll(v.c_str());
  }
  fclose(f);
  return m.partitions > 0 && m.elements > 0 && !m.example_shape.empty();
}
static std::string shape_str(const std::vector<long long>& s) {
  std::string o = "[";
  for (size_t i = 0; i < s.size(); ++i) { o += std::to_string(s[i]); if (i + 1 < s.size()) o += ", "; }
  return o + "]";
}
static bool meta_store(const char* path, const Meta& m) {
  FILE* f = fopen(path, "w");
  if (!f) return false;
  fprintf(f, "# Metadata file\n#\nexamples     : %s\nlabels       : %s\npartitions   : %lld\nelements     : %lld\nbatch size   : %lld\n",
          m.examples.c_str(), m.labels.c_str(), m.partitions, m.elements, m.batch);
  fprintf(f, "example shape: %s\nlabel shape  : %s\nexample type : %s\nlabel type   : %s\nexample pad  : %lld\nlabel pad    : %lld\n",
          shape_str(m.example_shape).c_str(), shape_str(m.label_shape).c_str(), m.example_type.c_str(), m.label_type.c_str(), m.example_pad, m.label_pad);
  fprintf(f, "batches per partition : %lld\n# EOF\n", m.batches_per_partition);
  fclose(f);
  return true;
}

// ---- writer ----------------------------------------------------------------------------------------------------------
struct Writer {
  Meta m;
  std::string meta_path;
  long long partition_bytes;
  FILE *fe = nullptr, *fl = nullptr;
  long long in_batch = 0, batches_in_file = 0, total = 0;
  std::vector<char> first_ex, first_lab;        // first batch, for refilling the tail
  bool open_next() {
    if (fe) fclose(fe); if (fl) fclose(fl);
    m.partitions++;
    fe = fopen((m.examples + "." + std::to_string(m.partitions)).c_str(), "wb");
    fl = fopen((m.labels + "." + std::to_string(m.partitions)).c_str(), "wb");
    batches_in_file = 0;
    return fe && fl;
  }
  void pad() {
    static const char zeros[4096] = {0};
    for (long long r = m.example_pad; r > 0; r -= 4096) fwrite(zeros, 1, (size_t)(r < 4096 ? r : 4096), fe);
    for (long long r = m.label_pad; r > 0; r -= 4096) fwrite(zeros, 1, (size_t)(r < 4096 ? r : 4096), fl);
  }
  bool append(const char* ex, const char* lab) {
    if (!fe && !open_next()) return false;
    if (in_batch == 0 && batches_in_file >= m.batches_per_partition && !open_next()) return false;
    fwrite(ex, 1, (size_t)m.example_bytes(), fe);
    fwrite(lab, 1, (size_t)m.label_bytes(), fl);
    if ((long long)first_ex.size() < m.batch * m.example_bytes()) { first_ex.insert(first_ex.end(), ex, ex + m.example_bytes()); first_lab.insert(first_lab.end(), lab, lab + m.label_bytes()); }
    ++total;
    if (++in_batch == m.batch) { pad(); in_batch = 0; ++batches_in_file; }
    return true;
  }
  bool close() {
    // refill the last batch with the first tuples of the data set
    long long i = 0;
    while (in_batch != 0) {
      if (!append(first_ex.data() + i * m.example_bytes(), first_lab.data() + i * m.label_bytes())) return false;
      ++i;
    }
    if (fe) fclose(fe); if (fl) fclose(fl);
    fe = fl = nullptr;
    m.elements = total;
    return meta_store(meta_path.c_str(), m);
  }
};

// ---- mapped partitions -------------------------------------------------------------------------------------------------
struct Mapped { char* base = nullptr; size_t bytes = 0; int fd = -1; };
static bool map_file(const std::string& path, Mapped& mp) {
  mp.fd = open(path.c_str(), O_RDONLY);
  if (mp.fd < 0) return false;
  struct stat st;
  if (fstat(mp.fd, &st) != 0) return false;
  mp.bytes = (size_t)st.st_size;
  mp.base = (char*)mmap(nullptr, mp.bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE, mp.fd, 0);
  return mp.base != MAP_FAILED;
}
static void unmap_file(Mapped& mp) {
  if (mp.base && mp.base != MAP_FAILED) munmap(mp.base, mp.bytes);
  if (mp.fd >= 0) close(mp.fd);
  mp.base = nullptr; mp.fd = -1;
}

typedef int (*RegisterFn)(void* ptr, size_t bytes);

struct Basic {
  Meta m;
  std::vector<Mapped> ex, lab;
  std::vector<long long> first_batch;           // first global batch index of each partition
  std::vector<std::atomic<int>> state;          // 0 out, 1 sliding in, 2 resident
  int window;
  RegisterFn reg = nullptr, unreg = nullptr;
  std::atomic<long long> lo{0};                 // first partition of the window
  std::atomic<bool> running{true};
  std::thread handler;
  std::atomic<long long> pinned_bytes{0};
  Basic(int parts) : state(parts) { for (auto& s : state) s.store(0); }
  void slide_in(int p) {
    int expect = 0;
    if (!state[p].compare_exchange_strong(expect, 1)) return;
    for (Mapped* mp : {&ex[p], &lab[p]}) {
      madvise(mp->base, mp->bytes, MADV_WILLNEED);
      madvise(mp->base, mp->bytes, MADV_SEQUENTIAL);
      mlock(mp->base, mp->bytes);               // best effort (RLIMIT_MEMLOCK may be small)
      if (reg) reg(mp->base, mp->bytes);
      pinned_bytes.fetch_add((long long)mp->bytes);
    }
    state[p].store(2, std::memory_order_release);
  }
  void slide_out(int p) {
    int expect = 2;
    if (!state[p].compare_exchange_strong(expect, 1)) return;
    for (Mapped* mp : {&ex[p], &lab[p]}) {
      if (unreg) unreg(mp->base, mp->bytes);
      munlock(mp->base, mp->bytes);
      madvise(mp->base, mp->bytes, MADV_DONTNEED);
      pinned_bytes.fetch_sub((long long)mp->bytes);
    }
    state[p].store(0, std::memory_order_release);
  }
  void handler_loop() {
    unsigned spins = 0;
    const int P = (int)ex.size();
    while (running.load()) {
      long long l = lo.load();
      bool did = false;
      for (int i = 0; i < P; ++i) {
        // window is circular: partitions l, l+1, ... l+window-1 (mod P)
        long long d = ((i - l) % P + P) % P;
        bool inside = d < window;
        int st = state[i].load();
        if (inside && st == 0) { slide_in(i); did = true; }
        else if (!inside && st == 2) { slide_out(i); did = true; }
      }
      if (!did) cpu_relax(++spins); else spins = 0;
    }
  }
  // host addresses of global batch b (wraps around the data set)
  int batch(long long b, const void** e, const void** l, double timeout_s) {
    const long long nb = m.batches();
    b %= nb;
    int p = (int)(std::upper_bound(first_batch.begin(), first_batch.end(), b) - first_batch.begin()) - 1;
    // advance the window so that p is its first partition once the task stream has moved on
    long long cur = lo.load();
    const int P = (int)ex.size();
    long long d = ((p - cur) % P + P) % P;
    if (d >= window) lo.store(p); else if (d > 0 && d >= window / 2) lo.store((cur + 1) % P);
    auto t0 = Clock::now(); unsigned spins = 0;
    while (state[p].load(std::memory_order_acquire) != 2) {
      cpu_relax(++spins);
      if (seconds_since(t0) > timeout_s) return -1;
    }
    long long i = b - first_batch[p];
    *e = ex[p].base + i * m.batch_example_bytes();
    *l = lab[p].base + i * m.batch_label_bytes();
    return 0;
  }
};

// ---- light-weight ring ---------------------------------------------------------------------------------------------------
struct Light {
  Meta m;
  std::vector<Mapped> ex, lab;
  std::vector<long long> first_batch;
  int nslots;
  char* ring_ex = nullptr; char* ring_lab = nullptr;
  size_t slot_ex, slot_lab;
  struct alignas(64) Slot { std::atomic<int> state; long long batch; };
  std::vector<Slot> slots;
  std::atomic<long long> next_fill{0};          // next global batch to be prefetched
  std::atomic<long long> next_take{0};
  std::atomic<bool> running{true};
  std::vector<std::thread> copiers;
  explicit Light(int n) : nslots(n), slots(n) { for (auto& s : slots) { s.state.store(0); s.batch = -1; } }
  void copy_batch(long long b, int slot) {
    const long long nb = m.batches();
    b %= nb;
    int p = (int)(std::upper_bound(first_batch.begin(), first_batch.end(), b) - first_batch.begin()) - 1;
    long long i = b - first_batch[p];
    memcpy(ring_ex + (size_t)slot * slot_ex, ex[p].base + i * m.batch_example_bytes(), (size_t)(m.batch * m.example_bytes()));
    memcpy(ring_lab + (size_t)slot * slot_lab, lab[p].base + i * m.batch_label_bytes(), (size_t)(m.batch * m.label_bytes()));
    madvise(ex[p].base + i * m.batch_example_bytes() / page_size() * page_size(), (size_t)m.batch_example_bytes(), MADV_DONTNEED);
  }
  void copier_loop() {
    unsigned spins = 0;
    while (running.load()) {
      long long b = next_fill.load();
      int slot = (int)(b % nslots);
      int expect = 0;
      // batch b always lives in slot b % nslots: reserve it (0 -> 1) if it is free and nobody else took batch b
      if (slots[slot].state.load() == 0 && next_fill.compare_exchange_strong(b, b + 1)) {
        if (!slots[slot].state.compare_exchange_strong(expect, 1)) { continue; }
        slots[slot].state.store(2);
        copy_batch(b, slot);
        slots[slot].batch = b;
        slots[slot].state.store(3, std::memory_order_release);
        spins = 0;
      } else cpu_relax(++spins);
    }
  }
  int take(long long b, const void** e, const void** l, double timeout_s) {
    int slot = (int)(b % nslots);
    auto t0 = Clock::now(); unsigned spins = 0;
    for (;;) {
      int expect = 3;
      if (slots[slot].batch == b && slots[slot].state.compare_exchange_strong(expect, 4)) break;
      cpu_relax(++spins);
      if (seconds_since(t0) > timeout_s) return -1;
    }
    *e = ring_ex + (size_t)slot * slot_ex;
    *l = ring_lab + (size_t)slot * slot_lab;
    return slot;
  }
  void release(int slot) { slots[slot].batch = -1; slots[slot].state.store(0, std::memory_order_release); }
};

static bool open_partitions(const Meta& m, std::vector<Mapped>& ex, std::vector<Mapped>& lab, std::vector<long long>& first_batch) {
  ex.resize((size_t)m.partitions); lab.resize((size_t)m.partitions);
  long long b = 0;
  for (long long p = 0; p < m.partitions; ++p) {
    if (!map_file(m.examples + "." + std::to_string(p + 1), ex[p])) return false;
    if (!map_file(m.labels + "." + std::to_string(p + 1), lab[p])) return false;
    first_batch.push_back(b);
    b += (long long)(ex[p].bytes / (size_t)m.batch_example_bytes());
  }
  return b >= m.batches();
}

}  // namespace xb

using namespace xb;

// ---- C ABI --------------------------------------------------------------------------------------------------------------
RT_API void* ds_meta_load(const char* path) { Meta* m = new Meta(); if (!meta_load(path, *m)) { delete m; return nullptr; } return m; }
RT_API void ds_meta_free(void* m) { delete (Meta*)m; }
RT_API long long ds_meta_get(void* mp, int what) {
  Meta* m = (Meta*)mp;
  switch (what) {
    case 0: return m->partitions; case 1: return m->elements; case 2: return m->batch; case 3: return m->example_bytes();
    case 4: return m->label_bytes(); case 5: return m->example_pad; case 6: return m->label_pad; case 7: return (long long)m->example_shape.size();
    case 8: return m->batches(); case 9: return m->batch_example_bytes(); case 10: return m->batch_label_bytes();
  }
  return -1;
}
RT_API long long ds_meta_shape(void* mp, int i) { Meta* m = (Meta*)mp; return i < (int)m->example_shape.size() ? m->example_shape[i] : -1; }

// pad_to_page: every batch starts on a page boundary (needed to lock / register batches individually)
RT_API void* ds_writer_create(const char* meta_path, const char* examples_prefix, const char* labels_prefix, long long batch, const long long* example_shape,
                              int example_dims, long long partition_bytes, int pad_to_page) {
  Writer* w = new Writer();
  w->meta_path = meta_path; w->m.examples = examples_prefix; w->m.labels = labels_prefix; w->m.batch = batch;
  w->m.example_shape.assign(example_shape, example_shape + example_dims); w->m.label_shape = {1};
  long long eb = batch * w->m.example_bytes(), lb = batch * w->m.label_bytes();
  if (pad_to_page) { w->m.example_pad = (long long)round_up((size_t)eb, page_size()) - eb; w->m.label_pad = (long long)round_up((size_t)lb, page_size()) - lb; }
  long long per = partition_bytes / (eb + w->m.example_pad);
  w->m.batches_per_partition = per < 1 ? 1 : per;
  w->partition_bytes = partition_bytes;
  return w;
}
RT_API int ds_writer_append(void* w, const void* examples, const void* labels, long long count) {
  Writer* wr = (Writer*)w;
  for (long long i = 0; i < count; ++i)
    if (!wr->append((const char*)examples + i * wr->m.example_bytes(), (const char*)labels + i * wr->m.label_bytes())) return -1;
  return 0;
}
RT_API int ds_writer_close(void* w) { Writer* wr = (Writer*)w; int ok = wr->close() ? 0 : -1; delete wr; return ok; }

RT_API void* ds_basic_open(const char* meta_path, int window, void* register_fn, void* unregister_fn) {
  Meta m;
  if (!meta_load(meta_path, m)) return nullptr;
  Basic* d = new Basic((int)m.partitions);
  d->m = m; d->window = window < 1 ? 1 : window; d->reg = (RegisterFn)register_fn; d->unreg = (RegisterFn)unregister_fn;
  if (!open_partitions(m, d->ex, d->lab, d->first_batch)) { delete d; return nullptr; }
  d->handler = std::thread([d] { d->handler_loop(); });
  return d;
}
RT_API int ds_basic_batch(void* d, long long b, const void** e, const void** l, double timeout_s) { return ((Basic*)d)->batch(b, e, l, timeout_s); }
RT_API long long ds_basic_resident_bytes(void* d) { return ((Basic*)d)->pinned_bytes.load(); }
RT_API int ds_basic_resident_partitions(void* d) { int c = 0; for (auto& s : ((Basic*)d)->state) c += s.load() == 2; return c; }
RT_API void ds_basic_close(void* dp) {
  Basic* d = (Basic*)dp;
  d->running.store(false);
  if (d->handler.joinable()) d->handler.join();
  for (size_t p = 0; p < d->ex.size(); ++p) { if (d->state[p].load() == 2) d->slide_out((int)p); unmap_file(d->ex[p]); unmap_file(d->lab[p]); }
  delete d;
}

RT_API void* ds_light_open(const char* meta_path, int slots, int copiers) {
  Meta m;
  if (!meta_load(meta_path, m) || slots < 2) return nullptr;
  Light* d = new Light(slots);
  d->m = m;
  if (!open_partitions(m, d->ex, d->lab, d->first_batch)) { delete d; return nullptr; }
  d->slot_ex = round_up((size_t)(m.batch * m.example_bytes()), page_size());
  d->slot_lab = round_up((size_t)(m.batch * m.label_bytes()), page_size());
  if (posix_memalign((void**)&d->ring_ex, page_size(), d->slot_ex * slots) || posix_memalign((void**)&d->ring_lab, page_size(), d->slot_lab * slots)) { delete d; return nullptr; }
  mlock(d->ring_ex, d->slot_ex * slots); mlock(d->ring_lab, d->slot_lab * slots);
  for (int i = 0; i < (copiers < 1 ? 1 : copiers); ++i) d->copiers.emplace_back([d] { d->copier_loop(); });
  return d;
}
RT_API void* ds_light_ring(void* d, int which, long long* bytes) {
  Light* l = (Light*)d;
  *bytes = (long long)((which == 0 ? l->slot_ex : l->slot_lab) * l->nslots);
  return which == 0 ? l->ring_ex : l->ring_lab;
}
RT_API int ds_light_take(void* d, long long b, const void** e, const void** l, double timeout_s) { return ((Light*)d)->take(b, e, l, timeout_s); }
RT_API void ds_light_release(void* d, int slot) { ((Light*)d)->release(slot); }
RT_API void ds_light_close(void* dp) {
  Light* d = (Light*)dp;
  d->running.store(false);
  for (auto& t : d->copiers) if (t.joinable()) t.join();
  for (size_t p = 0; p < d->ex.size(); ++p) { unmap_file(d->ex[p]); unmap_file(d->lab[p]); }
  free(d->ring_ex); free(d->ring_lab);
  delete d;
}

// ---- adapters with the host runtime's data-source signature (task -> batch = task*stride + offset) ---------------------
struct DsSource { void* ds; int kind; long long stride, offset; double timeout_s; };
RT_API void* ds_source_create(void* ds, int kind /*0 basic, 1 light*/, long long stride, long long offset, double timeout_s) {
  return new DsSource{ds, kind, stride, offset, timeout_s};
}
RT_API void ds_source_free(void* s) { delete (DsSource*)s; }
RT_API int ds_source_take(void* sp, unsigned long long task, int phase, const void** e, const void** l) {
  (void)phase;
  DsSource* s = (DsSource*)sp;
  long long b = (long long)task * s->stride + s->offset;
  if (s->kind == 0) return ((Basic*)s->ds)->batch(b, e, l, s->timeout_s) == 0 ? 0 : -1;
  return ((Light*)s->ds)->take(b, e, l, s->timeout_s);
}
RT_API void ds_source_release(void* sp, int slot) {
  DsSource* s = (DsSource*)sp;
  if (s->kind == 1) ((Light*)s->ds)->release(slot);
}
