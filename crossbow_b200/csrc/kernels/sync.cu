// Fused model synchronisation: ONE kernel per GPU per clock.
//
// What the reference does with ~4k+6 cuBLAS launches, two cudaDeviceSynchronize and an ncclAllReduce per clock
// (clib-multigpu/synch/sma.c:13-231, synch/common.c:3-57, synch/synchronoussgd.c:13-110) happens here in a single
// persistent kernel per GPU:
//
//   phase 1 (local)   per 16 KB chunk: reduce the k replicas of this GPU against the central average model z,
//                     correct every replica in place, and PUSH the partial sum over NVLink into the inbox of the
//                     GPU(s) that need it (all peers: one-shot; the chunk's owner: two-shot), then raise a flag there.
//   phase 2 (owner)   two-shot only: the owner of a chunk waits for all partials, adds them in rank order and pushes
//                     the total into every GPU's result buffer, then raises the second flag.
//   phase 3 (update)  wait for the chunk's total (one-shot: for all partials, summed locally in rank order, so every
//                     GPU gets bit-identical z), apply momentum to the total, update z, optionally overwrite replicas.
// Owner-apply (two-shot, when every GPU's central model lives in peer-visible memory): the owner of a chunk also applies
// momentum and the update and stores the NEW z straight into every GPU's central model, so phase 3 shrinks to waiting for
// the flags (plus the replica overwrite where the algorithm asks for one).  That is 12 -> 7.4 passes over the vector per
// GPU at 8 GPUs.  The momentum buffer of the central model is then only maintained for the chunks a GPU owns.
//
// Transport is plain st.global on peer-mapped pointers plus st.release.sys / ld.acquire.sys flags; no TMA and no
// cluster multicast anywhere in this file.  Flags carry the synchronisation epoch, so nothing is ever reset, and the
// data buffers are double-buffered by epoch parity.  All blocks of a launch are resident at once (grid <= SM count;
// the multi-rank-on-one-GPU test entry uses a cooperative launch) because blocks wait on other GPUs' blocks.
// Every wait is bounded by a wall-clock limit: on expiry the kernel records XB_TIMEOUT_FLAG in `status`, skips the
// chunk's update and carries on to the end, so the context stays usable and the host can raise an error.
//
// Early release (model averaging without a replica overwrite): a replica's weights are final as soon as phase 1 has
// corrected them - phases 2 and 3 only touch the central model.  The last block of a GPU to finish phase 1 therefore
// stores the epoch into a RELEASE word, and the learners' streams wait for that word (a stream memory operation), not
// for the end of the kernel: the replicas' next forward pass runs under the exchange and the central update, and a
// learner never waits for another GPU.  The reference gets the same overlap by recording each replica's `updated`
// event right after its correction, before the all-reduce is issued (clib-multigpu/synch/sma.c:108-118, :130).
// NVLS variant (two-shot with owner-apply, optional): the partial sums stay in each GPU's own memory, which is bound to an
// NVLink multicast object; the owner of a chunk reads the SUM of all GPUs' partials with one multimem.ld_reduce per 16
// bytes (the switch fetches and adds the eight copies) and stores the new central model into every GPU with one
// multimem.st.  That moves about 4n (1 + 1/G) bytes per direction per GPU instead of the (G-1)/G * 4n of pushed partials
// plus (G-1)/G * 4n of unicast stores of the peer-store path, and the adds happen in the switch.  These are multimem instructions on multicast ADDRESSES; no TMA is involved.
// The variant is a kernel of its own (fused_sync_nvls_kernel) whose blocks interleave local and owner reductions.
// The kernel also keeps a small time line per GPU (%globaltimer at entry, at the release and at the exit of its last
// block, plus running sums), which is what the benchmarks report as synchronisation time per step.
#include "common.cuh"
#include <cuda.h>
#include <string.h>

namespace {

constexpr int CHUNK_SMALL = 4096;    // floats per chunk: 16 KB for latency-bound (small) vectors,
constexpr int CHUNK_LARGE = 32768;   // 128 KB for bandwidth-bound ones (fewer system fences and flag round trips: 25.6 M floats,
                                     // one replica: 318 -> 248 us on 2 GPUs and 360 -> 320 us on 8 against 64 KB chunks; 256 KB
                                     // chunks gain a little more on 2 GPUs and lose on 8, where an owner then has too few)
constexpr long long LARGE_N = 4LL << 20;
constexpr int NT = 256;
constexpr int MAXK = 16, MAXG = 8;

enum Algo : int { ALGO_SMA = 0, ALGO_SSGD = 1, ALGO_POLYAK = 2 };

struct SyncArgs {
  int rank, G, k, algo;
  long long n;                 // elements (multiple of 4)
  int nchunks;
  int chunk;                   // floats per chunk (multiple of 4*U*NT)
  unsigned int epoch;          // >= 1, increases by one per call
  int two_shot;
  int copy_to_replicas;        // overwrite replicas with z at the end
  int use_prev;                // SMA: difference against the pre-update snapshot (1) or current weights (0)
  float alpha, mu, scale;      // scale: 1/wpc (S-SGD), 1/(k*G) (Polyak), unused (SMA)
  float blend;                 // Polyak: running-average factor
  float* w[MAXK];
  const float* prev[MAXK];
  float* z; float* zlast; float* gacc;
  float* inbox[MAXG];          // inbox base of every GPU (index = destination GPU)
  float* result[MAXG];         // two-shot result buffer of every GPU
  float* zpeer[MAXG];          // owner-apply: every GPU's central model (index = GPU), else null
  int owner_apply;
  unsigned int* ready1[MAXG];  // [G][nchunks] on every GPU: partial of (src, chunk) has landed
  unsigned int* ready2[MAXG];  // [nchunks] on every GPU: total of chunk has landed
  int* status;
  unsigned long long timeout_ns;
  // NVLS variant: this GPU's partial buffer (2 x n floats, by epoch parity), the multicast address of the same buffer on
  // all GPUs, and the multicast address of every GPU's central model; all null when the variant is off
  float* part_local; const float* part_mc; float* z_mc;
  unsigned int* release;       // [0] release word (epoch once every replica of this GPU is corrected), [1] block counter; may be null
  unsigned long long* stamps;  // time line, see XB_SYNC_STAMP_*; may be null
};

// Layout of the time line (64-bit words).  ENTRY / RELEASE / EXIT[epoch & 1] describe the most recent launch (the exit
// stamp is the maximum over the blocks; two slots by epoch parity, so an early block of the next launch cannot disturb
// it); COUNT, SUM_RELEASE and SUM_TOTAL accumulate (entry -> release) and (entry -> exit) nanoseconds of the launches
// BEFORE the most recent one.
enum { XB_SYNC_STAMP_ENTRY = 0, XB_SYNC_STAMP_RELEASE = 1, XB_SYNC_STAMP_EXIT = 2 /* and 3 */, XB_SYNC_STAMP_COUNT = 4,
       XB_SYNC_STAMP_SUM_RELEASE = 5, XB_SYNC_STAMP_SUM_TOTAL = 6, XB_SYNC_STAMP_WORDS = 8 };

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait until *p >= epoch (wrap-safe). Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int epoch, unsigned long long timeout_ns) {
  if ((int)(ld_acquire_sys(p) - epoch) >= 0) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if ((int)(ld_acquire_sys(p) - epoch) >= 0) return true;
      __nanosleep(64);
    }
    if (global_ns() - t0 > timeout_ns) return false;
  }
}

// sum over all GPUs of the multicast group of the 16 bytes at `mc` (in-switch reduction)
__device__ __forceinline__ float4 multimem_ld_reduce_add(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
// the same 16 bytes stored into every GPU of the multicast group
__device__ __forceinline__ void multimem_st(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ float4 f4add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 f4axpy(float s, float4 a, float4 b) { return make_float4(fmaf(s, a.x, b.x), fmaf(s, a.y, b.y), fmaf(s, a.z, b.z), fmaf(s, a.w, b.w)); }
__device__ __forceinline__ float4 f4sub(float4 a, float4 b) { return make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
__device__ __forceinline__ float4 f4scale(float s, float4 a) { return make_float4(s * a.x, s * a.y, s * a.z, s * a.w); }

// The element loops below handle U float4 lanes per thread and iteration (lanes j, j+NT, ...): all loads of a step are
// issued before the first dependent store, so every thread keeps 2U..3U 16-byte loads in flight - a plain one-lane loop
// leaves the memory system half idle because the compiler may not move loads across the stores to possibly aliasing
// pointers.
constexpr int U = 4;

// local reduction of U float4 lanes + in-place replica correction; lanes with ok[u] == false are skipped
__device__ __forceinline__ void local_part(const SyncArgs& a, const long long (&i4)[U], const bool (&ok)[U], float4 (&acc)[U]) {
#pragma unroll
  for (int u = 0; u < U; ++u) acc[u] = make_float4(0, 0, 0, 0);
  if (a.algo == ALGO_SMA) {
    float4 z[U];
#pragma unroll
    for (int u = 0; u < U; ++u) if (ok[u]) z[u] = reinterpret_cast<const float4*>(a.z)[i4[u]];
    for (int r = 0; r < a.k; ++r) {
      float4* wp = reinterpret_cast<float4*>(a.w[r]);
      const float4* pp = reinterpret_cast<const float4*>(a.prev[r]);
      float4 w[U], src[U];
#pragma unroll
      for (int u = 0; u < U; ++u) if (ok[u]) w[u] = wp[i4[u]];
      if (a.use_prev) {
#pragma unroll
        for (int u = 0; u < U; ++u) if (ok[u]) src[u] = pp[i4[u]];
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) src[u] = w[u];
      }
#pragma unroll
      for (int u = 0; u < U; ++u) if (ok[u]) {
        const float4 d = f4scale(a.alpha, f4sub(src[u], z[u]));
        wp[i4[u]] = f4sub(w[u], d);
        acc[u] = f4add(acc[u], d);
      }
    }
  } else if (a.algo == ALGO_SSGD) {
    float4* gp = reinterpret_cast<float4*>(a.gacc);
#pragma unroll
    for (int u = 0; u < U; ++u) if (ok[u]) acc[u] = gp[i4[u]];
#pragma unroll
    for (int u = 0; u < U; ++u) if (ok[u]) gp[i4[u]] = make_float4(0, 0, 0, 0);
  } else {  // ALGO_POLYAK: sum of replicas
    for (int r = 0; r < a.k; ++r) {
      const float4* wp = reinterpret_cast<const float4*>(a.w[r]);
#pragma unroll
      for (int u = 0; u < U; ++u) if (ok[u]) acc[u] = f4add(acc[u], wp[i4[u]]);
    }
  }
}

// apply the all-reduced values D to z (and replicas)
__device__ __forceinline__ void apply_total(const SyncArgs& a, const long long (&i4)[U], const bool (&ok)[U], float4 (&D)[U]) {
  float4* zp = reinterpret_cast<float4*>(a.z);
  float4 z[U];
#pragma unroll
  for (int u = 0; u < U; ++u) if (ok[u]) z[u] = zp[i4[u]];
  if (a.algo == ALGO_POLYAK) {
#pragma unroll
    for (int u = 0; u < U; ++u) if (ok[u]) {
      const float4 mean = f4scale(a.scale, D[u]);
      z[u] = make_float4(z[u].x + a.blend * (mean.x - z[u].x), z[u].y + a.blend * (mean.y - z[u].y), z[u].z + a.blend * (mean.z - z[u].z),
                         z[u].w + a.blend * (mean.w - z[u].w));
      zp[i4[u]] = z[u];
    }
    if (a.alpha > 0.f)
      for (int r = 0; r < a.k; ++r) {
        float4* wp = reinterpret_cast<float4*>(a.w[r]);
        float4 w[U];
#pragma unroll
        for (int u = 0; u < U; ++u) if (ok[u]) w[u] = wp[i4[u]];
#pragma unroll
        for (int u = 0; u < U; ++u) if (ok[u]) wp[i4[u]] = f4sub(w[u], f4scale(a.alpha, f4sub(w[u], z[u])));
      }
    return;
  }
  if (a.algo == ALGO_SSGD) {
#pragma unroll
    for (int u = 0; u < U; ++u) D[u] = f4scale(a.scale, D[u]);
  }
  if (a.mu > 0.f) {
    float4* lp = reinterpret_cast<float4*>(a.zlast);
    float4 l[U];
#pragma unroll
    for (int u = 0; u < U; ++u) if (ok[u]) l[u] = lp[i4[u]];
#pragma unroll
    for (int u = 0; u < U; ++u) if (ok[u]) { D[u] = f4axpy(a.mu, l[u], D[u]); lp[i4[u]] = D[u]; }
  }
#pragma unroll
  for (int u = 0; u < U; ++u) if (ok[u]) { z[u] = f4add(z[u], D[u]); zp[i4[u]] = z[u]; }
  if (a.copy_to_replicas || a.algo == ALGO_SSGD)
    for (int r = 0; r < a.k; ++r) {
      float4* wp = reinterpret_cast<float4*>(a.w[r]);
#pragma unroll
      for (int u = 0; u < U; ++u) if (ok[u]) wp[i4[u]] = z[u];
    }
}

// Called by every block once its share of phase 1 is done (all threads; contains a block barrier).  The last block of
// the rank to arrive publishes the epoch in the release word: every replica of this GPU then holds its corrected weights.
__device__ __forceinline__ void release_replicas(const SyncArgs& a) {
  if (!a.release) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int arrived = atomicAdd(a.release + 1, 1u) + 1u;
    if (arrived == gridDim.x) {
      a.release[1] = 0;                                   // launches on one stream do not overlap: ready for the next one
      if (a.stamps) a.stamps[XB_SYNC_STAMP_RELEASE] = global_ns();
      __threadfence();
      st_release_sys(a.release, a.epoch);
    }
  }
}
__device__ __forceinline__ void stamp_entry(const SyncArgs& a) {
  if (!a.stamps || blockIdx.x != 0 || threadIdx.x != 0) return;
  unsigned long long* s = a.stamps;
  const unsigned long long e0 = s[XB_SYNC_STAMP_ENTRY], r0 = s[XB_SYNC_STAMP_RELEASE], x0 = s[XB_SYNC_STAMP_EXIT + ((a.epoch - 1) & 1)];
  if (e0 && x0 >= e0) {                                   // fold the previous launch into the running sums
    s[XB_SYNC_STAMP_COUNT] += 1;
    s[XB_SYNC_STAMP_SUM_RELEASE] += (r0 >= e0 ? r0 : x0) - e0;
    s[XB_SYNC_STAMP_SUM_TOTAL] += x0 - e0;
  }
  s[XB_SYNC_STAMP_ENTRY] = global_ns();
  s[XB_SYNC_STAMP_RELEASE] = 0;
}
__device__ __forceinline__ void stamp_exit(const SyncArgs& a) {
  if (a.stamps && threadIdx.x == 0) atomicMax(a.stamps + XB_SYNC_STAMP_EXIT + (a.epoch & 1), global_ns());
}

__global__ void __launch_bounds__(NT, 2) fused_sync_kernel(const SyncArgs* __restrict__ per_rank) {
  // the argument block is read thousands of times (pointer tables): keep a copy in shared memory
  __shared__ SyncArgs a;
  __shared__ int s_fail;
  {
    const int* src = reinterpret_cast<const int*>(per_rank + blockIdx.y);
    int* dst = reinterpret_cast<int*>(&a);
    for (int i = threadIdx.x; i < (int)(sizeof(SyncArgs) / sizeof(int)); i += NT) dst[i] = src[i];
  }
  __syncthreads();
  const int CHUNK = a.chunk;
  const int tid = threadIdx.x, B = gridDim.x, G = a.G, me = a.rank;
  const long long n4 = a.n / 4;
  const int parity = a.epoch & 1;
  stamp_entry(a);

  if (G == 1) {   // no exchange: one pass
    for (int c = blockIdx.x; c < a.nchunks; c += B)
      for (int j0 = tid; j0 < CHUNK / 4; j0 += U * NT) {
        long long i4[U]; bool ok[U]; float4 acc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { i4[u] = (long long)c * (CHUNK / 4) + j0 + u * NT; ok[u] = i4[u] < n4; }
        local_part(a, i4, ok, acc);
        apply_total(a, i4, ok, acc);
      }
    release_replicas(a);
    stamp_exit(a);
    return;
  }

  const int owned_slots = (a.nchunks + G - 1) / G;
  const long long slot_elems = (long long)(a.two_shot ? owned_slots : a.nchunks) * CHUNK;

  // ---- phase 1: local reduce, replica correction, push partials -------------------------------------------
  for (int c = blockIdx.x; c < a.nchunks; c += B) {
    const int owner = c % G;
    const long long dst_chunk = a.two_shot ? (c / G) : c;
    const long long off4 = (((long long)parity * G + me) * slot_elems + dst_chunk * CHUNK) / 4;
    for (int j0 = tid; j0 < CHUNK / 4; j0 += U * NT) {
      long long i4[U]; bool ok[U]; float4 acc[U];
#pragma unroll
      for (int u = 0; u < U; ++u) { i4[u] = (long long)c * (CHUNK / 4) + j0 + u * NT; ok[u] = i4[u] < n4; }
      local_part(a, i4, ok, acc);                         // (lanes past the end contribute zeros)
      if (a.two_shot) {
#pragma unroll
        for (int u = 0; u < U; ++u) reinterpret_cast<float4*>(a.inbox[owner])[off4 + j0 + u * NT] = acc[u];
      } else {
        for (int g = 0; g < G; ++g) {
#pragma unroll
          for (int u = 0; u < U; ++u) reinterpret_cast<float4*>(a.inbox[g])[off4 + j0 + u * NT] = acc[u];
        }
      }
    }
    __syncthreads();
    if (a.two_shot) {
      if (tid == 0) { __threadfence_system(); st_release_sys(a.ready1[owner] + (long long)me * a.nchunks + c, a.epoch); }
    } else if (tid < G) {
      __threadfence_system();
      st_release_sys(a.ready1[tid] + (long long)me * a.nchunks + c, a.epoch);
    }
  }
  // every replica chunk this block is responsible for now holds its corrected weights
  if (!(a.copy_to_replicas || a.algo != ALGO_SMA)) release_replicas(a);

  // ---- phase 2 (two-shot): owners reduce and broadcast the totals -----------------------------------------
  if (a.two_shot) {
    int jb = 0;
    for (int c = me; c < a.nchunks; c += G, ++jb) {
      if (jb % B != (int)blockIdx.x) continue;
      if (tid == 0) s_fail = 0;
      __syncthreads();
      if (tid < G && !wait_flag(a.ready1[me] + (long long)tid * a.nchunks + c, a.epoch, a.timeout_ns)) { s_fail = 1; atomicExch(a.status, XB_TIMEOUT_FLAG); }
      __syncthreads();
      const bool ok = !s_fail;
      const long long res4 = ((long long)parity * a.nchunks + c) * (CHUNK / 4);
      for (int j0 = tid; j0 < CHUNK / 4 && ok; j0 += U * NT) {
        float4 t[U];
#pragma unroll
        for (int u = 0; u < U; ++u) t[u] = make_float4(0, 0, 0, 0);
        for (int src = 0; src < G; ++src) {               // rank order: every owner adds in the same order
          const long long o4 = (((long long)parity * G + src) * slot_elems + (long long)(c / G) * CHUNK) / 4 + j0;
          float4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) v[u] = __ldcg(reinterpret_cast<const float4*>(a.inbox[me]) + o4 + u * NT);
#pragma unroll
          for (int u = 0; u < U; ++u) t[u] = f4add(t[u], v[u]);
        }
        if (!a.owner_apply) {
          for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int u = 0; u < U; ++u) reinterpret_cast<float4*>(a.result[g])[res4 + j0 + u * NT] = t[u];
          }
        } else {
          // this GPU's z is the authoritative copy of the chunks it owns: update it here, store it everywhere
          long long i4[U]; bool okk[U]; float4 z[U];
#pragma unroll
          for (int u = 0; u < U; ++u) { i4[u] = (long long)c * (CHUNK / 4) + j0 + u * NT; okk[u] = i4[u] < n4; }
#pragma unroll
          for (int u = 0; u < U; ++u) if (okk[u]) z[u] = reinterpret_cast<const float4*>(a.z)[i4[u]];
          if (a.algo == ALGO_POLYAK) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const float4 mean = f4scale(a.scale, t[u]);
              z[u] = make_float4(z[u].x + a.blend * (mean.x - z[u].x), z[u].y + a.blend * (mean.y - z[u].y), z[u].z + a.blend * (mean.z - z[u].z),
                                 z[u].w + a.blend * (mean.w - z[u].w));
            }
          } else {
            if (a.algo == ALGO_SSGD) {
#pragma unroll
              for (int u = 0; u < U; ++u) t[u] = f4scale(a.scale, t[u]);
            }
            if (a.mu > 0.f) {
              float4* lp = reinterpret_cast<float4*>(a.zlast);
              float4 l[U];
#pragma unroll
              for (int u = 0; u < U; ++u) if (okk[u]) l[u] = lp[i4[u]];
#pragma unroll
              for (int u = 0; u < U; ++u) if (okk[u]) { t[u] = f4axpy(a.mu, l[u], t[u]); lp[i4[u]] = t[u]; }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) z[u] = f4add(z[u], t[u]);
          }
          for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int u = 0; u < U; ++u) if (okk[u]) reinterpret_cast<float4*>(a.zpeer[g])[i4[u]] = z[u];
          }
        }
      }
      __syncthreads();
      if (ok && tid < G) { __threadfence_system(); st_release_sys(a.ready2[tid] + c, a.epoch); }
    }
  }

  // ---- phase 3: totals -> z (and replicas) ----------------------------------------------------------------
  for (int c = blockIdx.x; c < a.nchunks; c += B) {
    if (tid == 0) s_fail = 0;
    __syncthreads();
    if (a.two_shot) {
      if (tid == 0 && !wait_flag(a.ready2[me] + c, a.epoch, a.timeout_ns)) { s_fail = 1; atomicExch(a.status, XB_TIMEOUT_FLAG); }
    } else if (tid < G) {
      if (!wait_flag(a.ready1[me] + (long long)tid * a.nchunks + c, a.epoch, a.timeout_ns)) { s_fail = 1; atomicExch(a.status, XB_TIMEOUT_FLAG); }
    }
    __syncthreads();
    const bool fail = s_fail != 0;
    __syncthreads();            // everyone has read s_fail before thread 0 may reset it in the next iteration
    if (fail) continue;
    if (a.owner_apply) {
      // z of this chunk is final; only the algorithms that rewrite the replicas from it have work left
      const bool pull = a.algo == ALGO_POLYAK && a.alpha > 0.f;
      if (!(a.copy_to_replicas || a.algo == ALGO_SSGD || pull)) continue;
      for (int j0 = tid; j0 < CHUNK / 4; j0 += U * NT) {
        long long i4[U]; bool ok[U]; float4 z[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { i4[u] = (long long)c * (CHUNK / 4) + j0 + u * NT; ok[u] = i4[u] < n4; }
#pragma unroll
        for (int u = 0; u < U; ++u) if (ok[u]) z[u] = __ldcg(reinterpret_cast<const float4*>(a.z) + i4[u]);
        for (int r = 0; r < a.k; ++r) {
          float4* wp = reinterpret_cast<float4*>(a.w[r]);
          if (pull) {
            float4 w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) if (ok[u]) w[u] = wp[i4[u]];
#pragma unroll
            for (int u = 0; u < U; ++u) if (ok[u]) wp[i4[u]] = f4sub(w[u], f4scale(a.alpha, f4sub(w[u], z[u])));
          } else {
#pragma unroll
            for (int u = 0; u < U; ++u) if (ok[u]) wp[i4[u]] = z[u];
          }
        }
      }
      __syncthreads();
      continue;
    }
    for (int j0 = tid; j0 < CHUNK / 4; j0 += U * NT) {
      long long i4[U]; bool ok[U]; float4 D[U];
#pragma unroll
      for (int u = 0; u < U; ++u) { i4[u] = (long long)c * (CHUNK / 4) + j0 + u * NT; ok[u] = i4[u] < n4; D[u] = make_float4(0, 0, 0, 0); }
      if (a.two_shot) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (ok[u]) D[u] = __ldcg(reinterpret_cast<const float4*>(a.result[me]) + ((long long)parity * a.nchunks + c) * (CHUNK / 4) + j0 + u * NT);
      } else {
        for (int src = 0; src < G; ++src) {
          const long long o4 = (((long long)parity * G + src) * slot_elems + (long long)c * CHUNK) / 4 + j0;
          float4 v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) if (ok[u]) v[u] = __ldcg(reinterpret_cast<const float4*>(a.inbox[me]) + o4 + u * NT);
#pragma unroll
          for (int u = 0; u < U; ++u) if (ok[u]) D[u] = f4add(D[u], v[u]);
        }
      }
      apply_total(a, i4, ok, D);
    }
    __syncthreads();
  }
  // algorithms that rewrite the replicas from the new central model release them only now
  if (a.copy_to_replicas || a.algo != ALGO_SMA) release_replicas(a);
  stamp_exit(a);
}

// The NVLS variant as a kernel of its own.  The partial sums never leave their GPU by a store: the owner of a chunk pulls
// the SUM of all GPUs' copies through the switch (multimem.ld_reduce) and pushes the new central model with multimem.st.
// Run as "all local reductions, then all owner reductions" the links idle during the first half and the HBM during the
// second, so every block interleaves the two: after each chunk of its local reduction it looks whether the next chunk it
// owns has been flagged by every GPU and, if so, reduces it; only when its local work is done does it wait (bounded) for
// the rest.  All GPUs walk the chunks in the same order, so the first owned chunks become ready one wave of local work
// after the start.  No wait sits in front of local work, hence no cycle: every flag a block waits for is raised by work
// that waits for nothing.
__global__ void __launch_bounds__(NT, 2) fused_sync_nvls_kernel(const SyncArgs* __restrict__ per_rank) {
  __shared__ SyncArgs a;
  __shared__ int s_fail;
  {
    const int* src = reinterpret_cast<const int*>(per_rank + blockIdx.y);
    int* dst = reinterpret_cast<int*>(&a);
    for (int i = threadIdx.x; i < (int)(sizeof(SyncArgs) / sizeof(int)); i += NT) dst[i] = src[i];
  }
  __syncthreads();
  const int CHUNK = a.chunk, C4 = CHUNK / 4;
  const int tid = threadIdx.x, B = gridDim.x, G = a.G, me = a.rank;
  const long long n4 = a.n / 4;
  const int parity = a.epoch & 1;
  const bool early = !(a.copy_to_replicas || a.algo != ALGO_SMA);
  stamp_entry(a);

  int c1 = blockIdx.x;          // next chunk of the local reduction
  int j2 = blockIdx.x;          // next of the chunks this GPU owns (chunk me + j2 * G) to reduce across the GPUs
  bool released = false;
  for (;;) {
    const bool more1 = c1 < a.nchunks;
    const int c2 = me + j2 * G;
    const bool more2 = c2 < a.nchunks;
    if (!more1 && !more2) break;
    if (more1) {
      float4* dst = reinterpret_cast<float4*>(a.part_local) + ((long long)parity * a.nchunks + c1) * C4;
      for (int j0 = tid; j0 < C4; j0 += U * NT) {
        long long i4[U]; bool ok[U]; float4 acc[U];
#pragma unroll
        for (int u = 0; u < U; ++u) { i4[u] = (long long)c1 * C4 + j0 + u * NT; ok[u] = i4[u] < n4; }
        local_part(a, i4, ok, acc);                       // (lanes past the end contribute zeros)
#pragma unroll
        for (int u = 0; u < U; ++u) dst[j0 + u * NT] = acc[u];
      }
      __syncthreads();
      if (tid == 0) { __threadfence_system(); st_release_sys(a.ready1[c1 % G] + (long long)me * a.nchunks + c1, a.epoch); }
      c1 += B;
      if (c1 >= a.nchunks && early) { release_replicas(a); released = true; }
    }
    if (more2) {
      const bool must = c1 >= a.nchunks;                  // nothing local left: wait instead of looking
      int ready = 1;
      if (tid < G) {
        const unsigned int* f = a.ready1[me] + (long long)tid * a.nchunks + c2;
        if (must) {
          if (!wait_flag(f, a.epoch, a.timeout_ns)) { ready = 0; atomicExch(a.status, XB_TIMEOUT_FLAG); }
        } else {
          ready = (int)(ld_acquire_sys(f) - a.epoch) >= 0;
        }
      }
      ready = __syncthreads_and(ready);
      if (ready) {
        __threadfence_system();                           // the multimem loads below follow the flags observed above
        const float* mc = a.part_mc + ((long long)parity * a.nchunks + c2) * CHUNK;
        for (int j0 = tid; j0 < C4; j0 += U * NT) {
          float4 t[U], z[U]; long long i4[U]; bool ok[U];
#pragma unroll
          for (int u = 0; u < U; ++u) { i4[u] = (long long)c2 * C4 + j0 + u * NT; ok[u] = i4[u] < n4; }
#pragma unroll
          for (int u = 0; u < U; ++u) t[u] = multimem_ld_reduce_add(mc + 4 * (j0 + u * NT));
#pragma unroll
          for (int u = 0; u < U; ++u) if (ok[u]) z[u] = reinterpret_cast<const float4*>(a.z)[i4[u]];
          if (a.algo == ALGO_POLYAK) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const float4 mean = f4scale(a.scale, t[u]);
              z[u] = make_float4(z[u].x + a.blend * (mean.x - z[u].x), z[u].y + a.blend * (mean.y - z[u].y), z[u].z + a.blend * (mean.z - z[u].z),
                                 z[u].w + a.blend * (mean.w - z[u].w));
            }
          } else {
            if (a.algo == ALGO_SSGD) {
#pragma unroll
              for (int u = 0; u < U; ++u) t[u] = f4scale(a.scale, t[u]);
            }
            if (a.mu > 0.f) {
              float4* lp = reinterpret_cast<float4*>(a.zlast);
              float4 l[U];
#pragma unroll
              for (int u = 0; u < U; ++u) if (ok[u]) l[u] = lp[i4[u]];
#pragma unroll
              for (int u = 0; u < U; ++u) if (ok[u]) { t[u] = f4axpy(a.mu, l[u], t[u]); lp[i4[u]] = t[u]; }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) z[u] = f4add(z[u], t[u]);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) if (ok[u]) multimem_st(a.z_mc + 4 * i4[u], z[u]);
        }
        __syncthreads();
        if (tid < G) { __threadfence_system(); st_release_sys(a.ready2[tid] + c2, a.epoch); }
        j2 += B;
      } else if (must) {
        j2 += B;                                          // gave up on this chunk: the status word says so
      }
    }
  }
  if (early && !released) release_replicas(a);

  // the central model is complete on this GPU once every owner has flagged its chunks
  for (int c = blockIdx.x; c < a.nchunks; c += B) {
    if (tid == 0) s_fail = 0;
    __syncthreads();
    if (tid == 0 && !wait_flag(a.ready2[me] + c, a.epoch, a.timeout_ns)) { s_fail = 1; atomicExch(a.status, XB_TIMEOUT_FLAG); }
    __syncthreads();
    const bool fail = s_fail != 0;
    __syncthreads();            // everyone has read s_fail before thread 0 may reset it in the next iteration
    if (fail) continue;
    const bool pull = a.algo == ALGO_POLYAK && a.alpha > 0.f;
    if (!(a.copy_to_replicas || a.algo == ALGO_SSGD || pull)) continue;
    for (int j0 = tid; j0 < C4; j0 += U * NT) {
      long long i4[U]; bool ok[U]; float4 z[U];
#pragma unroll
      for (int u = 0; u < U; ++u) { i4[u] = (long long)c * C4 + j0 + u * NT; ok[u] = i4[u] < n4; }
#pragma unroll
      for (int u = 0; u < U; ++u) if (ok[u]) z[u] = __ldcg(reinterpret_cast<const float4*>(a.z) + i4[u]);
      for (int r = 0; r < a.k; ++r) {
        float4* wp = reinterpret_cast<float4*>(a.w[r]);
        if (pull) {
          float4 w[U];
#pragma unroll
          for (int u = 0; u < U; ++u) if (ok[u]) w[u] = wp[i4[u]];
#pragma unroll
          for (int u = 0; u < U; ++u) if (ok[u]) wp[i4[u]] = f4sub(w[u], f4scale(a.alpha, f4sub(w[u], z[u])));
        } else {
#pragma unroll
          for (int u = 0; u < U; ++u) if (ok[u]) wp[i4[u]] = z[u];
        }
      }
    }
    __syncthreads();
  }
  if (!early) release_replicas(a);
  stamp_exit(a);
}

// Plain copy with 16-byte accesses: the yardstick for what st.global over NVLink sustains when every GPU pushes to every
// peer at once (the synchronisation micro-benchmark measures the exchange against it).
__global__ void __launch_bounds__(NT) peer_copy_kernel(float4* __restrict__ dst, const float4* __restrict__ src, long long n4) {
  const long long stride = (long long)gridDim.x * NT * U;
  for (long long i0 = (long long)blockIdx.x * NT * U + threadIdx.x; i0 < n4; i0 += stride) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) if (i0 + u * NT < n4) v[u] = src[i0 + u * NT];
#pragma unroll
    for (int u = 0; u < U; ++u) if (i0 + u * NT < n4) dst[i0 + u * NT] = v[u];
  }
}

// The same, to every peer in ONE launch (blockIdx.y = destination): what a GPU can push when all its outgoing traffic is in
// flight at once, as it is in the exchange.
struct PeerCopyAll { float4* dst[MAXG]; const float4* src[MAXG]; long long n4; };
__global__ void __launch_bounds__(NT) peer_copy_all_kernel(PeerCopyAll a) {
  float4* __restrict__ dst = a.dst[blockIdx.y];
  const float4* __restrict__ src = a.src[blockIdx.y];
  const long long stride = (long long)gridDim.x * NT * U;
  for (long long i0 = (long long)blockIdx.x * NT * U + threadIdx.x; i0 < a.n4; i0 += stride) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) if (i0 + u * NT < a.n4) v[u] = src[i0 + u * NT];
#pragma unroll
    for (int u = 0; u < U; ++u) if (i0 + u * NT < a.n4) dst[i0 + u * NT] = v[u];
  }
}

// replicas <- z (DEFAULT update model, and LR-drop copies when no averaging is due)
__global__ void broadcast_z_kernel(const float* __restrict__ z, float* const* w, int k, long long n4) {
  for (long long i = blockIdx.x * (long long)NT + threadIdx.x; i < n4; i += (long long)gridDim.x * NT) {
    float4 v = reinterpret_cast<const float4*>(z)[i];
    for (int r = 0; r < k; ++r) reinterpret_cast<float4*>(w[r])[i] = v;
  }
}

}  // namespace

// Sizes (in floats / words) of the peer-visible buffers a GPU must allocate for vectors of n elements.
// (tuning: floats per chunk of a large vector; a multiple of 4 * U * NT.  Must be the same on every rank and set before the
// buffers of a synchroniser are sized.)
static int g_chunk_large = CHUNK_LARGE;
XB_API void xb_sync_set_large_chunk(int floats) {
  const int unit = 4 * U * NT;
  g_chunk_large = floats >= unit ? floats / unit * unit : CHUNK_LARGE;
}
static inline long long chunk_for(long long n) { return n >= LARGE_N ? g_chunk_large : CHUNK_SMALL; }
XB_API long long xb_sync_chunk(long long n) { return chunk_for(n); }
XB_API long long xb_sync_nchunks(long long n) { return (n + chunk_for(n) - 1) / chunk_for(n); }
XB_API long long xb_sync_inbox_floats(long long n, int G, int two_shot) {
  long long nc = xb_sync_nchunks(n);
  long long slots = two_shot ? (nc + G - 1) / G : nc;
  return 2LL * G * slots * chunk_for(n);
}
XB_API long long xb_sync_result_floats(long long n) { return 2LL * xb_sync_nchunks(n) * chunk_for(n); }
XB_API long long xb_sync_flag_words(long long n, int G) { return (long long)(G + 1) * xb_sync_nchunks(n); }
XB_API int xb_sync_args_size() { return (int)sizeof(SyncArgs); }

// Host-side mirror used by the Python binding to fill SyncArgs without knowing its layout.
struct XbSyncDesc {
  int rank, G, k, algo;
  long long n;
  unsigned int epoch;
  int two_shot, copy_to_replicas, use_prev;
  float alpha, mu, scale, blend;
  float* w[MAXK];
  const float* prev[MAXK];
  float* z; float* zlast; float* gacc;
  float* inbox[MAXG]; float* result[MAXG];
  unsigned int* flags[MAXG];      // per GPU: ready1 [G*nchunks] followed by ready2 [nchunks]
  int* status;
  double timeout_s;
  float* zpeer[MAXG];             // every GPU's central model as seen from this process, or all null
  float* part_local; const float* part_mc; float* z_mc;   // NVLS variant (see SyncArgs), or all null
  unsigned int* release;          // two words owned by the caller (zero-initialised once), or null: see SyncArgs::release
  unsigned long long* stamps;     // XB_SYNC_STAMP_WORDS 64-bit words owned by the caller (zero-initialised once), or null
};

static void fill_args(SyncArgs& a, const XbSyncDesc& d) {
  memset(&a, 0, sizeof(a));
  a.rank = d.rank; a.G = d.G; a.k = d.k; a.algo = d.algo; a.n = d.n; a.nchunks = (int)xb_sync_nchunks(d.n); a.chunk = (int)chunk_for(d.n);
  a.epoch = d.epoch; a.two_shot = d.two_shot; a.copy_to_replicas = d.copy_to_replicas; a.use_prev = d.use_prev;
  a.alpha = d.alpha; a.mu = d.mu; a.scale = d.scale; a.blend = d.blend;
  for (int i = 0; i < MAXK; ++i) { a.w[i] = d.w[i]; a.prev[i] = d.prev[i]; }
  a.z = d.z; a.zlast = d.zlast; a.gacc = d.gacc;
  for (int g = 0; g < MAXG; ++g) {
    a.inbox[g] = d.inbox[g]; a.result[g] = d.result[g];
    a.ready1[g] = d.flags[g];
    a.ready2[g] = d.flags[g] ? d.flags[g] + (long long)d.G * a.nchunks : nullptr;
  }
  a.owner_apply = (d.two_shot && d.G > 1 && d.zpeer[0]) ? 1 : 0;
  for (int g = 0; g < MAXG; ++g) a.zpeer[g] = d.zpeer[g];
  a.status = d.status;
  a.timeout_ns = (unsigned long long)(d.timeout_s * 1e9);
  a.release = d.release; a.stamps = d.stamps;
  const bool nvls = a.owner_apply && d.part_local && d.part_mc && d.z_mc;
  a.part_local = nvls ? d.part_local : nullptr; a.part_mc = nvls ? d.part_mc : nullptr; a.z_mc = nvls ? d.z_mc : nullptr;
}
XB_API long long xb_sync_part_floats(long long n) { return 2LL * xb_sync_nchunks(n) * chunk_for(n); }

static int sync_grid(int nchunks, int max_blocks) {
  int b = nchunks < max_blocks ? nchunks : max_blocks;
  return b < 1 ? 1 : b;
}

// One rank (this process's GPU). `args_dev` is a device buffer of xb_sync_args_size() bytes owned by the caller;
// `args_pinned` a pinned host staging buffer of the same size.
XB_API int xb_fused_sync(const XbSyncDesc* d, void* args_dev, void* args_pinned, int max_blocks, cudaStream_t st) {
  if (d->n % 4 || d->k < 0 || d->k > MAXK || d->G < 1 || d->G > MAXG) return -XB_BAD_ARG;
  SyncArgs* h = reinterpret_cast<SyncArgs*>(args_pinned);
  fill_args(*h, *d);
  XB_CUDA_CHECK(cudaMemcpyAsync(args_dev, h, sizeof(SyncArgs), cudaMemcpyHostToDevice, st));
  if (max_blocks <= 0) {
    // two blocks per SM (one covers the other's fences and flag waits); every block must become resident, because blocks
    // wait on other GPUs' blocks - the learners' kernels running next to this one never wait on it, so they drain
    static int cached = 0;
    if (!cached) {
      int dev = 0, sms = 148, per_sm = 1;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      int per_sm_nvls = 1;
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_sync_kernel, NT, 0);
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_nvls, fused_sync_nvls_kernel, NT, 0);
      cached = sms * ((per_sm >= 2 && per_sm_nvls >= 2) ? 2 : 1);
    }
    max_blocks = cached;
  }
  dim3 grid(sync_grid(h->nchunks, max_blocks), 1);
  if (h->part_mc) fused_sync_nvls_kernel<<<grid, NT, 0, st>>>(reinterpret_cast<const SyncArgs*>(args_dev));
  else fused_sync_kernel<<<grid, NT, 0, st>>>(reinterpret_cast<const SyncArgs*>(args_dev));
  return (int)cudaGetLastError();
}

// G ranks emulated on ONE GPU: a single cooperative launch with gridDim.y = G, so every rank's blocks are resident
// together (separate launches that wait on one another must never share a GPU).
XB_API int xb_fused_sync_emulated(const XbSyncDesc* descs, int G, void* args_dev, int blocks_per_rank, cudaStream_t st) {
  if (G < 1 || G > MAXG) return -XB_BAD_ARG;
  SyncArgs h[MAXG];
  for (int g = 0; g < G; ++g) { if (descs[g].n % 4 || descs[g].k > MAXK) return -XB_BAD_ARG; fill_args(h[g], descs[g]); }
  XB_CUDA_CHECK(cudaMemcpyAsync(args_dev, h, sizeof(SyncArgs) * G, cudaMemcpyHostToDevice, st));
  XB_CUDA_CHECK(cudaStreamSynchronize(st));   // h is on the stack
  int dev = 0, sms = 0, per_sm = 0;
  XB_CUDA_CHECK(cudaGetDevice(&dev));
  XB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  XB_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_sync_kernel, NT, 0));
  int bpr = sync_grid(h[0].nchunks, blocks_per_rank > 0 ? blocks_per_rank : 16);
  while (bpr > 1 && (long long)bpr * G > (long long)sms * per_sm) --bpr;
  dim3 grid(bpr, G);
  const SyncArgs* p = reinterpret_cast<const SyncArgs*>(args_dev);
  void* kargs[] = {(void*)&p};
  XB_CUDA_CHECK(cudaLaunchCooperativeKernel((void*)fused_sync_kernel, grid, dim3(NT), kargs, 0, st));
  return (int)cudaGetLastError();
}

// Make `st` wait (a stream memory operation, no kernel) until the 32-bit word at `word` has reached `value`
// (cyclic comparison).  Used to hold a learner's next task until its replica has been released by the kernel above.
// The driver entry point is looked up at run time, so the library loads on machines without a driver.
typedef CUresult (*StreamWaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
static StreamWaitValue32Fn stream_wait_fn() {
  static StreamWaitValue32Fn fn = nullptr;
  static bool looked = false;
  if (!looked) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (StreamWaitValue32Fn)p;
    looked = true;
  }
  return fn;
}
XB_API int xb_stream_wait_value32(cudaStream_t st, const unsigned int* word, unsigned int value) {
  StreamWaitValue32Fn fn = stream_wait_fn();
  if (!fn) return -XB_BAD_ARG;
  CUresult r = fn((CUstream)st, (CUdeviceptr)word, value, CU_STREAM_WAIT_VALUE_GEQ);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 1000;
}
// 1 when streams of the current device can wait on a memory word (CUDA 12 drivers: the second generation of stream
// memory operations is part of the base feature set)
XB_API int xb_stream_wait_value_supported() {
  int drv = 0;
  if (cudaDriverGetVersion(&drv) != cudaSuccess || drv < 12000) return 0;
  return stream_wait_fn() != nullptr ? 1 : 0;
}
XB_API int xb_sync_stamp_words() { return XB_SYNC_STAMP_WORDS; }

// dst (possibly another GPU's memory) <- src (this GPU's), n floats (multiple of 4), `blocks` CTAs
XB_API int xb_peer_copy(float* dst, const float* src, long long n, int blocks, cudaStream_t st) {
  if (n % 4 || blocks < 1) return -XB_BAD_ARG;
  peer_copy_kernel<<<blocks, NT, 0, st>>>(reinterpret_cast<float4*>(dst), reinterpret_cast<const float4*>(src), n / 4);
  return (int)cudaGetLastError();
}

// dsts[i] <- srcs[i], n floats each (multiple of 4), for i < count <= 8, in one launch of blocks x count CTAs
XB_API int xb_peer_copy_all(float* const* dsts, const float* const* srcs, int count, long long n, int blocks, cudaStream_t st) {
  if (n % 4 || blocks < 1 || count < 1 || count > MAXG) return -XB_BAD_ARG;
  PeerCopyAll a{};
  for (int i = 0; i < count; ++i) { a.dst[i] = reinterpret_cast<float4*>(dsts[i]); a.src[i] = reinterpret_cast<const float4*>(srcs[i]); }
  a.n4 = n / 4;
  peer_copy_all_kernel<<<dim3(blocks, count), NT, 0, st>>>(a);
  return (int)cudaGetLastError();
}

XB_API int xb_broadcast_model(const float* z, float* const* w_dev_array, int k, long long n, cudaStream_t st) {
  if (n % 4) return -XB_BAD_ARG;
  long long n4 = n / 4;
  int blocks = (int)((n4 + NT - 1) / NT); if (blocks > 148 * 8) blocks = 148 * 8; if (blocks < 1) blocks = 1;
  broadcast_z_kernel<<<blocks, NT, 0, st>>>(z, w_dev_array, k, n4);
  return (int)cudaGetLastError();
}
