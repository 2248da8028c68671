// Device program = the flat list of kernel launches one task needs, plus the learner that owns it.
//
// The reference walks its operator list on the host for every task and calls one function pointer per operator,
// each of which issues several library calls (clib-multigpu/executioncontext.c:558-726, taskhandler.c:24-151,
// operator.c:57-60, kernelmap.c:27-50).  Here the graph is lowered ONCE into an array of XbOp records with all
// pointers and shapes resolved; a learner replays it either directly or, normally, as a captured CUDA graph, so a
// task costs one graph launch on the host.  Values that differ between tasks (learning rate, task id, ...) live in a
// per-learner XbTaskParams block that is uploaded by the first node of the program.
#include <nvtx3/nvToolsExt.h>
#include <atomic>
#include <chrono>
#include <mutex>
#include "../kernels/common.cuh"
#include <vector>
#include <string.h>
#include <stdio.h>

// ---- kernel entry points implemented in ../kernels --------------------------------------------------------------
struct XbTransposeDesc;
XB_API int xb_conv_fprop_simt(const float*, const float*, const float*, float*, float*, const XbConvGeom*, int, cudaStream_t);
XB_API int xb_conv_dgrad_simt(const float*, const float*, float*, const XbConvGeom*, int, cudaStream_t);
XB_API int xb_conv_wgrad_simt(const float*, const float*, float*, const XbConvGeom*, cudaStream_t);
XB_API int xb_conv_fprop_tc(const float*, const float*, const float*, float*, float*, const XbConvGeom*, int, int*, cudaStream_t);
XB_API int xb_conv_dgrad_tc(const float*, const float*, float*, const XbConvGeom*, int, int*, cudaStream_t, const XbBnFuse*);
XB_API int xb_conv_wgrad_tc(const float*, const float*, float*, const XbConvGeom*, int*, cudaStream_t);
XB_API int xb_conv_fprop_im2col(const float*, const float*, const float*, float*, float*, const XbConvGeom*, int, float*, int*, cudaStream_t);
XB_API int xb_conv3x3_s2_dgrad(const float*, const float*, float*, const XbConvGeom*, int, float*, int*, cudaStream_t, const XbBnFuse*);
XB_API int xb_conv_wgrad_im2col(const float*, const float*, float*, const XbConvGeom*, float*, int, int*, cudaStream_t);
XB_API int xb_tc_supported(const XbConvGeom*, int which);
XB_API int xb_transpose_weights(const float*, float*, const XbTransposeDesc*, int, int, cudaStream_t);
XB_API int xb_bn_stats(const float*, float*, int, int, cudaStream_t);
XB_API int xb_bn_forward_mask(const float*, const float*, float*, const float*, const float*, const float*, float*, float*, float*, float*,
                              const XbTaskParams*, int, int, float, int, int, int, float, unsigned char*, cudaStream_t);
XB_API int xb_bn_backward_remask(const float*, const float*, const float*, const float*, const float*, const float*, float*, float*, float*, float*, int, int,
                                 int, cudaStream_t);
XB_API int xb_bn_backward_apply(const float*, const float*, const float*, const float*, const float*, const float*, const float*, float*, float*, float*,
                                float*, int, int, int, int, int, cudaStream_t);
XB_API int xb_bn_backward(const float*, const float*, const float*, const float*, const float*, const float*, float*, float*, float*, float*,
                          float*, int, int, int, int, int, cudaStream_t);
XB_API int xb_act_forward(const float*, float*, long long, int, float, float, cudaStream_t);
XB_API int xb_act_backward(const float*, const float*, const float*, float*, long long, int, float, float, int, cudaStream_t);
XB_API int xb_weighted_sum(const float* const*, const float*, int, float*, long long, int, cudaStream_t);
XB_API int xb_dropout(const float*, float*, long long, float, unsigned, const XbTaskParams*, int, cudaStream_t);
XB_API int xb_concat_copy(const float*, float*, long long, int, int, int, int, int, cudaStream_t);
XB_API int xb_pool_forward(const float*, float*, const int*, int, cudaStream_t);
XB_API int xb_pool_backward(const float*, const float*, float*, const int*, int, int, cudaStream_t);
XB_API int xb_lrn_forward(const float*, float*, float*, long long, int, int, float, float, float, cudaStream_t);
XB_API int xb_lrn_backward(const float*, const float*, const float*, const float*, float*, long long, int, int, float, float, int, cudaStream_t);
XB_API int xb_transform(const float*, float*, const float*, int, int, int, int, int, int, int, int, float, int, unsigned, const XbTaskParams*, cudaStream_t);
XB_API int xb_colsum(const float*, float*, int, int, cudaStream_t);
XB_API int xb_softmax_xent(const float*, const int*, float*, float*, float*, int, int, int, int, int, int, cudaStream_t);
XB_API int xb_classify(const float*, float*, int, int, cudaStream_t);
XB_API int xb_grad_sumsq(const float*, float*, long long, cudaStream_t);
XB_API int xb_matfact(const float*, int, const int*, const float*, const float*, float*, float*, float*, int, int, float, int, int, cudaStream_t);
XB_API int xb_fused_optimiser(float*, float*, float*, float*, float*, const float*, const float*, const XbTaskParams*, long long, int, cudaStream_t);

enum XbOpKind : int {
  OP_MEMSET = 0, OP_UPLOAD = 1, OP_TRANSFORM = 2, OP_CONV_FPROP = 3, OP_CONV_DGRAD = 4, OP_CONV_WGRAD = 5, OP_COLSUM = 6,
  OP_BN_STATS = 7, OP_BN_FWD = 8, OP_BN_BWD = 9, OP_ACT_FWD = 10, OP_ACT_BWD = 11, OP_SUM = 12, OP_DROPOUT = 13,
  OP_CONCAT = 14, OP_POOL_FWD = 15, OP_POOL_BWD = 16, OP_LRN_FWD = 17, OP_LRN_BWD = 18, OP_SOFTMAX_XENT = 19,
  OP_CLASSIFY = 20, OP_TRANSPOSE_W = 21, OP_GRAD_SUMSQ = 22, OP_OPTIMISER = 23, OP_COPY = 24, OP_MATFACT = 25,
  OP_MARK = 26,   // no launch: end of gradient bucket ia[0] - the learner records that bucket's event here
};

// One launch. Field meaning depends on `kind` (documented where the Python lowering fills them).
struct XbOp {
  int kind;
  int flags;
  int ia[16];
  float fa[8];
  long long la[4];
  void* p[12];
};

constexpr int XB_MAX_BUCKETS = 8;

struct XbProgram {
  std::vector<XbOp> ops;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  // A program with OP_MARK ops is cut there: one graph per segment, so the caller can record an ordinary stream event
  // between two segments (segs[i] covers ops [seg_first[i], seg_first[i+1]) and ends in mark seg_mark[i], or -1).
  std::vector<cudaGraphExec_t> segs;
  std::vector<int> seg_first, seg_mark;
  int marks = 0;
  int launches = 0;       // kernel launches issued by one replay (for accounting)
  int use_tc = 1;         // allow tensor-core convolution kernels
  int* tc_status = nullptr;
  // Set by the learner that owns the program: the task parameters are then copied to `params_dst` by the learner itself
  // at submission (from a per-task slot of a pinned ring), and the program's own first operator - the upload from the
  // learner's single parameter block - is left out of captures and replays.
  bool skip_upload = false;
  void* params_dst = nullptr;
  std::vector<cudaEvent_t> capture_events;   // fork / join events of a capture with operator branches (live only during it)
  cudaStream_t side_stream = nullptr;
};

static inline XbConvGeom geom_of(const XbOp& o) {
  XbConvGeom g;
  memcpy(&g, o.ia, sizeof(XbConvGeom));
  return g;
}

static int run_op(XbProgram* pr, const XbOp& o, cudaStream_t st) {
  switch (o.kind) {
    case OP_MEMSET: return (int)cudaMemsetAsync(o.p[0], 0, (size_t)o.la[0], st);
    case OP_UPLOAD: return (int)cudaMemcpyAsync(o.p[0], o.p[1], (size_t)o.la[0], cudaMemcpyHostToDevice, st);
    case OP_COPY:   return (int)cudaMemcpyAsync(o.p[0], o.p[1], (size_t)o.la[0], cudaMemcpyDeviceToDevice, st);
    case OP_TRANSFORM:
      return xb_transform((const float*)o.p[0], (float*)o.p[1], (const float*)o.p[2], o.ia[0], o.ia[1], o.ia[2], o.ia[3], o.ia[4], o.ia[5],
                          o.ia[6], o.ia[7], o.fa[0], o.ia[8], (unsigned)o.ia[9], (const XbTaskParams*)o.p[3], st);
    case OP_CONV_FPROP: {
      XbConvGeom g = geom_of(o);
      if (pr->use_tc && (o.flags & 0x100) && o.p[5])       // patch matrix + GEMM, scratch provided by the lowering
        return xb_conv_fprop_im2col((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (float*)o.p[3], (float*)o.p[4], &g, o.flags & 0xff,
                                    (float*)o.p[5], pr->tc_status, st);
      if (pr->use_tc && (o.flags & 0x100) && xb_tc_supported(&g, 0))
        return xb_conv_fprop_tc((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (float*)o.p[3], (float*)o.p[4], &g, o.flags & 0xff, pr->tc_status, st);
      return xb_conv_fprop_simt((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (float*)o.p[3], (float*)o.p[4], &g, o.flags & 0xff, st);
    }
    case OP_CONV_DGRAD: {
      XbConvGeom g = geom_of(o);
      // p[4..8]: batch-norm backward sums of the layer that owns dX, produced by this kernel's epilogue (flags 0x8; 0x10 = ReLU mask)
      XbBnFuse bn{(const float*)o.p[4], (const float*)o.p[5], (const float*)o.p[6], (const float*)o.p[7], (float*)o.p[8], (o.flags & 0x10) ? 1 : 0};
      const XbBnFuse* bnp = (o.flags & 0x8) ? &bn : nullptr;
      if (pr->use_tc && (o.flags & 0x100) && o.p[3])       // stride-2 3x3: zero-inserted gradient + stride-1 slab kernel
        return xb_conv3x3_s2_dgrad((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], &g, o.flags & 1, (float*)o.p[3], pr->tc_status, st, bnp);
      if (pr->use_tc && (o.flags & 0x100) && xb_tc_supported(&g, 1))
        return xb_conv_dgrad_tc((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], &g, o.flags & 1, pr->tc_status, st, bnp);
      if (bnp) return -XB_BAD_ARG;
      return xb_conv_dgrad_simt((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], &g, o.flags & 1, st);
    }
    case OP_CONV_WGRAD: {
      XbConvGeom g = geom_of(o);
      if (pr->use_tc && (o.flags & 0x100) && o.p[3])
        return xb_conv_wgrad_im2col((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], &g, (float*)o.p[3], o.flags & 0x20, pr->tc_status, st);
      if (pr->use_tc && (o.flags & 0x100) && xb_tc_supported(&g, 2))
        return xb_conv_wgrad_tc((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], &g, pr->tc_status, st);
      return xb_conv_wgrad_simt((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], &g, st);
    }
    case OP_COLSUM: return xb_colsum((const float*)o.p[0], (float*)o.p[1], o.ia[0], o.ia[1], st);
    case OP_BN_STATS: return xb_bn_stats((const float*)o.p[0], (float*)o.p[1], o.ia[0], o.ia[1], st);
    case OP_BN_FWD:
      // p[11]: packed sign mask of the output (layers with ReLU and a residual input; their backward pass reads it instead of y)
      return xb_bn_forward_mask((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], (const float*)o.p[3], (const float*)o.p[4],
                                (const float*)o.p[5], (float*)o.p[6], (float*)o.p[7], (float*)o.p[8], (float*)o.p[9], (const XbTaskParams*)o.p[10],
                                o.ia[0], o.ia[1], o.fa[0], o.ia[2], o.ia[3], o.ia[4], o.fa[1], (unsigned char*)o.p[11], st);
    case OP_BN_BWD:
      if (o.p[11] && !o.ia[5])   // ReLU without residual: mask re-derived from x, the layer's output is not read
        return xb_bn_backward_remask((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[3], (const float*)o.p[4], (const float*)o.p[5],
                                     (const float*)o.p[11], (float*)o.p[6], (float*)o.p[7], (float*)o.p[9], (float*)o.p[10], o.ia[0], o.ia[1], o.ia[3], st);
      if (o.ia[5])     // the sums were produced by the operator that completed dy
        return xb_bn_backward_apply((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (const float*)o.p[3], (const float*)o.p[4],
                                    (const float*)o.p[5], (const float*)o.p[6], (float*)o.p[7], (float*)o.p[8], (float*)o.p[9], (float*)o.p[10],
                                    o.ia[0], o.ia[1], o.ia[2], o.ia[3], o.ia[4], st);
      return xb_bn_backward((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (const float*)o.p[3], (const float*)o.p[4],
                            (const float*)o.p[5], (float*)o.p[6], (float*)o.p[7], (float*)o.p[8], (float*)o.p[9], (float*)o.p[10],
                            o.ia[0], o.ia[1], o.ia[2], o.ia[3], o.ia[4], st);
    case OP_ACT_FWD: return xb_act_forward((const float*)o.p[0], (float*)o.p[1], o.la[0], o.ia[0], o.fa[0], o.fa[1], st);
    case OP_ACT_BWD:
      return xb_act_backward((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (float*)o.p[3], o.la[0], o.ia[0], o.fa[0], o.fa[1], o.ia[1], st);
    case OP_SUM: {
      const float* xs[4] = {(const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (const float*)o.p[3]};
      return xb_weighted_sum(xs, o.fa, o.ia[0], (float*)o.p[4], o.la[0], o.ia[1], st);
    }
    case OP_DROPOUT: return xb_dropout((const float*)o.p[0], (float*)o.p[1], o.la[0], o.fa[0], (unsigned)o.ia[0], (const XbTaskParams*)o.p[2], o.ia[1], st);
    case OP_CONCAT: return xb_concat_copy((const float*)o.p[0], (float*)o.p[1], o.la[0], o.ia[0], o.ia[1], o.ia[2], o.ia[3], o.ia[4], st);
    case OP_POOL_FWD: return xb_pool_forward((const float*)o.p[0], (float*)o.p[1], o.ia, o.flags & 1, st);
    case OP_POOL_BWD: return xb_pool_backward((const float*)o.p[0], (const float*)o.p[1], (float*)o.p[2], o.ia, o.flags & 1, (o.flags >> 1) & 1, st);
    case OP_LRN_FWD: return xb_lrn_forward((const float*)o.p[0], (float*)o.p[1], (float*)o.p[2], o.la[0], o.ia[0], o.ia[1], o.fa[0], o.fa[1], o.fa[2], st);
    case OP_LRN_BWD:
      return xb_lrn_backward((const float*)o.p[0], (const float*)o.p[1], (const float*)o.p[2], (const float*)o.p[3], (float*)o.p[4], o.la[0], o.ia[0],
                             o.ia[1], o.fa[0], o.fa[1], o.ia[2], st);
    case OP_SOFTMAX_XENT:
      return xb_softmax_xent((const float*)o.p[0], (const int*)o.p[1], (float*)o.p[2], (float*)o.p[3], (float*)o.p[4], o.ia[0], o.ia[1], o.ia[2], o.ia[3], o.ia[4], o.ia[5], st);
    case OP_CLASSIFY: return xb_classify((const float*)o.p[0], (float*)o.p[1], o.ia[0], o.ia[1], st);
    case OP_TRANSPOSE_W: return xb_transpose_weights((const float*)o.p[0], (float*)o.p[1], (const XbTransposeDesc*)o.p[2], o.ia[0], o.ia[1], st);
    case OP_MATFACT:
      return xb_matfact((const float*)o.p[0], o.ia[0], (const int*)o.p[1], (const float*)o.p[2], (const float*)o.p[3], (float*)o.p[4], (float*)o.p[5],
                        (float*)o.p[6], o.ia[1], o.ia[2], o.fa[0], o.ia[3], o.ia[4], st);
    case OP_MARK: return 0;
    case OP_GRAD_SUMSQ: return xb_grad_sumsq((const float*)o.p[0], (float*)o.p[1], o.la[0], st);
    case OP_OPTIMISER:
      return xb_fused_optimiser((float*)o.p[0], (float*)o.p[1], (float*)o.p[2], (float*)o.p[3], (float*)o.p[4], (const float*)o.p[5],
                                (const float*)o.p[6], (const XbTaskParams*)o.p[7], o.la[0], o.ia[0], st);
  }
  return -XB_BAD_ARG;
}

XB_API int xb_op_size() { return (int)sizeof(XbOp); }

XB_API XbProgram* xb_program_create(const XbOp* ops, int n, int use_tc, int* tc_status_dev) {
  XbProgram* p = new XbProgram();
  p->ops.assign(ops, ops + n);
  p->use_tc = use_tc;
  p->tc_status = tc_status_dev;
  int l = 0;
  for (int i = 0; i < n; ++i) {
    int k = ops[i].kind;
    if (k == OP_MARK) { p->marks++; continue; }
    if (k == OP_MEMSET || k == OP_UPLOAD || k == OP_COPY) continue;
    l += (k == OP_BN_BWD) ? 2 : 1;
  }
  p->launches = l;
  return p;
}
static void drop_segments(XbProgram* p) {
  for (cudaGraphExec_t g : p->segs) if (g) cudaGraphExecDestroy(g);
  p->segs.clear(); p->seg_first.clear(); p->seg_mark.clear();
}
XB_API void xb_program_destroy(XbProgram* p) {
  if (!p) return;
  drop_segments(p);
  if (p->exec) cudaGraphExecDestroy(p->exec);
  if (p->graph) cudaGraphDestroy(p->graph);
  delete p;
}
XB_API int xb_program_launches(XbProgram* p) { return p->launches; }
XB_API int xb_program_num_ops(XbProgram* p) { return (int)p->ops.size(); }

// Issue every op on `st`. Returns 0 or (1000*op_index + error) so the caller can name the failing op.
// ---- tracing (utils.h:13-16 __NVPROF_MARK_TASK / __NVPROF_MARK_OPERATOR, INTRA_ / INTER_TASK_MEASUREMENTS of the reference) ----
// level 0: off.  1: an NVTX range around every task submission, device time of every task (two timing events per task) and
// host inter-arrival time of submissions.  2: also an NVTX range per operator while a program is issued or captured.
static int g_trace = 0;
XB_API void xb_trace_set(int level) { g_trace = level; }
XB_API int xb_trace_level() { return g_trace; }
static const char* op_name(int kind) {
  static const char* names[] = {"memset", "upload", "transform", "conv-fprop", "conv-dgrad", "conv-wgrad", "colsum", "bn-stats", "bn-fwd", "bn-bwd",
                                "act-fwd", "act-bwd", "sum", "dropout", "concat", "pool-fwd", "pool-bwd", "lrn-fwd", "lrn-bwd", "softmax-xent",
                                "classify", "transpose-w", "grad-sumsq", "optimiser", "copy", "matfact", "mark"};
  return (kind >= 0 && kind < (int)(sizeof(names) / sizeof(names[0]))) ? names[kind] : "op";
}
struct TaskTrace {
  std::mutex mu;
  std::vector<float> device_ms;        // per finished task
  std::vector<float> arrival_us;       // host time between consecutive submissions
  std::chrono::steady_clock::time_point last_submit; bool have_last = false;
};
static TaskTrace g_tt;
// copies up to n values (most recent last) into out; which: 0 device time per task (ms), 1 inter-arrival (us). Returns the count.
XB_API int xb_trace_read(int which, float* out, int n, int clear) {
  std::lock_guard<std::mutex> g(g_tt.mu);
  std::vector<float>& v = which == 0 ? g_tt.device_ms : g_tt.arrival_us;
  int m = (int)v.size() < n ? (int)v.size() : n;
  for (int i = 0; i < m; ++i) out[i] = v[v.size() - m + i];
  if (clear) v.clear();
  return m;
}

static inline int run_op_traced(XbProgram* p, const XbOp& o, cudaStream_t st) {
  if (g_trace < 2) return run_op(p, o, st);
  nvtxRangePushA(op_name(o.kind));
  int e = run_op(p, o, st);
  nvtxRangePop();
  return e;
}
// (captures and the learner's own replays leave the upload operator out when the learner copies the parameters itself;
// a program that is run directly - xb_program_run, xb_program_run_range - executes every operator)
static inline bool skipped(const XbProgram* p, size_t i) { return p->skip_upload && i == 0 && p->ops[0].kind == OP_UPLOAD; }
static int run_ops(XbProgram* p, int first, int last, cudaStream_t st, bool for_learner) {
  for (int i = first; i < last && i < (int)p->ops.size(); ++i) {
    if (for_learner && skipped(p, (size_t)i)) continue;
    int e = run_op_traced(p, p->ops[i], st);
    if (e != 0) return 1000 * (i + 1) + (e < 0 ? -e : e);
  }
  return 0;
}
XB_API int xb_program_run(XbProgram* p, cudaStream_t st) { return run_ops(p, 0, (int)p->ops.size(), st, false); }
// Run a sub-range [first, last) - used by tests that inspect intermediate tensors.
XB_API int xb_program_run_range(XbProgram* p, int first, int last, cudaStream_t st) { return run_ops(p, first, last, st, false); }

// Operator branches inside a task.  An operator flagged XB_OP_SIDE does not feed the operators that follow it in the list:
// the weight (and bias) gradient of a layer is only read by the optimiser at the end of the task, while the chain
// data gradient -> normalisation backward -> data gradient ... is what the task's latency consists of.  When the program
// is captured, such operators are recorded on a second stream that forks off the main one right where the operator stands
// and joins it again in front of the next operator that reads the gradient vector (the optimiser, or the gradient-norm
// reduction of clipping); in the CUDA graph they become a parallel branch, so the device runs them next to the main
// chain.  (The reference has per-operator stream "branches" with event dependencies, executioncontext.c:657-671, but
// its labelling pass is switched off and the branch factor stays 1, SubGraph.java:208-212.)  A program that is issued
// directly, not captured, runs its operators in list order on one stream.
// XB_OP_JOIN on an operator of the main chain: it reads what the branch has produced so far (the first data gradient
// reads the transposed weight copy, which is written on the branch while the forward pass runs), so the main stream waits
// for the branch in front of it.
constexpr int XB_OP_SIDE = 0x1000, XB_OP_JOIN = 0x2000;
static int g_side_low = 0;
XB_API void xb_program_side_priority(int low) { g_side_low = low ? 1 : 0; }
static inline bool joins_side(int kind) { return kind == OP_OPTIMISER || kind == OP_GRAD_SUMSQ; }

static int capture_with_branches(XbProgram* p, cudaStream_t st) {
  cudaStream_t side = nullptr;
  std::vector<cudaEvent_t> events;
  auto event = [&]() { cudaEvent_t ev = nullptr; cudaEventCreateWithFlags(&ev, cudaEventDisableTiming); events.push_back(ev); return ev; };
  int e = 0;
  bool open = false;
  auto join = [&]() -> int {
    if (!open) return 0;
    cudaEvent_t ev = event();
    XB_CUDA_CHECK(cudaEventRecord(ev, side));
    XB_CUDA_CHECK(cudaStreamWaitEvent(st, ev, 0));
    open = false;
    return 0;
  };
  for (size_t i = 0; i < p->ops.size() && e == 0; ++i) {
    const XbOp& o = p->ops[i];
    if (skipped(p, i)) continue;
    if (o.flags & XB_OP_SIDE) {
      if (!side) {
        // the branch's kernels inherit this stream's priority in the graph: with g_side_low they only take what the main
        // chain leaves free
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        if (cudaStreamCreateWithPriority(&side, cudaStreamNonBlocking, g_side_low ? lo : 0) != cudaSuccess) { e = -XB_BAD_ARG; break; }
      }
      cudaEvent_t ev = event();                                  // fork: everything issued on the main stream so far
      if ((e = (int)cudaEventRecord(ev, st)) != 0) break;
      if ((e = (int)cudaStreamWaitEvent(side, ev, 0)) != 0) break;
      open = true;
      e = run_op_traced(p, o, side);
      if (e != 0) e = (int)(1000 * (i + 1) + (e < 0 ? -e : e));
      continue;
    }
    if ((joins_side(o.kind) || (o.flags & XB_OP_JOIN)) && (e = join()) != 0) break;
    e = run_op_traced(p, o, st);
    if (e != 0) e = (int)(1000 * (i + 1) + (e < 0 ? -e : e));
  }
  if (e == 0) e = join(); else join();                             // a capture can only end with every branch joined
  p->capture_events = events;                                      // destroyed with the program (after the capture has ended)
  p->side_stream = side;
  return e;
}

// Record the program into a CUDA graph (the stream must not be the legacy default stream).
XB_API int xb_program_capture_segments(XbProgram* p, cudaStream_t st);
XB_API int xb_program_capture(XbProgram* p, cudaStream_t st) {
  if (p->marks > 0) return xb_program_capture_segments(p, st);
  if (p->exec) { cudaGraphExecDestroy(p->exec); p->exec = nullptr; }
  if (p->graph) { cudaGraphDestroy(p->graph); p->graph = nullptr; }
  bool branches = false;
  for (const XbOp& o : p->ops) branches |= (o.flags & XB_OP_SIDE) != 0;
  XB_CUDA_CHECK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
  int e = branches ? capture_with_branches(p, st) : run_ops(p, 0, (int)p->ops.size(), st, true);
  cudaGraph_t g = nullptr;
  cudaError_t ce = cudaStreamEndCapture(st, &g);
  for (cudaEvent_t ev : p->capture_events) cudaEventDestroy(ev);
  p->capture_events.clear();
  if (p->side_stream) { cudaStreamDestroy(p->side_stream); p->side_stream = nullptr; }
  if (e != 0) { if (g) cudaGraphDestroy(g); return e; }
  if (ce != cudaSuccess) return (int)ce;
  p->graph = g;
  XB_CUDA_CHECK(cudaGraphInstantiate(&p->exec, g, 0));
  return 0;
}
// The same, cut at the marks: one graph per segment (see XbProgram::segs).
XB_API int xb_program_capture_segments(XbProgram* p, cudaStream_t st) {
  drop_segments(p);
  const int n = (int)p->ops.size();
  int first = 0;
  while (first < n) {
    int last = first, mark = -1;
    while (last < n && p->ops[last].kind != OP_MARK) ++last;
    if (last < n) { mark = p->ops[last].ia[0]; ++last; }          // the mark closes the segment
    XB_CUDA_CHECK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    int e = run_ops(p, first, last, st, true);
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(st, &g);
    if (e != 0 || ce != cudaSuccess) { if (g) cudaGraphDestroy(g); drop_segments(p); return e != 0 ? e : (int)ce; }
    cudaGraphExec_t ex = nullptr;
    ce = cudaGraphInstantiate(&ex, g, 0);
    cudaGraphDestroy(g);
    if (ce != cudaSuccess) { drop_segments(p); return (int)ce; }
    p->segs.push_back(ex); p->seg_first.push_back(first); p->seg_mark.push_back(mark);
    first = last;
  }
  return 0;
}
XB_API int xb_program_marks(XbProgram* p) { return p->marks; }
// Replay; `marks[b]` (may be null) is recorded on `st` right after the ops that precede mark b.
XB_API int xb_program_launch_marked(XbProgram* p, cudaStream_t st, cudaEvent_t* marks, int nmarks) {
  if (!p->segs.empty()) {
    for (size_t i = 0; i < p->segs.size(); ++i) {
      XB_CUDA_CHECK(cudaGraphLaunch(p->segs[i], st));
      const int m = p->seg_mark[i];
      if (m >= 0 && m < nmarks && marks && marks[m]) XB_CUDA_CHECK(cudaEventRecord(marks[m], st));
    }
    return 0;
  }
  if (p->exec && p->marks == 0) return (int)cudaGraphLaunch(p->exec, st);
  for (size_t i = 0; i < p->ops.size(); ++i) {
    const XbOp& o = p->ops[i];
    if (skipped(p, i)) continue;
    if (o.kind == OP_MARK) {
      if (o.ia[0] >= 0 && o.ia[0] < nmarks && marks && marks[o.ia[0]]) XB_CUDA_CHECK(cudaEventRecord(marks[o.ia[0]], st));
      continue;
    }
    int e = run_op_traced(p, o, st);
    if (e != 0) return (int)(1000 * (i + 1) + (e < 0 ? -e : e));
  }
  return 0;
}
XB_API int xb_program_launch(XbProgram* p, cudaStream_t st) { return xb_program_launch_marked(p, st, nullptr, 0); }

__global__ void copy_result_kernel(const float* __restrict__ src, float* __restrict__ dst) {
  if (threadIdx.x < 2) dst[threadIdx.x] = src[threadIdx.x];
}

// ---- learner: stream + staging buffers + programs ------------------------------------------------------------------
struct XbLearner {
  cudaStream_t stream = nullptr;
  cudaEvent_t done = nullptr, start = nullptr;
  cudaEvent_t bucket[XB_MAX_BUCKETS] = {};   // gradient bucket b of the last training task is complete (created on demand)
  XbProgram* train = nullptr;
  XbProgram* test = nullptr;
  void* d_examples = nullptr; size_t examples_bytes = 0;
  void* d_labels = nullptr; size_t labels_bytes = 0;
  XbTaskParams* h_params = nullptr;   // pinned; what a program's own upload operator reads (programs run outside a learner)
  // A learner may hold several tasks in flight, and a copy enqueued on its stream reads its source when it EXECUTES, not
  // when the task is submitted: each submission therefore writes its parameters into its own slot of this pinned ring and
  // enqueues the host-to-device copy from that slot, so a task can never see the parameters of a later one (the learning
  // rate at a schedule boundary, the task number that seeds dropout and crops).
  static constexpr int PARAM_RING = 16;
  XbTaskParams* h_params_ring = nullptr;
  float* h_result = nullptr;          // pinned + mapped: [loss, accuracy] written by the loss kernel
  float* d_result = nullptr;          // device alias of h_result
  // Run-ahead: a learner may hold several tasks in flight.  After each task a one-thread kernel copies the live result pair
  // into the ring slot of that task (floats [4 + 2 s, 4 + 2 s + 2) of the same mapped allocation) and an event of its own
  // is recorded, so the host can wait for and read one particular task.
  static constexpr int RING = 4;
  cudaEvent_t ring_done[RING] = {};
  cudaEvent_t ring_t0[RING] = {}, ring_t1[RING] = {};   // tracing: timing events around the task (created on demand)
  bool ring_timed[RING] = {};
  unsigned long long ring_task[RING] = {};
  int ring_phase[RING] = {};
  std::atomic<unsigned long long> submitted{0};   // written by the submitting thread, read by the thread that waits for a task
  int busy = 0;
};

XB_API XbLearner* xb_learner_create(int priority, void* d_examples, long long examples_bytes, void* d_labels, long long labels_bytes) {
  XbLearner* l = new XbLearner();
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  int pr = priority < hi ? hi : (priority > lo ? lo : priority);
  if (cudaStreamCreateWithPriority(&l->stream, cudaStreamNonBlocking, pr) != cudaSuccess) { delete l; return nullptr; }
  cudaEventCreateWithFlags(&l->done, cudaEventDisableTiming);
  cudaEventCreate(&l->start);
  cudaHostAlloc((void**)&l->h_params, sizeof(XbTaskParams), cudaHostAllocDefault);
  cudaHostAlloc((void**)&l->h_params_ring, sizeof(XbTaskParams) * XbLearner::PARAM_RING, cudaHostAllocDefault);
  cudaHostAlloc((void**)&l->h_result, 64, cudaHostAllocMapped);
  for (int i = 0; i < XbLearner::RING; ++i) { cudaEventCreateWithFlags(&l->ring_done[i], cudaEventDisableTiming); l->ring_task[i] = ~0ull; }
  memset(l->h_params, 0, sizeof(XbTaskParams));
  memset(l->h_result, 0, 64);
  cudaHostGetDevicePointer((void**)&l->d_result, l->h_result, 0);
  l->d_examples = d_examples; l->examples_bytes = (size_t)examples_bytes;
  l->d_labels = d_labels; l->labels_bytes = (size_t)labels_bytes;
  return l;
}
XB_API void xb_learner_destroy(XbLearner* l) {
  if (!l) return;
  cudaStreamSynchronize(l->stream);
  cudaEventDestroy(l->done); cudaEventDestroy(l->start);
  for (cudaEvent_t ev : l->bucket) if (ev) cudaEventDestroy(ev);
  for (cudaEvent_t ev : l->ring_done) if (ev) cudaEventDestroy(ev);
  for (int i = 0; i < XbLearner::RING; ++i) { if (l->ring_t0[i]) cudaEventDestroy(l->ring_t0[i]); if (l->ring_t1[i]) cudaEventDestroy(l->ring_t1[i]); }
  cudaFreeHost(l->h_params); cudaFreeHost(l->h_params_ring); cudaFreeHost(l->h_result);
  cudaStreamDestroy(l->stream);
  delete l;
}
XB_API void* xb_learner_stream(XbLearner* l) { return (void*)l->stream; }
XB_API XbTaskParams* xb_learner_params(XbLearner* l) { return l->h_params; }
XB_API float* xb_learner_result_host(XbLearner* l) { return l->h_result; }
XB_API float* xb_learner_result_dev(XbLearner* l) { return l->d_result; }
XB_API void xb_learner_set_programs(XbLearner* l, XbProgram* train, XbProgram* test) {
  l->train = train; l->test = test;
  for (XbProgram* p : {train, test})
    if (p && !p->ops.empty() && p->ops[0].kind == OP_UPLOAD && p->ops[0].p[1] == (void*)l->h_params
        && (size_t)p->ops[0].la[0] == sizeof(XbTaskParams)) {
      p->skip_upload = true; p->params_dst = p->ops[0].p[0];      // (call this before the program is captured)
    }
}

// Enqueue one task: copy the batch from (pinned) host memory, replay the program, record the completion event.
// phase 0 = train, 1 = test.  Never blocks.
// `tag` is the number xb_learner_wait_task finds the task by (the submitting scheduler's own task counter, which may
// differ from the job-wide number in the parameter block).
static int learner_submit_tagged(XbLearner* l, const void* h_examples, const void* h_labels, const XbTaskParams* params, int phase, unsigned long long tag);
XB_API int xb_learner_submit(XbLearner* l, const void* h_examples, const void* h_labels, const XbTaskParams* params, int phase) {
  return learner_submit_tagged(l, h_examples, h_labels, params, phase, params->task_id);
}
static int learner_submit_tagged(XbLearner* l, const void* h_examples, const void* h_labels, const XbTaskParams* params, int phase, unsigned long long tag) {
  XbProgram* p = phase == 0 ? l->train : l->test;
  if (!p) return -XB_BAD_ARG;
  *l->h_params = *params;
  if (p->skip_upload) {
    XbTaskParams* mine = l->h_params_ring + (l->submitted.load() % XbLearner::PARAM_RING);
    *mine = *params;
    XB_CUDA_CHECK(cudaMemcpyAsync(p->params_dst, mine, sizeof(XbTaskParams), cudaMemcpyHostToDevice, l->stream));
  }
  if (h_examples) XB_CUDA_CHECK(cudaMemcpyAsync(l->d_examples, h_examples, l->examples_bytes, cudaMemcpyHostToDevice, l->stream));
  if (h_labels) XB_CUDA_CHECK(cudaMemcpyAsync(l->d_labels, h_labels, l->labels_bytes, cudaMemcpyHostToDevice, l->stream));
  if (p->marks > 0)
    for (int b = 0; b < XB_MAX_BUCKETS && b < p->marks; ++b)
      if (!l->bucket[b]) XB_CUDA_CHECK(cudaEventCreateWithFlags(&l->bucket[b], cudaEventDisableTiming));
  const int slot = (int)(l->submitted.fetch_add(1) % XbLearner::RING);
  const bool timed = g_trace >= 1;
  if (timed) {
    char label[48]; snprintf(label, sizeof label, "%s task %u", phase == 0 ? "train" : "test", params->task_id);
    nvtxRangePushA(label);
    if (!l->ring_t0[slot]) { XB_CUDA_CHECK(cudaEventCreate(&l->ring_t0[slot])); XB_CUDA_CHECK(cudaEventCreate(&l->ring_t1[slot])); }
    XB_CUDA_CHECK(cudaEventRecord(l->ring_t0[slot], l->stream));
    auto now = std::chrono::steady_clock::now();
    std::lock_guard<std::mutex> g(g_tt.mu);
    if (g_tt.have_last) g_tt.arrival_us.push_back(std::chrono::duration<float, std::micro>(now - g_tt.last_submit).count());
    g_tt.last_submit = now; g_tt.have_last = true;
  }
  l->ring_timed[slot] = timed;
  int e = xb_program_launch_marked(p, l->stream, l->bucket, XB_MAX_BUCKETS);
  if (timed) { if (!e) e = (int)cudaEventRecord(l->ring_t1[slot], l->stream); nvtxRangePop(); }
  if (e) return e;
  l->ring_task[slot] = tag & 0xffffffffull; l->ring_phase[slot] = phase;
  copy_result_kernel<<<1, 32, 0, l->stream>>>(l->d_result, l->d_result + 4 + 2 * slot);
  XB_CUDA_CHECK(cudaGetLastError());
  XB_CUDA_CHECK(cudaEventRecord(l->ring_done[slot], l->stream));
  XB_CUDA_CHECK(cudaEventRecord(l->done, l->stream));
  l->busy = 1;
  return 0;
}
// Block until task `task` (the most recent submission with that id; of that phase unless phase < 0) has finished and
// return ITS loss / accuracy.
XB_API int xb_learner_wait_task(XbLearner* l, unsigned long long task, int phase, float* loss, float* accuracy) {
  const unsigned long long submitted = l->submitted.load();
  for (unsigned long long back = 0; back < (unsigned long long)XbLearner::RING && back < submitted; ++back) {
    const int slot = (int)((submitted - 1 - back) % XbLearner::RING);
    if (l->ring_task[slot] != (task & 0xffffffffull) || (phase >= 0 && l->ring_phase[slot] != phase)) continue;
    XB_CUDA_CHECK(cudaEventSynchronize(l->ring_done[slot]));
    if (l->ring_timed[slot]) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, l->ring_t0[slot], l->ring_t1[slot]) == cudaSuccess) { std::lock_guard<std::mutex> g(g_tt.mu); g_tt.device_ms.push_back(ms); }
      l->ring_timed[slot] = false;
    }
    if (loss) *loss = l->h_result[4 + 2 * slot];
    if (accuracy) *accuracy = l->h_result[4 + 2 * slot + 1];
    return 0;
  }
  return -XB_BAD_ARG;
}
// Block until the learner's last task has finished; loss/accuracy are then valid in the result slot.
XB_API int xb_learner_wait(XbLearner* l, float* loss, float* accuracy) {
  XB_CUDA_CHECK(cudaEventSynchronize(l->done));
  l->busy = 0;
  if (loss) *loss = l->h_result[0];
  if (accuracy) *accuracy = l->h_result[1];
  return 0;
}
XB_API int xb_learner_query(XbLearner* l) {
  cudaError_t e = cudaEventQuery(l->done);
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) { return 0; }
  return -(int)e;
}
// Make stream `st` wait for this learner's last task (used by the synchroniser) and vice versa.
XB_API int xb_stream_wait_learner(cudaStream_t st, XbLearner* l) { return (int)cudaStreamWaitEvent(st, l->done, 0); }
// `st` waits until gradient bucket b of the learner's last submitted training task is complete (the whole task if the
// program has no such mark)
XB_API int xb_stream_wait_learner_bucket(cudaStream_t st, XbLearner* l, int b) {
  cudaEvent_t ev = (b >= 0 && b < XB_MAX_BUCKETS && l->bucket[b]) ? l->bucket[b] : l->done;
  return (int)cudaStreamWaitEvent(st, ev, 0);
}
XB_API int xb_learner_wait_event(XbLearner* l, cudaEvent_t ev) { return (int)cudaStreamWaitEvent(l->stream, ev, 0); }

// ---- small CUDA plumbing used from Python (keeps torch out of the hot path) -----------------------------------------
XB_API void* xb_stream_create(int priority) {
  cudaStream_t s; int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  int pr = priority < hi ? hi : (priority > lo ? lo : priority);
  if (cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, pr) != cudaSuccess) return nullptr;
  return (void*)s;
}
XB_API int xb_stream_destroy(void* s) { return (int)cudaStreamDestroy((cudaStream_t)s); }
XB_API int xb_stream_sync(void* s) { return (int)cudaStreamSynchronize((cudaStream_t)s); }
XB_API void* xb_event_create(int timing) {
  cudaEvent_t e;
  if (cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming) != cudaSuccess) return nullptr;
  return (void*)e;
}
XB_API int xb_event_destroy(void* e) { return (int)cudaEventDestroy((cudaEvent_t)e); }
XB_API int xb_event_record(void* e, void* s) { return (int)cudaEventRecord((cudaEvent_t)e, (cudaStream_t)s); }
XB_API int xb_event_sync(void* e) { return (int)cudaEventSynchronize((cudaEvent_t)e); }
XB_API int xb_stream_wait_event(void* s, void* e) { return (int)cudaStreamWaitEvent((cudaStream_t)s, (cudaEvent_t)e, 0); }
XB_API float xb_event_elapsed_ms(void* a, void* b) { float ms = -1.f; cudaEventElapsedTime(&ms, (cudaEvent_t)a, (cudaEvent_t)b); return ms; }
XB_API void* xb_pinned_alloc(long long bytes) { void* p = nullptr; if (cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocPortable) != cudaSuccess) return nullptr; return p; }
XB_API int xb_pinned_free(void* p) { return (int)cudaFreeHost(p); }
XB_API void* xb_device_alloc(long long bytes) { void* p = nullptr; if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) return nullptr; cudaMemset(p, 0, (size_t)bytes); return p; }
XB_API int xb_device_free(void* p) { return (int)cudaFree(p); }
XB_API int xb_memcpy_h2d_async(void* d, const void* h, long long bytes, void* s) { return (int)cudaMemcpyAsync(d, h, (size_t)bytes, cudaMemcpyHostToDevice, (cudaStream_t)s); }
XB_API int xb_memcpy_d2h_async(void* h, const void* d, long long bytes, void* s) { return (int)cudaMemcpyAsync(h, d, (size_t)bytes, cudaMemcpyDeviceToHost, (cudaStream_t)s); }
XB_API int xb_memcpy_d2d_async(void* d, const void* s_, long long bytes, void* s) { return (int)cudaMemcpyAsync(d, s_, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)s); }
XB_API int xb_device_sync() { return (int)cudaDeviceSynchronize(); }
XB_API int xb_set_device(int d) { return (int)cudaSetDevice(d); }
XB_API const char* xb_error_string(int e) { return cudaGetErrorString((cudaError_t)e); }
XB_API int xb_last_error() { return (int)cudaGetLastError(); }

// ---- peer memory (one process per GPU): export / import of cudaMalloc'd buffers --------------------------------------
XB_API int xb_ipc_export(void* dptr, void* handle64) {
  cudaIpcMemHandle_t h;
  XB_CUDA_CHECK(cudaIpcGetMemHandle(&h, dptr));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
XB_API void* xb_ipc_import(const void* handle64) {
  cudaIpcMemHandle_t h; memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return nullptr;
  return p;
}
XB_API int xb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// ---- native executor: what the host runtime (libxbow_rt) drives through function pointers ----------------------------
//
// submit / wait / synchronise / batch have the exact signatures of the runtime's Executor table, so scheduler threads
// call straight into this library without passing through Python.  The learning-rate schedule is evaluated here per
// task (clib-multigpu/solverconfiguration.c:116-162 does the same natively), including the signal that makes the
// next synchronisation overwrite the replicas with the central model when a multi-step boundary has been crossed.
#include <math.h>

struct XbSolverState {
  int policy;            // 0 FIXED 1 INV 2 STEP 3 MULTISTEP 4 LSR 5 EXP
  float base_lr, gamma, power, momentum, weight_decay, clip, alpha;
  long long step_size, warmup;
  int nsteps; long long steps[32];
  int l1, nesterov, cma;
  int step_cursor; int copy_signal;
};

static float solver_lr(XbSolverState& s, unsigned long long task) {
  double t1 = (double)task + 1.0;
  switch (s.policy) {
    case 0: return s.base_lr;
    case 1: return s.base_lr * (float)pow(1.0 + s.gamma * t1, -s.power);
    case 2: return s.base_lr * (float)pow((double)s.gamma, floor(t1 / (double)(s.step_size > 0 ? s.step_size : 1)));
    case 4:
      if (s.warmup > 0 && (long long)task < s.warmup) return s.base_lr * (float)task / (float)s.warmup;
      // fall through
    case 3:
      if (s.step_cursor < s.nsteps && (long long)task + 1 >= s.steps[s.step_cursor]) { s.step_cursor++; s.copy_signal = 1; }
      return s.base_lr * (float)pow((double)s.gamma, (double)s.step_cursor);
    case 5: return s.base_lr * (float)pow((double)s.gamma, t1);
  }
  return s.base_lr;
}

// mirror of the descriptor in ../kernels/sync.cu (layout checked at start-up through xb_sync_desc_size)
struct XbSyncDescMirror {
  int rank, G, k, algo; long long n; unsigned int epoch; int two_shot, copy_to_replicas, use_prev;
  float alpha, mu, scale, blend;
  float* w[16]; const float* prev[16]; float* z; float* zlast; float* gacc;
  float* inbox[8]; float* result[8]; unsigned int* flags[8]; int* status; double timeout_s;
  float* zpeer[8];
  float* part_local; const float* part_mc; float* z_mc;
  unsigned int* release; unsigned long long* stamps;
};
XB_API int xb_stream_wait_value32(cudaStream_t st, const unsigned int* word, unsigned int value);
XB_API int xb_fused_sync(const XbSyncDescMirror* d, void* args_dev, void* args_pinned, int max_blocks, cudaStream_t st);
XB_API int xb_broadcast_model(const float* z, float* const* w_dev_array, int k, long long n, cudaStream_t st);
XB_API int xb_sync_args_size();

struct XbExec {
  std::vector<XbLearner*> learners;
  std::vector<float*> w, prev;
  XbSolverState solver;
  unsigned long long seed = 0;
  XbSyncDescMirror tmpl;
  // Bucketed synchronous SGD: one descriptor per gradient bucket (its own exchange buffers and flags, vector pointers
  // already moved to the bucket's first element); replica pointers are moved by bucket_off[b] floats.
  std::vector<XbSyncDescMirror> buckets;
  std::vector<long long> bucket_off;
  unsigned int launches = 0;   // picks the pinned staging slot of a launch
  int update_mode = 0;         // 0 averaging kernel, 1 broadcast z (DEFAULT)
  void* args_dev = nullptr; char* args_pinned = nullptr; int args_stride = 0; int max_blocks = 0;
  float** w_table_dev = nullptr;
  cudaStream_t sync_stream = nullptr; cudaEvent_t sync_event = nullptr;
  unsigned int epoch = 0;
  // Model averaging: the learners' next tasks wait for the kernel's release word (their replicas are corrected) instead of
  // the end of the synchronisation; test tasks, which read the central model, wait for the whole of it.
  int early_release = 0;
  // Training task t of this process is task t * world + rank of the job: the learning-rate schedule and the random
  // streams are indexed with the job-wide number, as the reference's single task counter over all GPUs is.
  int rank = 0, world = 1;
  std::atomic<unsigned long long> bn_updates{0};
  // ring data set in pinned memory: [phase]
  const char* ex_base[2] = {nullptr, nullptr}; const char* lab_base[2] = {nullptr, nullptr};
  long long ex_bytes[2] = {0, 0}, lab_bytes[2] = {0, 0}, ring[2] = {0, 0}, stride_tasks = 1, offset_tasks = 0;
  void* d_ex[2][64]; void* d_lab[2][64];
  // Input prefetch: the host-to-device copy of a task's examples runs on a copy stream of its own into a second device
  // buffer, so with two tasks of a replica in flight it overlaps the replica's running task; the learner's stream then
  // only does a device-to-device copy into the staging buffer its task graph reads.
  struct Prefetch { cudaStream_t copy = nullptr; void* next = nullptr; cudaEvent_t copied = nullptr, consumed = nullptr; bool used = false; };
  Prefetch pf[2][64];
  int prefetch = 1;
};

XB_API XbExec* xb_exec_create(const XbSolverState* solver, unsigned long long seed, void* sync_stream, int max_blocks) {
  XbExec* e = new XbExec();
  e->solver = *solver; e->seed = seed; e->max_blocks = max_blocks;
  memset(&e->tmpl, 0, sizeof(e->tmpl));
  e->sync_stream = (cudaStream_t)sync_stream;
  cudaEventCreateWithFlags(&e->sync_event, cudaEventDisableTiming);
  e->args_stride = (xb_sync_args_size() + 255) / 256 * 256;
  cudaMalloc(&e->args_dev, e->args_stride);
  cudaHostAlloc((void**)&e->args_pinned, 32 * e->args_stride, cudaHostAllocDefault);
  cudaMalloc((void**)&e->w_table_dev, 16 * sizeof(float*));
  memset(e->d_ex, 0, sizeof(e->d_ex)); memset(e->d_lab, 0, sizeof(e->d_lab));
  return e;
}
XB_API void xb_exec_destroy(XbExec* e) {
  if (!e) return;
  cudaFree(e->args_dev); cudaFreeHost(e->args_pinned); cudaFree(e->w_table_dev); cudaEventDestroy(e->sync_event);
  for (auto& row : e->pf)
    for (auto& pf : row) {
      if (pf.copy) { cudaStreamSynchronize(pf.copy); cudaStreamDestroy(pf.copy); }
      if (pf.next) cudaFree(pf.next);
      if (pf.copied) cudaEventDestroy(pf.copied);
      if (pf.consumed) cudaEventDestroy(pf.consumed);
    }
  delete e;
}
XB_API int xb_exec_add_learner(XbExec* e, XbLearner* l, float* w, float* prev, void* d_ex_train, void* d_lab_train, void* d_ex_test, void* d_lab_test) {
  int i = (int)e->learners.size();
  if (i >= 64) return -1;
  e->learners.push_back(l); e->w.push_back(w); e->prev.push_back(prev);
  e->d_ex[0][i] = d_ex_train; e->d_lab[0][i] = d_lab_train; e->d_ex[1][i] = d_ex_test; e->d_lab[1][i] = d_lab_test;
  return i;
}
XB_API void xb_exec_remove_learner(XbExec* e) { if (!e->learners.empty()) { e->learners.pop_back(); e->w.pop_back(); e->prev.pop_back(); } }
XB_API void xb_exec_set_sync(XbExec* e, const XbSyncDescMirror* tmpl, int update_mode) {
  e->tmpl = *tmpl; e->update_mode = update_mode; e->buckets.clear(); e->bucket_off.clear();
}
// Buckets in the order in which the backward pass completes them; `offset` in floats from the start of the flat vectors.
XB_API int xb_exec_add_bucket(XbExec* e, const XbSyncDescMirror* tmpl, long long offset) {
  if ((int)e->buckets.size() >= XB_MAX_BUCKETS) return -XB_BAD_ARG;
  e->buckets.push_back(*tmpl); e->bucket_off.push_back(offset);
  return (int)e->buckets.size() - 1;
}
XB_API void xb_exec_set_data(XbExec* e, int phase, const void* examples, long long ex_bytes, const void* labels, long long lab_bytes, long long ring,
                             long long stride_tasks, long long offset_tasks) {
  e->ex_base[phase] = (const char*)examples; e->ex_bytes[phase] = ex_bytes; e->lab_base[phase] = (const char*)labels; e->lab_bytes[phase] = lab_bytes;
  e->ring[phase] = ring; e->stride_tasks = stride_tasks; e->offset_tasks = offset_tasks;
}
XB_API int xb_sync_desc_size() { return (int)sizeof(XbSyncDescMirror); }
XB_API int xb_exec_copy_signal(XbExec* e) { return e->solver.copy_signal; }

XB_API int xb_exec_batch(void* ctx, unsigned long long task, int phase, const void** ex, const void** lab) {
  XbExec* e = (XbExec*)ctx;
  if (!e->ex_base[phase] || e->ring[phase] <= 0) { *ex = nullptr; *lab = nullptr; return 0; }
  unsigned long long slot = (task * (unsigned long long)e->stride_tasks + (unsigned long long)e->offset_tasks) % (unsigned long long)e->ring[phase];
  *ex = e->ex_base[phase] + slot * e->ex_bytes[phase];
  *lab = e->lab_base[phase] + slot * e->lab_bytes[phase];
  return 0;
}
XB_API int xb_exec_submit(void* ctx, int learner, const void* ex, const void* lab, unsigned long long task, int phase) {
  XbExec* e = (XbExec*)ctx;
  if (learner < 0 || learner >= (int)e->learners.size()) return -XB_BAD_ARG;
  XbLearner* l = e->learners[learner];
  XbTaskParams p; memset(&p, 0, sizeof(p));
  const bool training = phase == 0;
  const unsigned long long job_task = training ? task * (unsigned long long)e->world + (unsigned long long)e->rank : task;
  p.lr = training ? solver_lr(e->solver, job_task) : 0.f;
  p.momentum = e->solver.momentum; p.weight_decay = e->solver.weight_decay;
  p.bn_factor = 1.0f / (1.0f + (float)(training ? e->bn_updates.fetch_add(1) : e->bn_updates.load()));
  p.clip = e->solver.clip; p.alpha = e->solver.alpha;
  p.task_id = (unsigned)job_task; p.seed_lo = (unsigned)(e->seed & 0xffffffffu); p.seed_hi = (unsigned)(e->seed >> 32);
  p.training = training ? 1 : 0; p.l1 = e->solver.l1; p.nesterov = e->solver.nesterov;
  if (ex && e->prefetch && learner < 64) {
    XbExec::Prefetch& pf = e->pf[phase][learner];
    const size_t bytes = (size_t)e->ex_bytes[phase];
    if (!pf.copy) {
      XB_CUDA_CHECK(cudaStreamCreateWithFlags(&pf.copy, cudaStreamNonBlocking));
      XB_CUDA_CHECK(cudaMalloc(&pf.next, bytes));
      XB_CUDA_CHECK(cudaEventCreateWithFlags(&pf.copied, cudaEventDisableTiming));
      XB_CUDA_CHECK(cudaEventCreateWithFlags(&pf.consumed, cudaEventDisableTiming));
    }
    if (pf.used) XB_CUDA_CHECK(cudaStreamWaitEvent(pf.copy, pf.consumed, 0));       // the previous task has taken its batch out of `next`
    XB_CUDA_CHECK(cudaMemcpyAsync(pf.next, ex, bytes, cudaMemcpyHostToDevice, pf.copy));
    XB_CUDA_CHECK(cudaEventRecord(pf.copied, pf.copy));
    XB_CUDA_CHECK(cudaStreamWaitEvent(l->stream, pf.copied, 0));
    XB_CUDA_CHECK(cudaMemcpyAsync(e->d_ex[phase][learner], pf.next, bytes, cudaMemcpyDeviceToDevice, l->stream));
    XB_CUDA_CHECK(cudaEventRecord(pf.consumed, l->stream));
    pf.used = true;
  } else if (ex) {
    XB_CUDA_CHECK(cudaMemcpyAsync(e->d_ex[phase][learner], ex, (size_t)e->ex_bytes[phase], cudaMemcpyHostToDevice, l->stream));
  }
  if (lab) XB_CUDA_CHECK(cudaMemcpyAsync(e->d_lab[phase][learner], lab, (size_t)e->lab_bytes[phase], cudaMemcpyHostToDevice, l->stream));
  if (!training && e->early_release) XB_CUDA_CHECK(cudaStreamWaitEvent(l->stream, e->sync_event, 0));   // reads the central model
  return learner_submit_tagged(l, nullptr, nullptr, &p, phase, task);
}
XB_API void xb_exec_set_prefetch(XbExec* e, int on) { e->prefetch = on ? 1 : 0; }
XB_API void xb_exec_set_early_release(XbExec* e, int on) { e->early_release = on ? 1 : 0; }
XB_API void xb_exec_set_rank(XbExec* e, int rank, int world) { e->world = world < 1 ? 1 : world; e->rank = rank; }
XB_API int xb_exec_wait(void* ctx, int learner, float* loss, float* acc) {
  XbExec* e = (XbExec*)ctx;
  if (learner < 0 || learner >= (int)e->learners.size()) return -XB_BAD_ARG;
  return xb_learner_wait(e->learners[learner], loss, acc);
}
XB_API int xb_exec_wait_task(void* ctx, int learner, unsigned long long task, float* loss, float* acc) {
  XbExec* e = (XbExec*)ctx;
  if (learner < 0 || learner >= (int)e->learners.size()) return -XB_BAD_ARG;
  return xb_learner_wait_task(e->learners[learner], task, -1, loss, acc);
}
XB_API int xb_exec_synchronise(void* ctx, unsigned long long clock, const unsigned char* mask, int n, int copy) {
  XbExec* e = (XbExec*)ctx;
  (void)clock;
  XbSyncDescMirror d = e->tmpl;
  int k = 0;
  const bool bucketed = !e->buckets.empty() && e->update_mode == 0;
  for (int i = 0; i < n && i < (int)e->learners.size(); ++i) {
    if (!mask[i]) continue;
    if (k >= 16) return -XB_BAD_ARG;
    if (!bucketed) XB_CUDA_CHECK(cudaStreamWaitEvent(e->sync_stream, e->learners[i]->done, 0));
    d.w[k] = e->w[i]; d.prev[k] = e->prev[i]; ++k;
  }
  if (k == 0) return 0;
  d.k = k;
  if (bucketed) {
    // each bucket's exchange starts as soon as every participating learner has produced that bucket's gradients, while
    // the learners are still in the backward pass of the earlier layers
    const unsigned int epoch = ++e->epoch;
    const int copy_now = (copy || e->solver.copy_signal) ? 1 : 0;
    e->solver.copy_signal = 0;
    for (size_t b = 0; b < e->buckets.size(); ++b) {
      XbSyncDescMirror db = e->buckets[b];
      int kk = 0;
      for (int i = 0; i < n && i < (int)e->learners.size(); ++i) {
        if (!mask[i]) continue;
        { int r = xb_stream_wait_learner_bucket(e->sync_stream, e->learners[i], (int)b); if (r) return r; }
        db.w[kk] = e->w[i] + e->bucket_off[b]; db.prev[kk] = e->prev[i] + e->bucket_off[b]; ++kk;
      }
      db.k = kk; db.epoch = epoch; db.copy_to_replicas = copy_now;
      int r = xb_fused_sync(&db, e->args_dev, e->args_pinned + (e->launches++ % 32) * e->args_stride, e->max_blocks, e->sync_stream);
      if (r) return r;
    }
    for (int i = 0; i < n && i < (int)e->learners.size(); ++i)       // (a learner whose program has no marks)
      if (mask[i]) XB_CUDA_CHECK(cudaStreamWaitEvent(e->sync_stream, e->learners[i]->done, 0));
  } else if (e->update_mode == 1) {
    XB_CUDA_CHECK(cudaMemcpyAsync(e->w_table_dev, d.w, sizeof(float*) * k, cudaMemcpyHostToDevice, e->sync_stream));
    int r = xb_broadcast_model(d.z, e->w_table_dev, k, d.n, e->sync_stream);
    if (r) return r;
  } else {
    d.epoch = ++e->epoch;
    d.copy_to_replicas = (copy || e->solver.copy_signal) ? 1 : 0;
    e->solver.copy_signal = 0;
    if (d.algo == 2) { d.scale = 1.0f / (float)(k * d.G); d.blend = 1.0f / (float)d.epoch; }
    int r = xb_fused_sync(&d, e->args_dev, e->args_pinned + (e->launches++ % 32) * e->args_stride, e->max_blocks, e->sync_stream);
    if (r) return r;
  }
  XB_CUDA_CHECK(cudaEventRecord(e->sync_event, e->sync_stream));
  // averaging without a replica overwrite, several GPUs: a replica is final once the kernel's phase 1 is through
  const bool early = e->early_release && !bucketed && e->update_mode == 0 && d.algo == 0 && !d.copy_to_replicas && d.G > 1 && d.release;
  for (int i = 0; i < n && i < (int)e->learners.size(); ++i) {
    if (!mask[i]) continue;
    if (early) { int r = xb_stream_wait_value32(e->learners[i]->stream, d.release, d.epoch); if (r) return r; }
    else XB_CUDA_CHECK(cudaStreamWaitEvent(e->learners[i]->stream, e->sync_event, 0));
  }
  return 0;
}
XB_API unsigned int xb_exec_epoch(XbExec* e) { return e->epoch; }
XB_API void xb_exec_set_epoch(XbExec* e, unsigned int epoch) { e->epoch = epoch; }

// ---- page-locking of host memory owned by the data-set pipeline (mapped partition files, slot rings) -----------------
// Signature int(void*, size_t) matches the registration hooks of the host runtime's data sets.
XB_API int xb_host_register(void* p, size_t bytes) {
  cudaError_t e = cudaHostRegister(p, bytes, cudaHostRegisterPortable);
  if (e == cudaErrorHostMemoryAlreadyRegistered) { cudaGetLastError(); return 0; }
  return (int)e;
}
XB_API int xb_host_unregister(void* p, size_t) {
  cudaError_t e = cudaHostUnregister(p);
  if (e == cudaErrorHostMemoryNotRegistered) { cudaGetLastError(); return 0; }
  return (int)e;
}
