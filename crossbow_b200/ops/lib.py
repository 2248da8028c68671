"""ctypes binding of ``libxbow_cuda.so`` (kernels + device program executor).

The library is built in-tree on first use (see ``build.py``).  On a machine with a GPU a missing or unloadable
library is a hard error: there is no PyTorch fallback for the device path.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

from . import build as _build

c_void_p, c_int, c_float, c_ll, c_uint = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_uint


class XbConvGeom(C.Structure):
    _fields_ = [(n, c_int) for n in ("N", "H", "W", "C", "K", "R", "S", "P", "Q", "sh", "sw", "ph", "pw")]


class XbTaskParams(C.Structure):
    _fields_ = [("lr", c_float), ("momentum", c_float), ("weight_decay", c_float), ("bn_factor", c_float),
                ("clip", c_float), ("alpha", c_float), ("task_id", c_uint), ("seed_lo", c_uint), ("seed_hi", c_uint),
                ("training", c_int), ("l1", c_int), ("nesterov", c_int)]


class XbOp(C.Structure):
    _fields_ = [("kind", c_int), ("flags", c_int), ("ia", c_int * 16), ("fa", c_float * 8), ("la", c_ll * 4),
                ("p", c_void_p * 12)]


class XbTransposeDesc(C.Structure):
    _fields_ = [("src_off", c_ll), ("dst_off", c_ll), ("K", c_int), ("RS", c_int), ("C", c_int), ("first_block", c_int)]


MAXK, MAXG = 16, 8


class XbSyncDesc(C.Structure):
    _fields_ = [("rank", c_int), ("G", c_int), ("k", c_int), ("algo", c_int), ("n", c_ll), ("epoch", c_uint),
                ("two_shot", c_int), ("copy_to_replicas", c_int), ("use_prev", c_int),
                ("alpha", c_float), ("mu", c_float), ("scale", c_float), ("blend", c_float),
                ("w", c_void_p * MAXK), ("prev", c_void_p * MAXK), ("z", c_void_p), ("zlast", c_void_p), ("gacc", c_void_p),
                ("inbox", c_void_p * MAXG), ("result", c_void_p * MAXG), ("flags", c_void_p * MAXG),
                ("status", c_void_p), ("timeout_s", C.c_double), ("zpeer", c_void_p * MAXG),
                ("part_local", c_void_p), ("part_mc", c_void_p), ("z_mc", c_void_p),
                ("release", c_void_p), ("stamps", c_void_p)]


class XbBnFuse(C.Structure):
    _fields_ = [("x", c_void_p), ("y", c_void_p), ("mean", c_void_p), ("istd", c_void_p), ("sums", c_void_p), ("relu", c_int)]


class XbSolverState(C.Structure):
    _fields_ = [("policy", c_int), ("base_lr", c_float), ("gamma", c_float), ("power", c_float), ("momentum", c_float),
                ("weight_decay", c_float), ("clip", c_float), ("alpha", c_float), ("step_size", c_ll), ("warmup", c_ll),
                ("nsteps", c_int), ("steps", c_ll * 32), ("l1", c_int), ("nesterov", c_int), ("cma", c_int),
                ("step_cursor", c_int), ("copy_signal", c_int)]


# op kinds (csrc/runtime/program.cu)
(OP_MEMSET, OP_UPLOAD, OP_TRANSFORM, OP_CONV_FPROP, OP_CONV_DGRAD, OP_CONV_WGRAD, OP_COLSUM, OP_BN_STATS, OP_BN_FWD,
 OP_BN_BWD, OP_ACT_FWD, OP_ACT_BWD, OP_SUM, OP_DROPOUT, OP_CONCAT, OP_POOL_FWD, OP_POOL_BWD, OP_LRN_FWD, OP_LRN_BWD,
 OP_SOFTMAX_XENT, OP_CLASSIFY, OP_TRANSPOSE_W, OP_GRAD_SUMSQ, OP_OPTIMISER, OP_COPY, OP_MATFACT, OP_MARK) = range(27)

F_RELU, F_ACCUM, F_STATS, F_TC = 1, 2, 4, 0x100
F_SIDE = 0x1000          # operator runs on a parallel branch of the captured task graph (csrc/runtime/program.cu)
F_JOIN = 0x2000          # operator of the main chain that reads what the branch has produced so far: the branch is joined in front of it

_lib: Optional[C.CDLL] = None


def _sig(lib, name, restype, *argtypes):
    f = getattr(lib, name)
    f.restype = restype
    f.argtypes = list(argtypes)
    return f


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    path = _build.build_cuda()
    lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
    P, I, F, L = c_void_p, c_int, c_float, c_ll
    G = C.POINTER(XbConvGeom)
    _sig(lib, "xb_conv_fprop_simt", I, P, P, P, P, P, G, I, P)
    _sig(lib, "xb_conv_dgrad_simt", I, P, P, P, G, I, P)
    _sig(lib, "xb_conv_wgrad_simt", I, P, P, P, G, P)
    _sig(lib, "xb_conv_fprop_tc", I, P, P, P, P, P, G, I, P, P)
    _sig(lib, "xb_conv_dgrad_tc", I, P, P, P, G, I, P, P, P)
    _sig(lib, "xb_conv_dgrad_fuses_bn", I, G)
    _sig(lib, "xb_conv_wgrad_tc", I, P, P, P, G, P, P)
    _sig(lib, "xb_tc_supported", I, G, I)
    _sig(lib, "xb_tc_init", I)
    _sig(lib, "xb_tc_set_slab", None, I)
    _sig(lib, "xb_tc_set_tma", None, I)
    _sig(lib, "xb_sleep", I, C.c_longlong, P)
    _sig(lib, "xb_gemm_set_tn_ctas", None, I)
    _sig(lib, "xb_gemm_set_split_k", None, I)
    _sig(lib, "xb_gemm_set_max_bn", None, I, I)
    _sig(lib, "xb_set_pdl", None, I)
    _sig(lib, "xb_get_pdl", I)
    _sig(lib, "xb_conv3x3_wgrad_set_ctas", None, I)
    _sig(lib, "xb_bn_set_stream_blocks", None, I)
    _sig(lib, "xb_bn_set_reduce_blocks", None, I)
    _sig(lib, "xb_tc_set_tma_conv_min", None, I)
    _sig(lib, "xb_conv_tma_supported", I, G, I)
    _sig(lib, "xb_conv_im2col_wanted", C.c_longlong, G, I)
    _sig(lib, "xb_conv3x3_s2_dgrad_scratch", C.c_longlong, G)
    _sig(lib, "xb_conv3x3_s2_dgrad", I, P, P, P, G, I, P, P, P, P)
    _sig(lib, "xb_conv_im2col_scratch", C.c_longlong, G, I)
    _sig(lib, "xb_conv_fprop_im2col", I, P, P, P, P, P, G, I, P, P, P)
    _sig(lib, "xb_conv_wgrad_im2col", I, P, P, P, G, P, I, P, P)
    _sig(lib, "xb_conv1x1_tma_supported", I, G, I)
    _sig(lib, "xb_conv3x3_slab_supported", I, G, I)
    _sig(lib, "xb_transpose_weights", I, P, P, P, I, I, P)
    _sig(lib, "xb_transpose_blocks", I, I, I, I)
    _sig(lib, "xb_bn_stats", I, P, P, I, I, P)
    _sig(lib, "xb_bn_forward", I, P, P, P, P, P, P, P, P, P, P, P, I, I, F, I, I, I, F, P)
    _sig(lib, "xb_bn_forward_mask", I, P, P, P, P, P, P, P, P, P, P, P, I, I, F, I, I, I, F, P, P)
    _sig(lib, "xb_bn_backward", I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P)
    _sig(lib, "xb_act_forward", I, P, P, L, I, F, F, P)
    _sig(lib, "xb_act_backward", I, P, P, P, P, L, I, F, F, I, P)
    _sig(lib, "xb_weighted_sum", I, P, P, I, P, L, I, P)
    _sig(lib, "xb_dropout", I, P, P, L, F, c_uint, P, I, P)
    _sig(lib, "xb_concat_copy", I, P, P, L, I, I, I, I, I, P)
    _sig(lib, "xb_pool_forward", I, P, P, P, I, P)
    _sig(lib, "xb_pool_backward", I, P, P, P, P, I, I, P)
    _sig(lib, "xb_lrn_forward", I, P, P, P, L, I, I, F, F, F, P)
    _sig(lib, "xb_lrn_backward", I, P, P, P, P, P, L, I, I, F, F, I, P)
    _sig(lib, "xb_transform", I, P, P, P, I, I, I, I, I, I, I, I, F, I, c_uint, P, P)
    _sig(lib, "xb_nhwc_to_nchw", I, P, P, I, I, I, I, P)
    _sig(lib, "xb_colsum", I, P, P, I, I, P)
    _sig(lib, "xb_softmax_xent", I, P, P, P, P, P, I, I, I, I, I, I, P)
    _sig(lib, "xb_classify", I, P, P, I, I, P)
    _sig(lib, "xb_grad_sumsq", I, P, P, L, P)
    _sig(lib, "xb_fused_optimiser", I, P, P, P, P, P, P, P, P, L, I, P)
    _sig(lib, "xb_image_desc_size", I)
    _sig(lib, "xb_image_crop_resize", I, P, P, I, I, P, P)
    # sync
    _sig(lib, "xb_sync_chunk", L, L)
    _sig(lib, "xb_sync_nchunks", L, L)
    _sig(lib, "xb_sync_inbox_floats", L, L, I, I)
    _sig(lib, "xb_sync_result_floats", L, L)
    _sig(lib, "xb_sync_flag_words", L, L, I)
    _sig(lib, "xb_sync_args_size", I)
    _sig(lib, "xb_sync_part_floats", L, L)
    _sig(lib, "xb_fused_sync", I, C.POINTER(XbSyncDesc), P, P, I, P)
    _sig(lib, "xb_fused_sync_emulated", I, C.POINTER(XbSyncDesc), I, P, I, P)
    _sig(lib, "xb_broadcast_model", I, P, P, I, L, P)
    _sig(lib, "xb_peer_copy", I, P, P, L, I, P)
    _sig(lib, "xb_peer_copy_all", I, P, P, I, L, I, P)
    _sig(lib, "xb_sync_set_large_chunk", None, I)
    _sig(lib, "xb_gemm_set_smem_budgets", None, I, I)
    _sig(lib, "xb_stream_wait_value32", I, P, P, c_uint)
    _sig(lib, "xb_stream_wait_value_supported", I)
    _sig(lib, "xb_sync_stamp_words", I)
    _sig(lib, "xb_exec_set_early_release", None, P, I)
    _sig(lib, "xb_exec_set_rank", None, P, I, I)
    # program / learner
    _sig(lib, "xb_op_size", I)
    _sig(lib, "xb_program_create", P, C.POINTER(XbOp), I, I, P)
    _sig(lib, "xb_program_destroy", None, P)
    _sig(lib, "xb_program_launches", I, P)
    _sig(lib, "xb_program_num_ops", I, P)
    _sig(lib, "xb_program_run", I, P, P)
    _sig(lib, "xb_program_run_range", I, P, I, I, P)
    _sig(lib, "xb_program_capture", I, P, P)
    _sig(lib, "xb_program_marks", I, P)
    _sig(lib, "xb_program_side_priority", None, I)
    _sig(lib, "xb_program_launch", I, P, P)
    _sig(lib, "xb_learner_create", P, I, P, L, P, L)
    _sig(lib, "xb_learner_destroy", None, P)
    _sig(lib, "xb_learner_stream", P, P)
    _sig(lib, "xb_learner_params", C.POINTER(XbTaskParams), P)
    _sig(lib, "xb_learner_result_host", C.POINTER(c_float), P)
    _sig(lib, "xb_learner_result_dev", P, P)
    _sig(lib, "xb_learner_set_programs", None, P, P, P)
    _sig(lib, "xb_learner_submit", I, P, P, P, C.POINTER(XbTaskParams), I)
    _sig(lib, "xb_learner_wait", I, P, C.POINTER(c_float), C.POINTER(c_float))
    _sig(lib, "xb_learner_query", I, P)
    _sig(lib, "xb_stream_wait_learner", I, P, P)
    _sig(lib, "xb_stream_wait_learner_bucket", I, P, P, I)
    _sig(lib, "xb_learner_wait_event", I, P, P)
    # native executor (function-pointer table for the host runtime)
    _sig(lib, "xb_exec_create", P, C.POINTER(XbSolverState), C.c_ulonglong, P, I)
    _sig(lib, "xb_exec_destroy", None, P)
    _sig(lib, "xb_exec_add_learner", I, P, P, P, P, P, P, P, P)
    _sig(lib, "xb_exec_remove_learner", None, P)
    _sig(lib, "xb_exec_set_sync", None, P, C.POINTER(XbSyncDesc), I)
    _sig(lib, "xb_exec_add_bucket", I, P, C.POINTER(XbSyncDesc), C.c_longlong)
    _sig(lib, "xb_exec_set_data", None, P, I, P, L, P, L, L, L, L)
    _sig(lib, "xb_sync_desc_size", I)
    _sig(lib, "xb_exec_copy_signal", I, P)
    _sig(lib, "xb_exec_epoch", c_uint, P)
    _sig(lib, "xb_exec_submit", I, P, I, P, P, C.c_ulonglong, I)
    _sig(lib, "xb_exec_synchronise", I, P, C.c_ulonglong, P, I, I)
    _sig(lib, "xb_optimiser_set_blocks", None, I)
    _sig(lib, "xb_trace_set", None, I)
    _sig(lib, "xb_trace_level", I)
    _sig(lib, "xb_trace_read", I, I, C.POINTER(c_float), I, I)
    _sig(lib, "xb_learner_wait_task", I, P, C.c_ulonglong, I, C.POINTER(c_float), C.POINTER(c_float))
    _sig(lib, "xb_exec_set_epoch", None, P, c_uint)
    assert lib.xb_sync_desc_size() == C.sizeof(XbSyncDesc), (lib.xb_sync_desc_size(), C.sizeof(XbSyncDesc))
    # plumbing
    _sig(lib, "xb_stream_create", P, I)
    _sig(lib, "xb_stream_destroy", I, P)
    _sig(lib, "xb_stream_sync", I, P)
    _sig(lib, "xb_event_create", P, I)
    _sig(lib, "xb_event_destroy", I, P)
    _sig(lib, "xb_event_record", I, P, P)
    _sig(lib, "xb_event_sync", I, P)
    _sig(lib, "xb_stream_wait_event", I, P, P)
    _sig(lib, "xb_event_elapsed_ms", F, P, P)
    _sig(lib, "xb_pinned_alloc", P, L)
    _sig(lib, "xb_pinned_free", I, P)
    _sig(lib, "xb_device_alloc", P, L)
    _sig(lib, "xb_device_free", I, P)
    _sig(lib, "xb_memcpy_h2d_async", I, P, P, L, P)
    _sig(lib, "xb_memcpy_d2h_async", I, P, P, L, P)
    _sig(lib, "xb_memcpy_d2d_async", I, P, P, L, P)
    _sig(lib, "xb_device_sync", I)
    _sig(lib, "xb_set_device", I, I)
    _sig(lib, "xb_error_string", C.c_char_p, I)
    _sig(lib, "xb_last_error", I)
    _sig(lib, "xb_ipc_export", I, P, P)
    _sig(lib, "xb_ipc_import", P, P)
    _sig(lib, "xb_ipc_close", I, P)
    assert lib.xb_op_size() == C.sizeof(XbOp), (lib.xb_op_size(), C.sizeof(XbOp))
    _lib = lib
    return lib


_tc_ready = False


def init_device():
    """Per-process device set-up that must happen outside stream capture (shared-memory opt-in of the tcgen05 kernels)."""
    global _tc_ready
    lib = load()
    if not _tc_ready:
        check(lib.xb_tc_init(), "tensor-core kernel set-up")
        if os.environ.get("XBOW_PDL", "") != "":             # programmatic dependent launch between a task's kernels: 1 on, 0 off
            lib.xb_set_pdl(int(os.environ["XBOW_PDL"]))
        _tc_ready = True
    return lib


class CudaError(RuntimeError):
    pass


def check(code: int, what: str = ""):
    """Raise on a non-zero return of a native call. Program runs encode the failing op as 1000*(index+1)+error."""
    if code == 0:
        return
    lib = load()
    if code >= 1000:
        op, err = code // 1000 - 1, code % 1000
        msg = lib.xb_error_string(err).decode() if err > 3 else f"status {err}"
        raise CudaError(f"{what}: op #{op} failed: {msg}")
    err = -code if code < 0 else code
    msg = lib.xb_error_string(err).decode() if code > 0 else f"bad argument / status {err}"
    raise CudaError(f"{what}: {msg} ({code})")


def ptr(t) -> int:
    """Device (or pinned host) address of a torch tensor, 0 for None."""
    return 0 if t is None else t.data_ptr()
