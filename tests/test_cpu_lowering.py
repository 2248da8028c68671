"""The lowering on host tensors (no kernel is launched): placement of the gradient buckets of synchronous SGD, operator
replication for `--splits`, buffer sharing for `--reuse-memory`."""
import bisect

import pytest
import torch

from crossbow_b200 import UpdateModel
from helpers import build_model


def _lower(name="resnet8", batch=8, update_model=UpdateModel.WORKER, **kw):
    from crossbow_b200.lower import DeviceShared, Lowering, ReplicaBuffers
    from crossbow_b200.ops import lib as L
    try:
        L.load()                                     # shape queries (which kernel takes a layer) live in the native library
    except Exception as e:                           # pragma: no cover - a machine where the library cannot be loaded
        pytest.skip(f"native library not loadable here: {e}")
    spec, m, solver = build_model(name, batch)
    dev = torch.device("cpu")
    init = torch.from_numpy(m.to_device(m.initial_values(3)))
    rep, sh = ReplicaBuffers(m, dev, init), DeviceShared(m, dev, init)
    low = Lowering(spec.train, m, batch, spec.input_shape, dev, rep.w, rep, sh, torch.zeros(16, dtype=torch.int32), 0, 0,
                   update_model=update_model, training=True, use_tc=True, **kw)
    return L, m, rep, low


def test_gradient_buckets_cover_the_vector_and_follow_their_last_use():
    L, m, rep, low = _lower(gradient_buckets=3)
    n = m.device_elements
    assert len(low.buckets) >= 2
    # contiguous, disjoint, from the tail of the flat vector to its head (the order in which backward completes them)
    end = n
    for off, ln in low.buckets:
        assert off + ln == end and ln > 0 and off % 4 == 0
        end = off
    assert end == 0
    kinds = [o.kind for o in low.ops]
    marks = [i for i, k in enumerate(kinds) if k == L.OP_MARK]
    opts = [i for i, k in enumerate(kinds) if k == L.OP_OPTIMISER]
    assert len(marks) == len(opts) == len(low.buckets) and [low.ops[i].ia[0] for i in marks] == list(range(len(marks)))
    assert all(mk == op + 1 for mk, op in zip(marks, opts))          # accumulate step, then the mark
    g0, w0 = rep.g.data_ptr(), rep.w.data_ptr()
    for b, (off, ln) in enumerate(low.buckets):
        op = low.ops[opts[b]]
        assert op.ia[0] == 2 and op.la[0] == ln and op.p[0] == w0 + 4 * off and op.p[1] == g0 + 4 * off
        # nothing after the bucket's accumulate step may write its gradients or read its weights: the synchronisation of
        # the bucket overwrites the replica's weights of that range while the learner is still running
        for i in range(opts[b] + 1, len(low.ops)):
            o = low.ops[i]
            if o.kind in (L.OP_OPTIMISER, L.OP_MARK):
                continue
            for a in o.p:
                for base in (g0, w0):
                    assert not (a and base + 4 * off <= a < base + 4 * (off + ln)), (b, i, o.kind)


def test_no_buckets_with_clipping_splits_or_other_update_models():
    assert _lower(gradient_buckets=3, clip=True)[3].buckets == []
    assert _lower(gradient_buckets=3, splits=2)[3].buckets == []
    assert _lower(gradient_buckets=3, update_model=UpdateModel.SMA)[3].buckets == []
    assert _lower(gradient_buckets=1)[3].buckets == []


def test_splits_repeat_the_operator_list_and_reuse_memory_shrinks_the_arena():
    L, m, rep, one = _lower(update_model=UpdateModel.SMA)
    _, _, _, two = _lower(update_model=UpdateModel.SMA, splits=2)
    conv = lambda low: sum(1 for o in low.ops if o.kind == L.OP_CONV_FPROP)
    assert conv(two) == 2 * conv(one)
    assert sum(1 for o in two.ops if o.kind == L.OP_OPTIMISER) == 2      # the whole graph, optimiser included, once per sub-batch
    _, _, _, shared = _lower(update_model=UpdateModel.SMA, reuse_memory=True)
    assert shared.arena.total < 0.8 * one.arena.total and shared.bytes_before_reuse == one.arena.total


def test_rectangular_filters_reach_the_kernels_with_their_geometry():
    """Inception-v3's 1x7 / 7x1 / 1x3 / 3x1 convolutions: (R, S) and (pad_h, pad_w) of the lowered launches."""
    from crossbow_b200.lower import DeviceShared, Lowering, ReplicaBuffers
    from crossbow_b200.ops import lib as L
    try:
        L.load()
    except Exception as e:                           # pragma: no cover
        pytest.skip(f"native library not loadable here: {e}")
    spec, m, solver = build_model("inception-v3", 2, size=139, width=0.25, classes=10)
    dev = torch.device("cpu")
    init = torch.from_numpy(m.to_device(m.initial_values(3)))
    rep, sh = ReplicaBuffers(m, dev, init), DeviceShared(m, dev, init)
    low = Lowering(spec.train, m, 2, spec.input_shape, dev, rep.w, rep, sh, torch.zeros(16, dtype=torch.int32), 0, 0,
                   update_model=UpdateModel.SMA, training=True, use_tc=True)
    shapes = set()
    for o in low.ops:
        if o.kind == L.OP_CONV_FPROP:
            g = L.XbConvGeom.from_buffer_copy(bytes(o.ia)[: 13 * 4])
            shapes.add((g.R, g.S, g.ph, g.pw, g.sh))
            assert g.P == (g.H + 2 * g.ph - g.R) // g.sh + 1 and g.Q == (g.W + 2 * g.pw - g.S) // g.sw + 1
    assert {(7, 1, 3, 0, 1), (1, 7, 0, 3, 1), (3, 1, 1, 0, 1), (1, 3, 0, 1, 1), (3, 3, 0, 0, 2), (5, 5, 2, 2, 1), (1, 1, 0, 0, 1)} <= shapes
    # every convolution has its three launches (the stem has no data gradient)
    n_f = sum(o.kind == L.OP_CONV_FPROP for o in low.ops)
    assert sum(o.kind == L.OP_CONV_WGRAD for o in low.ops) == n_f and sum(o.kind == L.OP_CONV_DGRAD for o in low.ops) == n_f - 1
