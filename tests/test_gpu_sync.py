"""Fused synchronisation kernel: single rank, and several ranks emulated in ONE cooperative launch on one GPU
(kernels that wait on one another must never be separate launches on a shared GPU)."""
import ctypes as C

import numpy as np
import pytest
import torch

from crossbow_b200.oracle import DeviceState, ReplicaState, synchronise_sma, synchronise_ssgd, synchronise_polyak_ruppert

pytestmark = pytest.mark.gpu


def _state(G, k, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    devs = []
    base = torch.randn(n, generator=g) * 0.01
    for d in range(G):
        dv = DeviceState(base)
        dv.z_last = torch.randn(n, generator=g) * 0.001
        dv.G = torch.randn(n, generator=g) * 0.01
        for r in range(k):
            rs = ReplicaState(base + torch.randn(n, generator=g) * 0.01)
            rs.prev = base + torch.randn(n, generator=g) * 0.01
            dv.replicas.append(rs)
        devs.append(dv)
    # z_last must be identical on all devices for the devices to stay in step
    for dv in devs[1:]:
        dv.z_last = devs[0].z_last.clone()
    return devs


def _run_emulated(devs, n, algo, two_shot, epochs=3, **kw):
    from crossbow_b200.ops import lib as L
    lib = L.load()
    G, k = len(devs), len(devs[0].replicas)
    dev = torch.device("cuda")
    W = [[r.w.to(dev) for r in d.replicas] for d in devs]
    Pv = [[r.prev.to(dev) for r in d.replicas] for d in devs]
    Z = [d.z.to(dev) for d in devs]
    ZL = [d.z_last.to(dev) for d in devs]
    GA = [d.G.to(dev) for d in devs]
    inbox = [torch.zeros(lib.xb_sync_inbox_floats(n, G, int(two_shot)), device=dev) for _ in range(G)]
    result = [torch.zeros(lib.xb_sync_result_floats(n), device=dev) for _ in range(G)]
    flags = [torch.zeros(lib.xb_sync_flag_words(n, G), dtype=torch.int32, device=dev) for _ in range(G)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    args = torch.zeros(lib.xb_sync_args_size() * G, dtype=torch.uint8, device=dev)
    descs = (L.XbSyncDesc * G)()
    for e in range(1, epochs + 1):
        for g in range(G):
            d = descs[g]
            d.rank, d.G, d.k, d.algo, d.n, d.epoch = g, G, k, algo, n, e
            d.two_shot, d.copy_to_replicas, d.use_prev = int(two_shot), int(kw.get("copy", False)), int(kw.get("use_prev", True))
            d.alpha, d.mu, d.scale, d.blend = kw.get("alpha", 0.0), kw.get("mu", 0.0), kw.get("scale", 1.0), kw.get("blend", 0.0)
            for i in range(k):
                d.w[i], d.prev[i] = W[g][i].data_ptr(), Pv[g][i].data_ptr()
            d.z, d.zlast, d.gacc = Z[g].data_ptr(), ZL[g].data_ptr(), GA[g].data_ptr()
            for j in range(G):
                d.inbox[j], d.result[j], d.flags[j] = inbox[j].data_ptr(), result[j].data_ptr(), flags[j].data_ptr()
                d.zpeer[j] = Z[j].data_ptr() if kw.get("owner_apply", False) else None
            d.status, d.timeout_s = status.data_ptr(), 2.0
        L.check(lib.xb_fused_sync_emulated(descs, G, args.data_ptr(), 8, torch.cuda.current_stream().cuda_stream), "emulated sync")
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        yield e, W, Z, ZL, GA


@pytest.mark.parametrize("G,k,two_shot", [(1, 2, False), (2, 2, False), (4, 3, False), (4, 2, True), (8, 1, True), (8, 2, False)])
def test_sma_matches_oracle(G, k, two_shot):
    n = 4096 * 5 + 1024     # not a multiple of the chunk size
    devs = _state(G, k, n)
    for e, W, Z, ZL, GA in _run_emulated(devs, n, 0, two_shot, alpha=0.1, mu=0.9):
        synchronise_sma(devs, 0.1, 0.9)
        for g in range(G):
            assert torch.allclose(Z[g].cpu(), devs[g].z, rtol=1e-5, atol=1e-6), f"epoch {e} z[{g}]"
            assert torch.allclose(ZL[g].cpu(), devs[g].z_last, rtol=1e-5, atol=1e-6)
            for i in range(k):
                assert torch.allclose(W[g][i].cpu(), devs[g].replicas[i].w, rtol=1e-5, atol=1e-6)
        # all GPUs hold bit-identical central models
        for g in range(1, G):
            assert torch.equal(Z[g], Z[0])


def _owned(n, G, g):
    """Mask of the elements whose chunk belongs to rank g (chunk c -> rank c mod G)."""
    from crossbow_b200.ops import lib as L
    chunk = int(L.load().xb_sync_chunk(n))
    return ((torch.arange(n) // chunk) % G) == g


@pytest.mark.parametrize("G,k,algo,n", [(2, 2, 0, 4096 * 9 + 2048), (4, 1, 0, 4096 * 9 + 2048), (8, 2, 0, 4096 * 9 + 2048),
                                        (4, 2, 1, 4096 * 9 + 2048), (4, 2, 2, 4096 * 9 + 2048),
                                        (2, 1, 0, (4 << 20) + 32768 * 5 + 4096 + 8), (3, 2, 0, (4 << 20) + 32768 * 2 + 12)])
def test_owner_apply_matches_oracle(G, k, algo, n):
    """Two-shot exchange in which the owner of a chunk updates the central model and stores it on every GPU; the
    momentum of the central model is then kept by the owners only.  Small vectors use 16 KB chunks; the two cases above four
    million elements use 128 KB chunks, eight steps per chunk, with a ragged last chunk."""
    devs = _state(G, k, n, seed=7)
    kw = {0: dict(alpha=0.1, mu=0.9), 1: dict(mu=0.9, scale=1.0 / (G * k)), 2: dict(alpha=0.05, scale=1.0 / (G * k), blend=1.0, epochs=1)}[algo]
    for e, W, Z, ZL, GA in _run_emulated(devs, n, algo, True, owner_apply=True, **kw):
        if algo == 0:
            synchronise_sma(devs, 0.1, 0.9)
        elif algo == 1:
            synchronise_ssgd(devs, G * k, 0.9)
        else:
            synchronise_polyak_ruppert(devs, 0.05)
        for g in range(G):
            assert torch.allclose(Z[g].cpu(), devs[g].z, rtol=1e-5, atol=1e-6), f"epoch {e} z[{g}]"
            if algo != 2:
                own = _owned(n, G, g)
                assert torch.allclose(ZL[g].cpu()[own], devs[g].z_last[own], rtol=1e-5, atol=1e-6)
            for i in range(k):
                assert torch.allclose(W[g][i].cpu(), devs[g].replicas[i].w, rtol=1e-5, atol=1e-6)
        for g in range(1, G):
            assert torch.equal(Z[g], Z[0])


def test_sma_copy_and_current_weights():
    n = 4096 * 3
    devs = _state(2, 2, n, seed=1)
    for e, W, Z, ZL, GA in _run_emulated(devs, n, 0, False, epochs=1, alpha=0.2, mu=0.0, copy=True, use_prev=False):
        synchronise_sma(devs, 0.2, 0.0, copy=True, use_prev=False)
        for g in range(2):
            assert torch.allclose(Z[g].cpu(), devs[g].z, rtol=1e-5, atol=1e-6)
            for i in range(2):
                assert torch.equal(W[g][i], Z[g])


@pytest.mark.parametrize("two_shot", [False, True])
def test_ssgd_matches_oracle(two_shot):
    n = 4096 * 4
    devs = _state(4, 2, n, seed=2)
    for e, W, Z, ZL, GA in _run_emulated(devs, n, 1, two_shot, epochs=1, mu=0.9, scale=1.0 / 8):
        synchronise_ssgd(devs, 8, 0.9)
        for g in range(4):
            assert torch.allclose(Z[g].cpu(), devs[g].z, rtol=1e-5, atol=1e-6)
            assert float(GA[g].abs().max()) == 0.0
            for i in range(2):
                assert torch.equal(W[g][i], Z[g])


def test_polyak_matches_oracle():
    n = 4096 * 2
    devs = _state(2, 2, n, seed=3)
    for e, W, Z, ZL, GA in _run_emulated(devs, n, 2, False, epochs=1, scale=1.0 / 4, blend=1.0):
        synchronise_polyak_ruppert(devs, 0.0)
        for g in range(2):
            assert torch.allclose(Z[g].cpu(), devs[g].z, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("G,k,two_shot", [(2, 2, False), (4, 2, True)])
def test_release_word_orders_the_next_task(G, k, two_shot):
    """Model averaging releases a GPU's replicas before the exchange: a second stream that waits for the release word
    and then rewrites the replicas (what a replica's next task does) must see the corrected weights, and the central
    model must come out as if the two had run one after the other.  G ranks emulated in one cooperative launch."""
    from crossbow_b200.ops import lib as L
    lib = L.load()
    assert lib.xb_stream_wait_value_supported() == 1
    n = (1 << 20) + 4096 * 3
    devs = _state(G, k, n, seed=11)
    dev = torch.device("cuda")
    W = [[r.w.to(dev) for r in d.replicas] for d in devs]
    Pv = [[r.prev.to(dev) for r in d.replicas] for d in devs]
    Z = [d.z.to(dev) for d in devs]
    ZL = [d.z_last.to(dev) for d in devs]
    inbox = [torch.zeros(lib.xb_sync_inbox_floats(n, G, int(two_shot)), device=dev) for _ in range(G)]
    result = [torch.zeros(lib.xb_sync_result_floats(n), device=dev) for _ in range(G)]
    flags = [torch.zeros(lib.xb_sync_flag_words(n, G), dtype=torch.int32, device=dev) for _ in range(G)]
    release = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(G)]
    stamps = [torch.zeros(lib.xb_sync_stamp_words(), dtype=torch.int64, device=dev) for _ in range(G)]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    args = torch.zeros(lib.xb_sync_args_size() * G, dtype=torch.uint8, device=dev)
    descs = (L.XbSyncDesc * G)()
    sync_stream, task_stream = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    epochs = 3
    for e in range(1, epochs + 1):
        for g in range(G):
            d = descs[g]
            d.rank, d.G, d.k, d.algo, d.n, d.epoch = g, G, k, 0, n, e
            d.two_shot, d.copy_to_replicas, d.use_prev = int(two_shot), 0, 1
            d.alpha, d.mu, d.scale, d.blend = 0.1, 0.9, 1.0, 0.0
            for i in range(k):
                d.w[i], d.prev[i] = W[g][i].data_ptr(), Pv[g][i].data_ptr()
            d.z, d.zlast, d.gacc = Z[g].data_ptr(), ZL[g].data_ptr(), 0
            for j in range(G):
                d.inbox[j], d.result[j], d.flags[j] = inbox[j].data_ptr(), result[j].data_ptr(), flags[j].data_ptr()
            d.status, d.timeout_s = status.data_ptr(), 2.0
            d.release, d.stamps = release[g].data_ptr(), stamps[g].data_ptr()
        # the synchronisation follows the "tasks" of the previous round (an event), the tasks follow the release word only
        sync_stream.wait_stream(task_stream)
        L.check(lib.xb_fused_sync_emulated(descs, G, args.data_ptr(), 8, sync_stream.cuda_stream), "emulated sync")
        with torch.cuda.stream(task_stream):
            for g in range(G):
                L.check(lib.xb_stream_wait_value32(task_stream.cuda_stream, release[g].data_ptr(), e), "wait for release")
                for i in range(k):
                    Pv[g][i].copy_(W[g][i])          # the next task's optimiser: snapshot, then a step
                    W[g][i].mul_(1.5)
        # oracle: synchronise, then the same "task"
        synchronise_sma(devs, 0.1, 0.9)
        for dv in devs:
            for r in dv.replicas:
                r.prev = r.w.clone()
                r.w = r.w * 1.5
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for g in range(G):
        assert torch.allclose(Z[g].cpu(), devs[g].z, rtol=1e-5, atol=1e-6)
        assert torch.equal(Z[g], Z[0])
        for i in range(k):
            assert torch.allclose(W[g][i].cpu(), devs[g].replicas[i].w, rtol=1e-5, atol=1e-6)
        st = stamps[g].cpu().tolist()
        assert int(release[g][0].item()) == epochs and int(release[g][1].item()) == 0
        assert st[4] == epochs - 1 and 0 < st[5] <= st[6]             # launches folded so far; entry->release <= entry->exit
        assert st[0] < st[1] <= st[2 + (epochs & 1)]                  # last launch: entry < release <= exit


def test_wait_gives_up_with_status():
    """A flag that nothing sets: the kernel must return with a status, not hang."""
    from crossbow_b200.ops import lib as L
    lib = L.load()
    n, G = 4096, 2
    dev = torch.device("cuda")
    w, z, zl = torch.zeros(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    inbox = torch.zeros(lib.xb_sync_inbox_floats(n, G, 0), device=dev)
    result = torch.zeros(lib.xb_sync_result_floats(n), device=dev)
    flags = torch.zeros(lib.xb_sync_flag_words(n, G), dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    args = torch.zeros(lib.xb_sync_args_size(), dtype=torch.uint8, device=dev)
    pinned = torch.zeros(lib.xb_sync_args_size(), dtype=torch.uint8).pin_memory()
    d = L.XbSyncDesc()
    d.rank, d.G, d.k, d.algo, d.n, d.epoch = 0, G, 1, 0, n, 1
    d.w[0], d.prev[0], d.z, d.zlast = w.data_ptr(), w.data_ptr(), z.data_ptr(), zl.data_ptr()
    # the "peer" is a second set of buffers on this GPU that no kernel ever writes flags into
    peer_inbox, peer_flags = torch.zeros_like(inbox), torch.zeros_like(flags)
    d.inbox[0], d.inbox[1] = inbox.data_ptr(), peer_inbox.data_ptr()
    d.result[0], d.result[1] = result.data_ptr(), result.data_ptr()
    d.flags[0], d.flags[1] = flags.data_ptr(), peer_flags.data_ptr()
    d.status, d.timeout_s = status.data_ptr(), 0.2
    L.check(lib.xb_fused_sync(C.byref(d), args.data_ptr(), pinned.data_ptr(), 4, torch.cuda.current_stream().cuda_stream), "sync")
    torch.cuda.synchronize()
    assert int(status.item()) == 1        # XB_TIMEOUT_FLAG
    assert float(z.abs().max()) == 0.0    # the chunk was skipped


def test_engine_fused_equals_reference_sync():
    from crossbow_b200 import Phase, UpdateModel
    from crossbow_b200.parallel.sync import ReferenceSynchroniser
    from helpers import engines, make_batches
    spec, m, gpu, _ = engines("lenet-caffe", 8, k=2)
    try:
        xs, ys = make_batches(spec, 8, 2)
        for t in range(2):
            gpu.submit(t, xs[t].pin_memory(), ys[t].pin_memory(), t, Phase.TRAIN)
        gpu.wait(0), gpu.wait(1)
        torch.cuda.synchronize()
        ws = [l.rep.w.clone() for l in gpu.learners]
        z0, zl0 = gpu.shared.z.clone(), gpu.shared.zlast.clone()
        gpu.synchronise()
        gpu.finish()
        ref = ReferenceSynchroniser(m.device_elements)
        ref.synchronise(0, 0, ws, [l.rep.prev for l in gpu.learners], z0, zl0, alpha=0.1, mu=0.9)
        torch.cuda.synchronize()
        assert torch.allclose(z0, gpu.shared.z, rtol=1e-5, atol=1e-7)
        for w, l in zip(ws, gpu.learners):
            assert torch.allclose(w, l.rep.w, rtol=1e-5, atol=1e-7)
    finally:
        gpu.destroy()
