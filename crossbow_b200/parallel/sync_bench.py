"""Synchronisation micro-benchmark: fused kernel vs the reference-style sequence, per model size and replica count.

    python -m crossbow_b200.parallel.sync_bench                        # 1 GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m crossbow_b200.parallel.sync_bench

For flat fp32 vectors of 0.46 M (ResNet-32) and 25.6 M (ResNet-50) elements, values N(0, 0.01), k in {1, 2, 4}
replicas per GPU: device time per synchronisation (CUDA events around ``--iters`` back-to-back calls after warm-up,
maximum over ranks) of
  fused      one persistent kernel per GPU: replica reduction + peer-memory all-reduce + central update + correction
  reference  per-replica difference/axpy kernels + NCCL all_reduce + central update (the reference's sequence)
and the fused kernel's fraction of its roofline = max(HBM bytes / measured copy bandwidth, NVLink bytes / link rate),
printed for TWO link rates: the rate a plain copy kernel reaches here when every GPU stores into every peer at once
(measured by this program on the same buffers, ``peer_store_gbs``) and the nominal 900 GB/s per direction of NVLink 5.
Every row carries the SM clocks and throttle reasons sampled (NVML, read-only) while it was measured.
Consecutive calls touch 4*n*(3k+4) bytes; for the small model that fits in L2, so the small-model rows are L2-resident
numbers (as they are inside training); the large model exceeds L2 for every k.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--sizes", default="464154,25557032")
    ap.add_argument("--replicas", default="1,2,4")
    ap.add_argument("--two-shot", default="auto")
    ap.add_argument("--large-chunk", type=int, default=0, help="tuning: floats per chunk of the two-shot exchange (default 32768)")
    ap.add_argument("--max-blocks", type=int, default=0, help="tuning: CTAs of the fused kernel (default: two per SM)")
    ap.add_argument("--nvls", action="store_true", help="also time the NVLink-multicast (multimem) variant of the two-shot exchange")
    a = ap.parse_args()
    import torch.distributed as dist
    from ..ops import lib as L
    from ..ops.kernel_bench import peaks
    from .peer import init_process_group
    from .sync import ALGO_SMA, FusedSynchroniser, ReferenceSynchroniser
    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    init_process_group("nccl")
    lib = L.init_device()
    if a.large_chunk:
        lib.xb_sync_set_large_chunk(a.large_chunk)
    bw, _, how = peaks()
    from ..utils.gpumon import ClockSampler
    from .peer import PeerBuffer
    NOMINAL_LINK = 900.0                      # GB/s per direction per GPU (NVLink 5, 18 links)
    stream = torch.cuda.Stream()

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(a.iters):
            fn()
        e1.record(stream)
        e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / a.iters], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def peer_store_rate(n):
        """GB/s leaving one GPU when every rank copies (G - 1) / G of an n-float vector into its peers' buffers at once
        with a plain 16-byte copy kernel (slice g goes to rank g): the all-to-all pattern of the two-shot exchange."""
        if world == 1:
            return None
        part = (n // world + 3) // 4 * 4
        buf = PeerBuffer(4 * part * world, rank, world)
        src = torch.randn(part * world, device="cuda")
        s = stream.cuda_stream

        import ctypes as C
        peers = [g for g in range(world) if g != rank]
        dsts = (C.c_void_p * len(peers))(*[buf.ptrs[g] + 4 * part * rank for g in peers])
        srcs = (C.c_void_p * len(peers))(*[src.data_ptr() + 4 * part * g for g in peers])
        blocks = max(16, 592 // len(peers))            # ~4 CTAs per SM in total, all destinations in flight at once

        def push():
            L.check(lib.xb_peer_copy_all(dsts, srcs, len(peers), part, blocks, s), "peer copy")
        with torch.cuda.stream(stream):
            us = timed(push)
        torch.cuda.synchronize()
        dist.barrier()
        buf.close()
        return 4.0 * part * (world - 1) / (us * 1e3)

    for n in [int(v) for v in a.sizes.split(",")]:
        n = (n + 3) // 4 * 4
        peer_gbs = peer_store_rate(n)
        for k in [int(v) for v in a.replicas.split(",")]:
            g = torch.Generator(device="cuda").manual_seed(1 + rank)
            ws = [torch.randn(n, device="cuda", generator=g) * 0.01 for _ in range(k)]
            ps = [torch.randn(n, device="cuda", generator=g) * 0.01 for _ in range(k)]
            two = None if a.two_shot == "auto" else a.two_shot == "1"
            fs = FusedSynchroniser(n, rank, world, two_shot=two, max_blocks=a.max_blocks)
            fn = FusedSynchroniser(n, rank, world, two_shot=two, nvls=True, max_blocks=a.max_blocks) if (a.nvls and world > 1 and fs.two_shot) else None
            # the central model lives where the synchroniser wants it (peer-visible memory when chunk owners store into it)
            z = fs.central_storage()
            z = z.zero_() if z is not None else torch.zeros(n, device="cuda")
            zl = torch.zeros(n, device="cuda")
            rs = ReferenceSynchroniser(n, rank, world)
            s = stream.cuda_stream
            sampler = ClockSampler(local)
            sampler.start()
            with torch.cuda.stream(stream):
                t_f = timed(lambda: fs.synchronise(s, ALGO_SMA, ws, ps, z, zl, alpha=0.1, mu=0.9))
                torch.cuda.synchronize()
                fs.check()
                clocks = sampler.stop()
                tl = fs.timeline()
                t_n, tln = None, None
                if fn is not None and fn.nvls:
                    zn = fn.central_storage().zero_()
                    t_n = timed(lambda: fn.synchronise(s, ALGO_SMA, ws, ps, zn, zl, alpha=0.1, mu=0.9))
                    torch.cuda.synchronize()
                    fn.check()
                    tln = fn.timeline()
                t_r = timed(lambda: rs.synchronise(s, ALGO_SMA, ws, ps, z, zl, alpha=0.1, mu=0.9))
            # bytes this implementation moves through one GPU's HBM: replicas 3k, central model and its momentum 4, plus the
            # exchange (one-shot: G partials written and read; two-shot with owner-apply: partials once in, once out, 3/G)
            extra = 0.0 if world == 1 else (2.0 * world if not fs.two_shot else (3.0 / world if fs.owner_apply else 4.0))
            hbm = 4.0 * n * (3 * k + 4 + extra)
            link = 4.0 * n * ((world - 1) if not fs.two_shot else 2.0 * (world - 1) / world) if world > 1 else 0.0
            roof = lambda gbs: max(hbm / (bw * 1e3), link / (gbs * 1e3)) if gbs else hbm / (bw * 1e3)     # microseconds
            t_meas, t_nom = roof(peer_gbs), roof(NOMINAL_LINK if world > 1 else None)
            if rank == 0:
                print(json.dumps({"op": "sma_sync", "n": n, "replicas": k, "gpus": world, "two_shot": fs.two_shot, "owner_apply": bool(fs.owner_apply and world > 1),
                                  "fused_us": round(t_f, 2), "reference_us": round(t_r, 2), "speedup": round(t_r / t_f, 2),
                                  "release_us": round(tl["release_us"], 2), "chunk_floats": int(lib.xb_sync_chunk(n)), "max_blocks": a.max_blocks,
                                  "nvls_us": round(t_n, 2) if t_n else None, "nvls_release_us": round(tln["release_us"], 2) if tln else None,
                                  "nvls_fraction_of_roofline_900": round(t_nom / t_n, 3) if t_n else None,
                                  "peer_store_gbs": round(peer_gbs, 1) if peer_gbs else None,
                                  "roofline_us_measured_link": round(t_meas, 2), "fraction_of_roofline_measured_link": round(t_meas / t_f, 3),
                                  "roofline_us_900": round(t_nom, 2), "fraction_of_roofline_900": round(t_nom / t_f, 3),
                                  "hbm_bytes": hbm, "nvlink_bytes_per_gpu": link, "hbm_peak": how, "clocks": clocks}), flush=True)
            fs.close()
            if fn is not None:
                fn.close()
            del ws, ps, z, zl
            torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
