#!/usr/bin/env python
"""Host-side micro-benchmarks, the counterpart of the reference's src/test/java/.../microbenchmarks
(queues, slots, learningrate, random): throughput of the bounded MPMC queue and of the replica pool, the policy task
queue, learning-rate schedule evaluation and the model initialisers.  No GPU needed.

    python examples/microbenchmarks.py
"""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from crossbow_b200 import Model, Shape, SolverConf
    from crossbow_b200.models import build
    from crossbow_b200.runtime import TaskQueue, load
    lib = load()
    out = {}
    for p, c in ((1, 1), (2, 2), (4, 4)):
        out[f"mpmc_queue_{p}p{c}c_Mitems_per_s"] = round(lib.rt_bench_mpmc(p, c, 2_000_000), 2)
    for slots in (1, 4, 16):
        out[f"replica_pool_{slots}_slots_Mops_per_s"] = round(lib.rt_bench_theta(slots, 2_000_000), 2)
    q = TaskQueue("HLS")
    n = 20000
    for t in range(n):
        q.push(t, graph=t % 2)
    t0 = time.perf_counter()
    matrix = [[10, 40], [100, 20]]
    got = 0
    while len(q):
        for p in (1, 0):
            got += q.poll(p, matrix) >= 0
    out["hls_task_queue_Kpolls_per_s"] = round(got / (time.perf_counter() - t0) / 1e3, 1)
    for policy in ("FIXED", "INV", "STEP", "MULTISTEP", "EXP"):
        s = SolverConf().setLearningRateDecayPolicy(policy).setBaseLearningRate(0.1).setGamma(0.1).setPower(0.75).setStepSize(1000)
        if policy == "MULTISTEP":
            s.setStepValues(1000, 2000, 3000)
        t0 = time.perf_counter()
        for t in range(20000):
            s.learning_rate(t)
        out[f"learning_rate_{policy.lower()}_Kevals_per_s"] = round(20000 / (time.perf_counter() - t0) / 1e3, 1)
    spec = build("resnet32", solver_conf=SolverConf())
    m = Model()
    spec.train.init(Shape([64] + spec.input_shape), Shape([64]), m)
    m.finalise()
    t0 = time.perf_counter()
    m.initial_values(1)
    out["initialise_resnet32_Mparams_per_s"] = round(m.elements / (time.perf_counter() - t0) / 1e6, 2)
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()
