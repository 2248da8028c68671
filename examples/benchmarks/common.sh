#!/bin/bash
# Shared launcher: 1 GPU runs in-process, G > 1 GPUs through torch.distributed.run (one process per GPU).
#
#   GPUS=8 REPLICAS=2 ./resnet-32.sh [more --flag value pairs]
#   MEASURE=true ...    log nvidia-smi samples (200 ms) next to the run and print their statistics afterwards, as the
#                       reference's benchmark scripts do (scripts/benchmarks/resnet-32.sh:48-51,130-140, tools/measurements)
#   PROFILE=ncu ...     run under Nsight Compute with the clocks left alone (--clock-control none); one GPU only.  The
#                       counterpart of the nvprof wrapper of the reference's run script (scripts/run.sh:18,159-161).
#                       NCU_ARGS adds to "--metrics gpu__time_duration.sum -c 400".
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
GPUS="${GPUS:-1}"
MEASURE="${MEASURE:-false}"
PROFILE="${PROFILE:-}"
run_train () {
  local sampler="" log="measurements-$(date +%s).csv" rc=0
  if [ "$MEASURE" = "true" ]; then
    PYTHONPATH="$ROOT" python -m crossbow_b200.utils.gpumon sample "$log" &
    sampler=$!
  fi
  if [ "$GPUS" -gt 1 ]; then
    if [ -n "$PROFILE" ]; then echo "error: PROFILE needs GPUS=1 (a profiler is never wrapped around a multi-rank run)"; return 1; fi
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 "$ROOT/examples/train.py" "$@"; rc=$?
  elif [ "$PROFILE" = "ncu" ]; then
    ncu --clock-control none ${NCU_ARGS:---metrics gpu__time_duration.sum -c 400} python "$ROOT/examples/train.py" "$@"; rc=$?
  else
    python "$ROOT/examples/train.py" "$@"; rc=$?
  fi
  if [ -n "$sampler" ]; then
    kill "$sampler" 2>/dev/null; wait "$sampler" 2>/dev/null
    [ -s "$log" ] && PYTHONPATH="$ROOT" python -m crossbow_b200.utils.gpumon parse "$log"
  fi
  return $rc
}
