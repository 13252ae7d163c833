#!/usr/bin/env bash
# Run every test tier this machine can run, in one command (reference: scripts/run_tests.sh:18-28, which runs the unit
# tests, the example, and -- with 8 GPUs -- the multi-process suites through scripts/local_mc.sh:46-82):
#
#   tier 1  CPU suite: pure-Python units, compiler equivalence, multi-process runs over gloo on 127.0.0.1
#   tier 2  single-GPU suite (-m gpu): every native kernel against fp32 PyTorch math, bounded-wait time-outs
#   tier 3  multi-GPU suite (needs >= 2 GPUs; the 4-GPU cases skip themselves below 4)
#   tier 4  the basic example, pipelined against sequential
#
# Usage: tests/run_tests.sh [--cpu-only] [--gpu-only]     (exit code: non-zero if any tier failed)
set -u
cd "$(dirname "$0")/.."
PY=${PYTHON:-python}
export MASTER_ADDR=127.0.0.1
cpu=1; gpu=1
for a in "$@"; do
  case "$a" in
    --cpu-only) gpu=0 ;;
    --gpu-only) cpu=0 ;;
    *) echo "unknown argument $a" >&2; exit 2 ;;
  esac
done
n_gpus=$($PY - <<'PYEOF'
import torch
print(torch.cuda.device_count() if torch.cuda.is_available() else 0)
PYEOF
)
fail=0
run() { echo "=== $*"; "$@" || fail=1; }

$PY -m jaxpp_b200.csrc.build > /dev/null || { echo "native library failed to build" >&2; exit 1; }
if [ "$cpu" = 1 ]; then
  run $PY -m pytest tests -q -m "not gpu"
  run $PY examples/basic.py --steps 3
fi
if [ "$gpu" = 1 ]; then
  if [ "$n_gpus" -ge 1 ]; then
    run $PY -m pytest tests -q -m "gpu and not multigpu"
  else
    echo "=== no GPU: skipping the -m gpu tiers"
  fi
  if [ "$n_gpus" -ge 2 ]; then
    NCCL_NVLS_ENABLE=0 run $PY -m pytest tests/test_multigpu.py -q -m gpu
  fi
fi
exit $fail
