#!/bin/bash
# End-to-end regression: (1) 1-GPU run, (2) N-GPU run of the regression config, (3) reload of run (1)'s checkpoint
# for a few more iterations.  Loss curves land in regression_logs/ for comparison against a known-good run
# (role of the reference's run_regression_test.sh / slurm.regression.sh).
#   ./run_regression_test.sh [NGPUS=4] [ITERS=200]
set -euo pipefail
NGPUS=${1:-4}
ITERS=${2:-200}
OUT=regression_logs
mkdir -p "$OUT"
CFG=configs/test/regression_base.yml
python launch.py train.py "$CFG" --num_gpus 1 2>&1 | tee "$OUT/one_gpu.log"
python launch.py train.py "$CFG" --num_gpus "$NGPUS" 2>&1 | tee "$OUT/${NGPUS}_gpu.log"
python launch.py train.py configs/test/regression_reload.yml --num_gpus 1 2>&1 | tee "$OUT/reload.log"
grep -h "lm_loss" "$OUT"/*.log | tail -n 5
