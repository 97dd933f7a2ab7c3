#!/bin/bash
# Relaunch loop for multi-node jobs without a scheduler-side requeue: builds the host list, starts one
# torchrun per node over ssh and, when the job exits (failure, watchdog poison, pre-emption), waits and starts
# it again; every start resumes from the newest complete checkpoint because `load` == `save` in the config.
# (Role of the reference's launch_multinode_slurm.sh:12-27.)
#   HOSTS="node1 node2" GPUS_PER_NODE=8 ./launch_multinode.sh -d configs model.yml data.yml
set -uo pipefail
HOSTS=${HOSTS:?space separated host names}
GPUS_PER_NODE=${GPUS_PER_NODE:-8}
MASTER_PORT=${MASTER_PORT:-29500}
RETRY_SLEEP=${RETRY_SLEEP:-900}
read -r -a HOST_ARR <<< "$HOSTS"
MASTER=${HOST_ARR[0]}
NNODES=${#HOST_ARR[@]}
ARGS_FILE=$(mktemp)
python launch.py train.py "$@" --num_gpus $((NNODES * GPUS_PER_NODE)) --train-args-output "$ARGS_FILE" || exit 1
while true; do
  pids=()
  for i in "${!HOST_ARR[@]}"; do
    ssh "${HOST_ARR[$i]}" "cd $PWD && python -m torch.distributed.run --nnodes=$NNODES --node-rank=$i \
      --nproc-per-node=$GPUS_PER_NODE --master-addr $MASTER --master-port $MASTER_PORT train.py $(cat "$ARGS_FILE")" &
    pids+=($!)
  done
  rc=0
  for p in "${pids[@]}"; do wait "$p" || rc=$?; done
  if [ "$rc" -eq 0 ]; then echo "training finished"; break; fi
  echo "job exited with code $rc; relaunching in ${RETRY_SLEEP}s"
  sleep "$RETRY_SLEEP"
done
