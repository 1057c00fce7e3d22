#!/bin/bash
# Data-parallel training benchmark on N GPUs of this machine, one process per GPU:
#   benchmarks/run_ddp.sh 8                 all three backends (dccl, dccl_ddp, nccl), one after the other
#   benchmarks/run_ddp.sh 8 dccl --steps 20 one backend, extra options go to train_ddp.py
# Prints one JSON line per run (tokens/s, ms/step, exposed communication time).
set -e
N=${1:-1}; shift || true
BACKENDS="dccl dccl_ddp nccl"
case "$1" in dccl|dccl_ddp|nccl) BACKENDS=$1; shift;; esac
ROOT=$(cd "$(dirname "$0")/.." && pwd)
for B in $BACKENDS; do
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29551} \
        "$ROOT/benchmarks/train_ddp.py" --backend "$B" "$@"
done
