#!/bin/bash
# Bus-bandwidth sweep of this library against stock NCCL on N GPUs of this machine, one process per GPU.
#   benchmarks/run_sweep.sh 8 [extra dccl_sweep options]     e.g.  --symmetric --out results/sweep.json
# The single-box counterpart of the original's cluster run scripts (reference scripts/run_ompi_cli_4.1.5.sh,
# scripts/azure/run_dccl.sh): same tool on every rank, results collected by rank 0.
set -e
N=${1:-2}; shift || true
ROOT=$(cd "$(dirname "$0")/.." && pwd)
NCCL_LIB=$(python -c "import glob,sys,os; c=glob.glob(os.path.join(sys.prefix,'lib','python*','site-packages','nvidia','nccl','lib','libnccl.so.2')); print(c[0] if c else '')")
export DCCL_NCCL_LIB=${DCCL_NCCL_LIB:-$NCCL_LIB}
exec python -m torch.distributed.run --no-python --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29541} \
     -- "$ROOT/build/dccl_sweep" --gpu auto "$@"
