#!/bin/bash
# The original's evaluation matrix on one box: dccl_cli all_reduce over world sizes and algorithms, the
# stock-NCCL twin as comparator, per-rank timestamp files collected into one tarball per run
# (single-box counterpart of reference scripts/azure/run_dccl.sh and run_ompi.sh: there world sizes 20..2,
# 2^30 floats, 20 warm-up / 200 timed calls, ring and rabenseifner).
#   benchmarks/run_cli_matrix.sh [max_gpus=8] [count=268435456] [out_dir=results/cli_matrix]
# DEVICE=host runs the same matrix on host buffers (no GPU; the NCCL twin is left out).
set -e
MAXN=${1:-8}; COUNT=${2:-268435456}; OUT=${3:-results/cli_matrix}
ROOT=$(cd "$(dirname "$0")/.." && pwd)
NCCL_LIB=$(python -c "import glob,sys,os; c=glob.glob(os.path.join(sys.prefix,'lib','python*','site-packages','nvidia','nccl','lib','libnccl.so.2')); print(c[0] if c else '')")
export DCCL_NCCL_LIB=${DCCL_NCCL_LIB:-$NCCL_LIB}
mkdir -p "$OUT"
OUT=$(cd "$OUT" && pwd)
WARMUP=${WARMUP:-20}; REPEAT=${REPEAT:-200}
GPUARG="-g auto"; RUNS="dccl:ring dccl:rabenseifner dccl:auto nccl:nccl"
if [ "${DEVICE:-gpu}" = host ]; then GPUARG=""; RUNS="dccl:ring dccl:rabenseifner"; fi
for N in 8 4 2; do
    [ "$N" -le "$MAXN" ] || continue
    for RUN in $RUNS; do
        TOOL=${RUN%%:*}_cli; ALGO=${RUN##*:}
        WORK=$(mktemp -d "$OUT/run.XXXXXX")
        ARGS="-a all_reduce $GPUARG -t float32 -o sum -c $COUNT -w $WARMUP -r $REPEAT"
        [ "$TOOL" = dccl_cli ] && ARGS="$ARGS --tt-per-rank --algo $ALGO"   # nccl_cli always writes one file per rank
        (cd "$WORK" && python -m torch.distributed.run --no-python --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 \
            --master-port ${MASTER_PORT:-29561} -- "$ROOT/build/$TOOL" $ARGS > log.txt 2>&1) || echo "run $RUN on $N GPUs failed, see $WORK/log.txt"
        grep -h "avg latency" "$WORK/log.txt" | head -1 | sed "s/^/n=$N $RUN: /"
        tar -C "$WORK" -czf "$OUT/${TOOL}_n${N}_${ALGO}.tar.gz" . && rm -rf "$WORK"
    done
done
