#!/bin/bash
# Compares the optional variants with the table's choice and with stock NCCL on N GPUs, one JSON file per run:
#   benchmarks/run_variants.sh 8 [out_dir=results/variants]
# Runs: mid-size all-reduce (table / twoshot_ll / NCCL, ordinary and symmetric buffers), large all-reduce and
# reduce-scatter on peer-addressable buffers (table / zero-copy two-shot, symmetric and registered), broadcast and
# reduce with and without the pipelined switch form, graph replay latency, the tensor-parallel training step over NCCL /
# this library / this library reducing in place. The sweep files feed make_tune_table.py.
set -u
N=${1:-8}; OUT=${2:-results/variants}
ROOT=$(cd "$(dirname "$0")/.." && pwd)
mkdir -p "$OUT"; OUT=$(cd "$OUT" && pwd)
SWEEP="$ROOT/benchmarks/run_sweep.sh"
run() { local name=$1; shift; echo "== $name: $*"; "$@" > "$OUT/$name.log" 2>&1 || echo "   failed, see $OUT/$name.log"; grep -E "^(all_reduce|reduce_scatter|all_gather) " "$OUT/$name.log" | tail -n 12; }

# 64 KB - 4 MB all-reduce: the packet two-shot form against the table and NCCL
MID="--min 64K --max 4M --factor 2 --colls all_reduce"
run mid_table            "$SWEEP" "$N" $MID --impls dccl,nccl --out "$OUT/mid_table.json"
run mid_twoshot_ll       "$SWEEP" "$N" $MID --impls dccl --algo twoshot_ll --out "$OUT/mid_twoshot_ll.json"
run mid_table_sym        "$SWEEP" "$N" $MID --impls dccl --symmetric --out "$OUT/mid_table_sym.json"

# 1 MB - 1 GB on buffers every rank can address: zero-copy two-shot against the table (switch) choice
BIG="--min 1M --factor 4"
for C in all_reduce reduce_scatter; do
    run big_${C}_sym_table     "$SWEEP" "$N" $BIG --colls $C --impls dccl,nccl --symmetric --out "$OUT/big_${C}_sym_table.json"
    run big_${C}_sym_direct    "$SWEEP" "$N" $BIG --colls $C --impls dccl --symmetric --algo twoshot --out "$OUT/big_${C}_sym_direct.json"
    run big_${C}_reg_direct    "$SWEEP" "$N" $BIG --colls $C --impls dccl --register --algo twoshot --out "$OUT/big_${C}_reg_direct.json"
done

# broadcast / reduce / send-recv rows of bench.py, staged and pipelined switch forms
TORCHRUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29581}"
run extra_staged    $TORCHRUN "$ROOT/bench.py" --gpus "$N" --steps 5 --warmup 3 --sweep-extra --out "$OUT/extra_staged.json"
DCCL_NVLS_ROOTED_PIPE=1 run extra_pipelined $TORCHRUN "$ROOT/bench.py" --gpus "$N" --steps 5 --warmup 3 --sweep-extra --out "$OUT/extra_pipelined.json"
DCCL_REDUCE_ALGORITHM=twoshot_ll run extra_reduce_ll $TORCHRUN "$ROOT/bench.py" --gpus "$N" --steps 5 --warmup 3 --sweep-extra --out "$OUT/extra_reduce_ll.json"

# eager launches against CUDA-graph replay
run graph_latency $TORCHRUN "$ROOT/benchmarks/graph_latency.py" --out "$OUT/graph_latency.json"

# tensor-parallel training step: stock NCCL, this library on ordinary buffers, this library reducing in place
for ARM in "nccl" "dccl" "dccl --in-place-reduce" "nccl --sequence-parallel" "dccl --sequence-parallel"; do
    NAME=train_tp_$(echo $ARM | tr -d ' -' )
    run $NAME $TORCHRUN "$ROOT/benchmarks/train_tp.py" --backend $ARM --steps 8 --warmup 3
    grep -h '"metric"' "$OUT/$NAME.log" | tail -n 1
done
ls -la "$OUT"
