#!/bin/bash
# Builds the ORIGINAL library's only CUDA kernel, unmodified, into baseline/_ref/libdccl_reference_reduce.so:
# src/core/reduce.cu of the reference tree (dccl::do_device_reduce / reduce_kernel<T>), compiled for sm_100a against
# the reference's own headers plus a generated dccl/config.h (what its CMake writes from config.h.in when CUDA is
# found). The rest of the original needs Derecho, libfabric and spdlog and cannot be built offline; this file needs
# none of them because the source hides them behind NVCC_VISIBLE.
#   baseline/build_reference_kernel.sh <path to the reference tree>      (or DCCL_REFERENCE_DIR=<path>)
# benchmarks/local_reduce_bench.py times it against this library's dccl_local_reduce on the same buffers.
set -e
REF=${1:-$DCCL_REFERENCE_DIR}
if [ -z "$REF" ] || [ ! -f "$REF/src/core/reduce.cu" ]; then echo "usage: $0 <path to the reference tree>" >&2; exit 2; fi
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
mkdir -p "$OUT/gen/dccl"
cat > "$OUT/gen/dccl/config.h" <<CFG
#define ENABLE_EVALUATION
#define CACHELINE_SIZE 64
#define CUDA_FOUND
#define CUDA_L1_CACHELINE_SIZE 128
#define CUDA_L2_CACHELINE_SIZE 32
CFG
NVCC=${NVCC:-/usr/local/cuda/bin/nvcc}
"$NVCC" -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC -shared \
    -I"$OUT/gen" -I"$REF/include" -I"$REF/src/core" "$REF/src/core/reduce.cu" -o "$OUT/libdccl_reference_reduce.so" -lcuda
echo "built $OUT/libdccl_reference_reduce.so"
