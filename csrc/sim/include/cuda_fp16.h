/** 16-bit float types of the host simulation build: storage plus the conversions the kernels use. */
#pragma once
#include "cuda_runtime.h"
#include "../../core/types.hpp"

struct __half { uint16_t bits; };
struct __nv_bfloat16 { uint16_t bits; };
inline float __half2float(__half h) { return dccl::half_to_float(h.bits); }
inline __half __float2half_rn(float f) { return __half{dccl::float_to_half(f)}; }
inline float __bfloat162float(__nv_bfloat16 h) { return dccl::bf16_to_float(h.bits); }
inline __nv_bfloat16 __float2bfloat16_rn(float f) { return __nv_bfloat16{dccl::float_to_bf16(f)}; }
