#pragma once
#include "cuda_fp16.h"
