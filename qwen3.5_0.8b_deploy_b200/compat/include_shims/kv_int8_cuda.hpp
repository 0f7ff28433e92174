// Same file name as the reference header (src/backend/cuda/include/kv_int8_cuda.hpp); forwards to the b200attn-backed declarations.
#pragma once
#include "../qwen_cuda_compat.hpp"
