// Same file name as the reference header (src/backend/cuda/include/flash_attention.cuh); forwards to the b200attn-backed declarations.
#pragma once
#include "../qwen_cuda_compat.hpp"
