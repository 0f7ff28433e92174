// Same file name as the reference header (src/backend/cuda/include/linear_attention_v2.cuh); forwards to the b200attn-backed classes.
#pragma once
#include "../qwen_cuda_compat.hpp"
