// Same file name as the reference header (src/backend/cuda/include/full_attention_cuda.hpp); forwards to the b200attn-backed classes.
#pragma once
#include "../qwen_cuda_compat.hpp"
