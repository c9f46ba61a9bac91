#pragma once
#include <cuda_fp16.h>  // __half, __half2: named in discarded `if constexpr` branches
