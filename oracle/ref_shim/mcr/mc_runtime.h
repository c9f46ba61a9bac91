// Stand-in for the MetaX runtime header the mcSparse kernels include: the CUDA runtime
// under the names those kernels use. Only what the two CSR kernels need.
#pragma once
#include <cuda_runtime.h>
typedef cudaStream_t mcStream_t;
