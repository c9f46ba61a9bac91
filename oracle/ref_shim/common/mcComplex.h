// Complex types named by the mcSparse headers; the real-typed CSR kernels never touch them.
#pragma once
#include <cuComplex.h>
#include <complex>
typedef cuFloatComplex mcFloatComplex;
typedef cuDoubleComplex mcDoubleComplex;
typedef cuFloatComplex mcComplex;
namespace std {
__host__ __device__ inline mcFloatComplex conj(mcFloatComplex a) { return cuConjf(a); }
__host__ __device__ inline mcDoubleComplex conj(mcDoubleComplex a) { return cuConj(a); }
}  // namespace std
