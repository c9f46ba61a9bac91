// Value types of the kernels and the few operations the kernels need on them, so that one kernel
// source serves float, double and the two complex types (MACA_C_32F / MACA_C_64F: interleaved
// real and imaginary parts, as in the reference's mcspComplexFloat / mcspComplexDouble,
// mcsparse/src/include/mcsp_internal_types.h).
#ifndef MCSPARSE_B200_VALUE_TYPES_H_
#define MCSPARSE_B200_VALUE_TYPES_H_

#include <cuda_runtime.h>

#ifdef __CUDACC__
#define MCSP_HD __host__ __device__ __forceinline__
#define MCSP_D __device__ __forceinline__
#else
#define MCSP_HD inline
#endif

namespace mcsp_b200 {

template <typename F>
struct alignas(2 * sizeof(F)) Complex {
    F re, im;
    Complex() = default;
    MCSP_HD constexpr Complex(F r, F i = F(0)) : re(r), im(i) {}
};
using cfloat = Complex<float>;
using cdouble = Complex<double>;

template <typename F>
MCSP_HD Complex<F> operator+(Complex<F> a, Complex<F> b) { return Complex<F>(a.re + b.re, a.im + b.im); }
template <typename F>
MCSP_HD Complex<F>& operator+=(Complex<F>& a, Complex<F> b) {
    a.re += b.re;
    a.im += b.im;
    return a;
}
template <typename F>
MCSP_HD Complex<F> operator*(Complex<F> a, Complex<F> b) {
    return Complex<F>(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re);
}
template <typename F>
MCSP_HD Complex<F>& operator*=(Complex<F>& a, Complex<F> b) {
    a = a * b;
    return a;
}
template <typename F>
MCSP_HD bool operator!=(Complex<F> a, Complex<F> b) { return a.re != b.re || a.im != b.im; }

// conj() for every value type (identity on the real ones).
MCSP_HD float conj_value(float v) { return v; }
MCSP_HD double conj_value(double v) { return v; }
template <typename F>
MCSP_HD Complex<F> conj_value(Complex<F> v) { return Complex<F>(v.re, -v.im); }

#ifdef __CUDACC__
// Explicit fused multiply-add, a * b + c: the same rounding in every instantiation of the kernels
// (left to the compiler, contraction choices differed between template variants by one ulp).
MCSP_D float mad(float a, float b, float c) { return fmaf(a, b, c); }
MCSP_D double mad(double a, double b, double c) { return fma(a, b, c); }
MCSP_D cfloat mad(cfloat a, cfloat b, cfloat c) {
    return cfloat(fmaf(a.re, b.re, fmaf(-a.im, b.im, c.re)), fmaf(a.re, b.im, fmaf(a.im, b.re, c.im)));
}
MCSP_D cdouble mad(cdouble a, cdouble b, cdouble c) {
    return cdouble(fma(a.re, b.re, fma(-a.im, b.im, c.re)), fma(a.re, b.im, fma(a.im, b.re, c.im)));
}

// Read-only and streaming loads.
MCSP_D float ldg(const float* p) { return __ldg(p); }
MCSP_D double ldg(const double* p) { return __ldg(p); }
MCSP_D cfloat ldg(const cfloat* p) {
    const float2 v = __ldg(reinterpret_cast<const float2*>(p));
    return cfloat(v.x, v.y);
}
MCSP_D cdouble ldg(const cdouble* p) {
    const double2 v = __ldg(reinterpret_cast<const double2*>(p));
    return cdouble(v.x, v.y);
}
MCSP_D float ldcs(const float* p) { return __ldcs(p); }
MCSP_D double ldcs(const double* p) { return __ldcs(p); }
MCSP_D cfloat ldcs(const cfloat* p) {
    const float2 v = __ldcs(reinterpret_cast<const float2*>(p));
    return cfloat(v.x, v.y);
}
MCSP_D cdouble ldcs(const cdouble* p) {
    const double2 v = __ldcs(reinterpret_cast<const double2*>(p));
    return cdouble(v.x, v.y);
}

// Warp shuffles.
MCSP_D float shfl_xor(float v, int d, int w = 32) { return __shfl_xor_sync(0xffffffffu, v, d, w); }
MCSP_D double shfl_xor(double v, int d, int w = 32) { return __shfl_xor_sync(0xffffffffu, v, d, w); }
template <typename F>
MCSP_D Complex<F> shfl_xor(Complex<F> v, int d, int w = 32) {
    return Complex<F>(__shfl_xor_sync(0xffffffffu, v.re, d, w), __shfl_xor_sync(0xffffffffu, v.im, d, w));
}
MCSP_D float shfl_up(float v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
MCSP_D double shfl_up(double v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
template <typename F>
MCSP_D Complex<F> shfl_up(Complex<F> v, int d) {
    return Complex<F>(__shfl_up_sync(0xffffffffu, v.re, d), __shfl_up_sync(0xffffffffu, v.im, d));
}
MCSP_D float shfl_idx(unsigned mask, float v, int src, int w) { return __shfl_sync(mask, v, src, w); }
MCSP_D double shfl_idx(unsigned mask, double v, int src, int w) { return __shfl_sync(mask, v, src, w); }
template <typename F>
MCSP_D Complex<F> shfl_idx(unsigned mask, Complex<F> v, int src, int w) {
    return Complex<F>(__shfl_sync(mask, v.re, src, w), __shfl_sync(mask, v.im, src, w));
}
#endif  // __CUDACC__

}  // namespace mcsp_b200

#endif  // MCSPARSE_B200_VALUE_TYPES_H_
