// Scalar functors for the element-wise tile operations (reference: include/cell/compute/math_functor.hpp:7-176).
#pragma once

#include <cuda_fp16.h>

#include "config.hpp"

namespace tiledcuda::cell::compute {

template <typename T>
struct Add {
    DEVICE T operator()(T a, T b) const { return a + b; }
    DEVICE void operator()(const T& a, const T& b, T& out) const { out = a + b; }
};
template <typename T>
struct Sub {
    DEVICE T operator()(T a, T b) const { return a - b; }
    DEVICE void operator()(const T& a, const T& b, T& out) const { out = a - b; }
};
template <typename T>
struct Mul {
    DEVICE T operator()(T a, T b) const { return a * b; }
    DEVICE void operator()(const T& a, const T& b, T& out) const { out = a * b; }
};
template <typename T>
struct Div {
    DEVICE T operator()(T a, T b) const { return a / b; }
    DEVICE void operator()(const T& a, const T& b, T& out) const { out = a / b; }
};
template <typename T>
struct Max {
    DEVICE T operator()(T a, T b) const { return a > b ? a : b; }
    DEVICE void operator()(const T& a, const T& b, T& out) const { out = a > b ? a : b; }
};
template <typename T>
struct Min {
    DEVICE T operator()(T a, T b) const { return a < b ? a : b; }
    DEVICE void operator()(const T& a, const T& b, T& out) const { out = a < b ? a : b; }
};

template <typename T>
struct Exp {
    DEVICE T operator()(T a) const { return static_cast<T>(__expf(static_cast<float>(a))); }
    DEVICE void operator()(const T& a, T& out) const { out = (*this)(a); }
};
template <>
struct Exp<__half> {
    DEVICE __half operator()(__half a) const { return hexp(a); }
    DEVICE void operator()(const __half& a, __half& out) const { out = hexp(a); }
};
template <typename T>
struct Log {
    DEVICE T operator()(T a) const { return static_cast<T>(__logf(static_cast<float>(a))); }
    DEVICE void operator()(const T& a, T& out) const { out = (*this)(a); }
};
template <typename T>
struct Relu {
    DEVICE T operator()(T a) const { return a > T(0) ? a : T(0); }
    DEVICE void operator()(const T& a, T& out) const { out = (*this)(a); }
};

template <typename From, typename To>
struct Convert {
    DEVICE To operator()(From a) const { return static_cast<To>(a); }
    DEVICE void operator()(const From& a, To& out) const { out = static_cast<To>(a); }
};
template <>
struct Convert<float, __half> {
    DEVICE __half operator()(float a) const { return __float2half(a); }
    DEVICE void operator()(const float& a, __half& out) const { out = __float2half(a); }
};
template <>
struct Convert<__half, float> {
    DEVICE float operator()(__half a) const { return __half2float(a); }
    DEVICE void operator()(const __half& a, float& out) const { out = __half2float(a); }
};

}  // namespace tiledcuda::cell::compute
