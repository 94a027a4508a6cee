// TEST INFRASTRUCTURE ONLY.
// Stand-in for <torch/extension.h> that lets the reference project's CUDA kernel *source text*
// (the two __global__ templates at the top of models/kernels/wf_cuda/wf_cuda.cu) be compiled by
// g++ and executed on the CPU, one emulated thread at a time.  It provides only what those
// kernel bodies touch: the CUDA index variables, the __global__ marker, and an accessor type
// with the indexing / size() surface of torch::PackedTensorAccessor64.
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <c10/util/BFloat16.h>
#include <c10/util/BFloat16-math.h>

#define __global__

struct ShimDim3 { int x = 0, y = 0, z = 0; };
static thread_local ShimDim3 threadIdx, blockIdx, blockDim;

using std::exp;

namespace torch {

template <typename T>
struct RestrictPtrTraits { typedef T* PtrType; };

template <typename T, size_t N>
struct ShimAccessor {
    T* data; const int64_t* sizes; const int64_t* strides;
    ShimAccessor<T, N - 1> operator[](int64_t i) const { return {data + i * strides[0], sizes + 1, strides + 1}; }
};
template <typename T>
struct ShimAccessor<T, 1> {
    T* data; const int64_t* sizes; const int64_t* strides;
    T& operator[](int64_t i) const { return data[i * strides[0]]; }
};

template <typename T, size_t N, template <typename> class Traits>
struct PackedTensorAccessor64 {
    T* data; int64_t sizes_[N]; int64_t strides_[N];
    int64_t size(int k) const { return sizes_[k]; }
    ShimAccessor<T, N - 1> operator[](int64_t i) const { return {data + i * strides_[0], sizes_ + 1, strides_ + 1}; }
};

}  // namespace torch
