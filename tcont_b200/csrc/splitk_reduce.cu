// splitk_reduce.cu -- second pass of a split-K contraction: sums the partial tensors the contraction
// kernel wrote (one per range of the contracted extent, each laid out like C) into C, in ascending
// order of the split so that the result does not depend on scheduling.  Pure streaming: reads
// splits * |C| elements, writes |C|.
//
// Also here: the residual pass of the error-compensated Float32 mode (TCONT_TF32X3=1), which gives
// the tcgen05 kernel the part of each operand that narrowing to TF32 drops, so that three products
// (hi*hi + hi*lo + lo*hi), summed by the kernel above, carry fp32-level accuracy.
//
// The reference has no counterpart: its generated kernels give one CTA the whole contracted extent
// (backends/cogent/plan/generators/kernels/kernel_body.py) and its TTGT route leaves the split to
// cuBLAS (backends/ttgt_cutt/src/ttgt_cutt.cpp:764-809).
#include <algorithm>

#include "kernels.hpp"

namespace tcontb {
namespace {

template <typename T, typename V, int W>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const T* __restrict__ partial, T* __restrict__ C, long long elements,
                                                           int splits, long long stride, bool vector_ok, bool scaled, T alpha,
                                                           T beta)
{
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (vector_ok) {
        const long long nv = elements / W;
        for (; i < nv; i += step) {
            V acc = __ldcs(reinterpret_cast<const V*>(partial) + i);
            for (int s = 1; s < splits; ++s) {
                const V v = __ldcs(reinterpret_cast<const V*>(partial + static_cast<long long>(s) * stride) + i);
                acc.x += v.x;
                acc.y += v.y;
                if constexpr (W == 4) {
                    acc.z += v.z;
                    acc.w += v.w;
                }
            }
            if (scaled) {  // C = alpha * sum + beta * C; C is read only when beta is not zero
                V old{};
                if (beta != T(0)) old = reinterpret_cast<const V*>(C)[i];
                acc.x = alpha * acc.x + beta * old.x;
                acc.y = alpha * acc.y + beta * old.y;
                if constexpr (W == 4) {
                    acc.z = alpha * acc.z + beta * old.z;
                    acc.w = alpha * acc.w + beta * old.w;
                }
            }
            __stcs(reinterpret_cast<V*>(C) + i, acc);
        }
        i = nv * W + (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x);
    }
    for (; i < elements; i += step) {
        T acc = partial[i];
        for (int s = 1; s < splits; ++s) acc += partial[static_cast<long long>(s) * stride + i];
        if (scaled) acc = alpha * acc + (beta != T(0) ? beta * C[i] : T(0));
        C[i] = acc;
    }
}

// lo[i] = x[i] - (x[i] with the 13 low mantissa bits cleared): what the tensor core drops when it
// narrows an fp32 operand to TF32 (it truncates).  The difference is exact in fp32.
__global__ void __launch_bounds__(256) tf32_residual_kernel(const float* __restrict__ x, float* __restrict__ lo, long long elements,
                                                           bool vector_ok)
{
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    auto residual = [](float v) { return v - __uint_as_float(__float_as_uint(v) & 0xffffe000u); };
    if (vector_ok) {
        const long long nv = elements / 4;
        for (; i < nv; i += step) {
            float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
            v.x = residual(v.x);
            v.y = residual(v.y);
            v.z = residual(v.z);
            v.w = residual(v.w);
            reinterpret_cast<float4*>(lo)[i] = v;
        }
        i = nv * 4 + (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x);
    }
    for (; i < elements; i += step) lo[i] = residual(x[i]);
}

}  // namespace

cudaError_t launch_tf32_residual(const float* x, float* lo, long long elements, cudaStream_t stream)
{
    if (elements <= 0) return cudaErrorInvalidValue;
    const bool vector_ok = reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(lo) % 16 == 0;
    const long long work = vector_ok ? (elements + 3) / 4 : elements;
    const unsigned grid = static_cast<unsigned>(std::min<long long>((work + 255) / 256, 148ll * 8));
    tf32_residual_kernel<<<grid, 256, 0, stream>>>(x, lo, elements, vector_ok);
    return cudaGetLastError();
}

cudaError_t launch_splitk_reduce(const void* partial, void* C, long long elements, int splits, long long stride, int elt_bytes,
                                 cudaStream_t stream, double alpha, double beta)
{
    const bool scaled = alpha != 1.0 || beta != 0.0;
    if (elements <= 0 || splits < 1) return cudaErrorInvalidValue;
    const int w = elt_bytes == 8 ? 2 : 4;
    const bool vector_ok = reinterpret_cast<uintptr_t>(partial) % 16 == 0 && reinterpret_cast<uintptr_t>(C) % 16 == 0 &&
                           (stride * elt_bytes) % 16 == 0;
    const long long work = vector_ok ? (elements + w - 1) / w : elements;
    const unsigned grid = static_cast<unsigned>(std::min<long long>((work + 255) / 256, 148ll * 8));
    if (elt_bytes == 8)
        splitk_reduce_kernel<double, double2, 2><<<grid, 256, 0, stream>>>(static_cast<const double*>(partial), static_cast<double*>(C),
                                                                            elements, splits, stride, vector_ok, scaled, alpha, beta);
    else
        splitk_reduce_kernel<float, float4, 4><<<grid, 256, 0, stream>>>(static_cast<const float*>(partial), static_cast<float*>(C),
                                                                          elements, splits, stride, vector_ok, scaled,
                                                                          static_cast<float>(alpha), static_cast<float>(beta));
    return cudaGetLastError();
}

}  // namespace tcontb
