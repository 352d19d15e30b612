// peaks.cu -- arithmetic-peak microbenchmarks for the roofline denominators the driver does not
// measure: TF32 on the 5th-generation tensor cores (tcgen05.mma kind::tf32 issued back to back on
// resident shared-memory operands, no loads) and FP64 on the CUDA cores (DFMA) and on the FP64
// tensor path (mma.sync m8n8k4).  Every SM runs the same loop at once, so the figures include the
// clock the chip settles at under that load.
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/tcontb.h"

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint64_t desc_kmajor_sw128(uint32_t addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// One CTA per SM; thread 32 issues `iters` MMAs of shape 128 x N x 8 into one accumulator.
__global__ void __launch_bounds__(64, 1) tf32_peak_kernel(int iters, int N, int* status)
{
    extern __shared__ uint8_t raw[];
    uint8_t* smem = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    // operands: A 128 rows x 128 B, B 256 rows x 128 B, zero filled (the arithmetic rate does not depend on values)
    for (int i = threadIdx.x; i < (128 + 256) * 32; i += blockDim.x) reinterpret_cast<float*>(smem)[i] = 0.0f;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const int warp = threadIdx.x >> 5;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 32) {
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(N >> 3) << 17) | (8u << 24);
        const uint32_t a = smem_u32(smem), b = a + 128 * 128;
        for (int i = 0; i < iters; ++i) {
            const uint64_t da = desc_kmajor_sw128(a + (i & 3) * 32), db = desc_kmajor_sw128(b + (i & 3) * 32);
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                ::"r"(tmem), "l"(da), "l"(db), "r"(idesc), "r"(i ? 1u : 0u), "r"(0u) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
        // bounded wait for the last MMA
        uint32_t done = 0;
        for (long long spin = 0; spin < (1ll << 28) && !done; ++spin)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(smem_u32(&bar)), "r"(0u) : "memory");
        if (!done) atomicMax(status, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
}

// 8 independent DFMA chains per thread.
__global__ void __launch_bounds__(256) dfma_peak_kernel(int iters, double* sink)
{
    double a[8], x = 1.0 + threadIdx.x * 1e-9, y = 1e-9;
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = j;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = fma(a[j], x, y);
    }
    double s = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += a[j];
    if (s == 123.456) sink[0] = s;
}

// 8 independent m8n8k4 FP64 MMA accumulators per warp.
__global__ void __launch_bounds__(256) dmma_peak_kernel(int iters, double* sink)
{
    double c[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j) c[j][0] = c[j][1] = 0.0;
    const double a = 1.0 + threadIdx.x * 1e-9, b = 1e-9;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                         : "+d"(c[j][0]), "+d"(c[j][1]) : "d"(a), "d"(b));
    }
    double s = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) s += c[j][0] + c[j][1];
    if (s == 123.456) sink[0] = s;
}

thread_local std::string g_err;

}  // namespace

extern "C" const char* tcontb_peak_last_error(void) { return g_err.c_str(); }

// which: 0 = TF32 tcgen05 (128x256x8 MMAs), 1 = FP64 DFMA, 2 = FP64 mma.sync m8n8k4. Result in TFLOP/s.
extern "C" tcontb_status tcontb_measure_peak(int which, double* tflops)
{
    if (!tflops || which < 0 || which > 2) {
        g_err = "bad arguments";
        return TCONTB_INVALID_ARGUMENT;
    }
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    void* scratch = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&scratch, 256);
    if (e == cudaSuccess) e = cudaMemset(scratch, 0, 256);
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    double flops = 0;
    float ms = 0;
    for (int rep = 0; rep < 3 && e == cudaSuccess; ++rep) {  // last repetition is the one reported
        e = cudaEventRecord(e0);
        if (which == 0) {
            const int iters = 40000, N = 256, smem = (128 + 256) * 128 + 1024;
            e = cudaFuncSetAttribute(tf32_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e == cudaSuccess) tf32_peak_kernel<<<sms, 64, smem>>>(iters, N, static_cast<int*>(scratch));
            flops = 2.0 * 128 * N * 8 * double(iters) * sms;
        } else if (which == 1) {
            const int iters = 20000;
            dfma_peak_kernel<<<sms * 8, 256>>>(iters, static_cast<double*>(scratch));
            flops = 2.0 * 8 * double(iters) * 256 * sms * 8;
        } else {
            const int iters = 20000;
            dmma_peak_kernel<<<sms * 8, 256>>>(iters, static_cast<double*>(scratch));
            flops = 2.0 * 8 * 8 * 4 * 8 * double(iters) * 8 * sms * 8;  // 2*m*n*k per MMA, 8 MMAs per warp iteration, 8 warps per block
        }
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaEventRecord(e1);
        if (e == cudaSuccess) e = cudaEventSynchronize(e1);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    }
    int st = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&st, scratch, sizeof(int), cudaMemcpyDeviceToHost);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (scratch) cudaFree(scratch);
    if (e != cudaSuccess) {
        g_err = std::string("CUDA error: ") + cudaGetErrorString(e);
        return TCONTB_RUNTIME_ERROR;
    }
    if (which == 0 && st != 0) {
        g_err = "the MMA loop did not complete within its wait limit";
        return TCONTB_RUNTIME_ERROR;
    }
    *tflops = flops / (ms * 1e-3) / 1e12;
    return TCONTB_OK;
}
