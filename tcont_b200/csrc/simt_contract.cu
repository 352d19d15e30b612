// simt_contract.cu -- generic direct contraction on the CUDA cores (FP64 DFMA / FP32 FFMA).
//
// Every contraction the descriptor can express runs here: the GEMM view addresses the tensors
// through six offset tables (address(A,m,k) = offAm[m] + offAk[k], ...), which is exact because
// a column-major address is a sum of per-mode terms.  This is the path for FP64 and for Float32
// shapes the tcgen05 kernel cannot stage with TMA.  It stands where the reference runs its
// generated WMMA kernels (backends/cogent/plan/generators/kernels/kernel_body.py:1253+); like
// them it overwrites C with a zero-initialised accumulator.
#include "kernels.hpp"

namespace tcontb {
namespace {

template <typename T, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) simt_contract_kernel(SimtParams p)
{
    constexpr int TX = BM / TM;  // threads along m
    constexpr int TY = BN / TN;  // threads along n
    constexpr int THREADS = TX * TY;
    constexpr int A_PER_T = BM * BK / THREADS;
    constexpr int B_PER_T = BN * BK / THREADS;
    constexpr int PAD = 1;
    static_assert(THREADS % BM == 0 && THREADS % BN == 0 && THREADS % BK == 0, "load mapping");

    __shared__ T As[2][BK][BM + PAD];
    __shared__ T Bs[2][BK][BN + PAD];

    const T* __restrict__ A = static_cast<const T*>(p.A);
    const T* __restrict__ B = static_cast<const T*>(p.B);
    T* __restrict__ C = static_cast<T*>(p.C);

    const int tid = threadIdx.x;
    const int tx = tid % TX, ty = tid / TX;
    const int64_t tiles_m = (p.M + BM - 1) / BM;
    const int64_t m0 = (blockIdx.x % tiles_m) * BM;
    const int64_t n0 = (blockIdx.x / tiles_m) * BN;

    // Which (row, k) elements of the A and B tiles this thread fetches.  Threads run along the
    // dimension that is contiguous in memory so that a warp reads whole lines.
    int a_ml[A_PER_T], a_kl[A_PER_T], b_nl[B_PER_T], b_kl[B_PER_T];
    int64_t a_off[A_PER_T], b_off[B_PER_T];
#pragma unroll
    for (int i = 0; i < A_PER_T; ++i) {
        const int idx = tid + i * THREADS;
        a_ml[i] = p.a_along_k ? idx / BK : idx % BM;
        a_kl[i] = p.a_along_k ? idx % BK : idx / BM;
        const int64_t m = m0 + a_ml[i];
        a_off[i] = m < p.M ? __ldg(p.offAm + m) : -1;
    }
#pragma unroll
    for (int i = 0; i < B_PER_T; ++i) {
        const int idx = tid + i * THREADS;
        b_nl[i] = p.b_along_k ? idx / BK : idx % BN;
        b_kl[i] = p.b_along_k ? idx % BK : idx / BN;
        const int64_t n = n0 + b_nl[i];
        b_off[i] = n < p.N ? __ldg(p.offBn + n) : -1;
    }

    T ra[A_PER_T], rb[B_PER_T];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int i = 0; i < A_PER_T; ++i) {
            const int64_t k = k0 + a_kl[i];
            ra[i] = (a_off[i] >= 0 && k < p.K) ? __ldg(A + a_off[i] + __ldg(p.offAk + k)) : T(0);
        }
#pragma unroll
        for (int i = 0; i < B_PER_T; ++i) {
            const int64_t k = k0 + b_kl[i];
            rb[i] = (b_off[i] >= 0 && k < p.K) ? __ldg(B + b_off[i] + __ldg(p.offBk + k)) : T(0);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER_T; ++i) As[buf][a_kl[i]][a_ml[i]] = ra[i];
#pragma unroll
        for (int i = 0; i < B_PER_T; ++i) Bs[buf][b_kl[i]][b_nl[i]] = rb[i];
    };

    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = T(0);

    fetch(0);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
        const bool more = k0 + BK < p.K;
        if (more) fetch(k0 + BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            T a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[buf][kk][tx + TX * i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[buf][kk][ty + TY * j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        if (more) {
            stash(buf ^ 1);
            __syncthreads();
            buf ^= 1;
        }
    }

    // Overwrite C.  Consecutive threads hold consecutive m, and the planner makes C's stride-1
    // mode the fastest digit of m, so each half-warp writes one contiguous run.
#pragma unroll
    for (int j = 0; j < TN; ++j) {
        const int64_t n = n0 + ty + TY * j;
        if (n >= p.N) continue;
        const int64_t cn = __ldg(p.offCn + n);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const int64_t m = m0 + tx + TX * i;
            if (m < p.M) C[__ldg(p.offCm + m) + cn] = acc[i][j];
        }
    }
}

template <typename T>
cudaError_t launch_typed(const SimtParams& p, cudaStream_t stream)
{
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    const int64_t tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    if (tiles <= 0 || tiles > 0x7fffffffLL) return cudaErrorInvalidValue;
    simt_contract_kernel<T, BM, BN, BK, TM, TN>
        <<<static_cast<unsigned>(tiles), (BM / TM) * (BN / TN), 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_simt_contract(const SimtParams& p, int scalar_type, cudaStream_t stream)
{
    return scalar_type == 1 ? launch_typed<double>(p, stream) : launch_typed<float>(p, stream);
}

}  // namespace tcontb
