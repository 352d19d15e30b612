// dmma_f64.cu -- FP64 direct contraction on the FP64 tensor path (mma.sync m8n8k4), sm_100a.
//
// tcgen05 has no FP64 kind, so FP64 contractions run on warp-level DMMA.  Measured on B200 the
// m8n8k4 path peaks at 37.0 TFLOP/s against 34.1 for plain DFMA, and it needs an eighth of the
// shared-memory operand traffic of a 4x4 register tile, so the kernel is bound by the tensor
// path and by C's write bandwidth rather than by shared memory.  Same GEMM view and offset
// tables as the CUDA-core kernel (simt_contract.cu): any descriptor, ragged extents, C overwritten.
//
// Stands where the reference runs its generated FP64 WMMA kernels
// (backends/cogent/plan/generators/kernels/kernel_compute.py:127-850, wmma m8n8k4 double) and,
// for the transpose-assisted route, its cublasGemmEx FP64 call
// (backends/ttgt_cutt/src/ttgt_cutt.cpp:764-809).
#include <cstdlib>

#include "kernels.hpp"

namespace tcontb {
namespace {

// Block tile BM x BN = (WM x 64) x (WN x 32): every warp owns a 64 x 32 piece, i.e. 8 x 4 m8n8k4
// accumulators.  Operand tiles are gathered straight from global memory into a STAGES-deep ring
// of shared-memory buffers with cp.async (no staging registers), 16 bytes at a time where two
// neighbouring rows of the tile are neighbours in memory.  Row pitches satisfy pitch mod 16 == 4
// so that the fragment loads (row = lane%4, column = lane/4) hit 16 different 8-byte banks per half warp.
template <int WM, int WN, int BK_, int STAGES_>
struct DmmaCfg {
    static constexpr int BM = WM * 64, BN = WN * 32, BK = BK_, STAGES = STAGES_, THREADS = WM * WN * 32;
    static constexpr int LDA = BM + 4, LDB = BN + 4;
    static constexpr int LDK = BK + 4;  // pitch of a K-major operand kept as [row][k] (mode 3); LDK mod 16 == 4 as well
    static constexpr int kADoubles = BK * LDA > BM * LDK ? BK * LDA : BM * LDK;  // either form fits
    static constexpr int kBDoubles = BK * LDB > BN * LDK ? BK * LDB : BN * LDK;
    static constexpr int kStageDoubles = kADoubles + kBDoubles;
    static constexpr int kMaxKTable = 512;  // contracted extents up to this keep their offset tables in shared memory
    // ring of operand stages | K offset tables of A and B | ring of C offset tables (BM + BN entries per tile)
    static constexpr int kSmemBytes = (STAGES * kStageDoubles + 2 * kMaxKTable + STAGES * (BM + BN)) * static_cast<int>(sizeof(double));
    static constexpr int MIN_BLOCKS = THREADS <= 128 ? 2 : 1;
};

__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, bool valid)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(valid ? 8 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Gathers one BK x ROWS operand tile (rows = m or n, pitch LDX) for K offset k0 into shared memory.
// mode 0: threads run along the rows, one element each; mode 1: along k; mode 3: along k, two
// neighbouring k (16 bytes) each, tile kept as [row][k]; mode 2: along the rows,
// two neighbouring rows (16 bytes) each -- legal when the host verified that rows 2r and 2r+1
// are neighbours in memory and 16-byte aligned for every k.  In modes 0 and 2 a thread serves one
// row (pair) for the whole tile, whose offset the caller resolved once (`row_off`, -1 = beyond
// the tensor).  `off_k` points to shared memory when k_shared, else to the global table.
template <int ROWS, int BK, int LDX, int THREADS>
__device__ __forceinline__ void gather_tile(uint32_t smem_tile, const double* __restrict__ X, const int64_t* __restrict__ off_row,
                                            const int64_t* off_k, bool k_shared, int64_t row_off, int64_t row0,
                                            int64_t rows_total, int64_t k0, int64_t k_total, int mode, int tid)
{
    auto koff = [&](int64_t k) { return k_shared ? off_k[k] : __ldg(off_k + k); };
    constexpr int PAIRS = ROWS / 2;
    if (mode == 2 && THREADS % PAIRS == 0) {
        const int rl = (tid % PAIRS) * 2;
#pragma unroll
        for (int i = 0; i < PAIRS * BK / THREADS; ++i) {
            const int kl = tid / PAIRS + i * (THREADS / PAIRS);
            const int64_t k = k0 + kl;
            const bool ok = row_off >= 0 && k < k_total;
            const double* src = ok ? X + row_off + koff(k) : X;
            cp_async_16(smem_tile + static_cast<uint32_t>(kl * LDX + rl) * 8u, src, ok);
        }
    } else if (mode == 0 && THREADS % ROWS == 0) {
        const int rl = tid % ROWS;
#pragma unroll
        for (int i = 0; i < ROWS * BK / THREADS; ++i) {
            const int kl = tid / ROWS + i * (THREADS / ROWS);
            const int64_t k = k0 + kl;
            const bool ok = row_off >= 0 && k < k_total;
            const double* src = ok ? X + row_off + koff(k) : X;
            cp_async_8(smem_tile + static_cast<uint32_t>(kl * LDX + rl) * 8u, src, ok);
        }
    } else if (mode == 3) {
        // K-major operand, two neighbouring k (16 bytes) per copy, stored as [row][k] with pitch BK + 4
        constexpr int KP = BK / 2, LDK = BK + 4;
#pragma unroll
        for (int i = 0; i < ROWS * KP / THREADS; ++i) {
            const int idx = tid + i * THREADS;
            const int kl = (idx % KP) * 2, rl = idx / KP;
            const int64_t r = row0 + rl, k = k0 + kl;
            const bool ok = r < rows_total && k < k_total;  // k_total is even on this path
            const double* src = ok ? X + __ldg(off_row + r) + koff(k) : X;
            cp_async_16(smem_tile + static_cast<uint32_t>(rl * LDK + kl) * 8u, src, ok);
        }
    } else if (mode == 2) {  // more row pairs than threads: resolve the row offset per copy
#pragma unroll
        for (int i = 0; i < PAIRS * BK / THREADS; ++i) {
            const int idx = tid + i * THREADS;
            const int rl = (idx % PAIRS) * 2, kl = idx / PAIRS;
            const int64_t r = row0 + rl, k = k0 + kl;
            const bool ok = r < rows_total && k < k_total;
            const double* src = ok ? X + __ldg(off_row + r) + koff(k) : X;
            cp_async_16(smem_tile + static_cast<uint32_t>(kl * LDX + rl) * 8u, src, ok);
        }
    } else {
#pragma unroll
        for (int i = 0; i < ROWS * BK / THREADS; ++i) {
            const int idx = tid + i * THREADS;
            const int rl = mode == 1 ? idx / BK : idx % ROWS;
            const int kl = mode == 1 ? idx % BK : idx / ROWS;
            const int64_t r = row0 + rl, k = k0 + kl;
            const bool ok = r < rows_total && k < k_total;
            const double* src = ok ? X + __ldg(off_row + r) + koff(k) : X;
            cp_async_8(smem_tile + static_cast<uint32_t>(kl * LDX + rl) * 8u, src, ok);
        }
    }
}

__device__ __forceinline__ void dmma_m8n8k4(double (&c)[2], double a, double b)
{
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                 : "+d"(c[0]), "+d"(c[1])
                 : "d"(a), "d"(b));
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::MIN_BLOCKS) dmma_contract_kernel(SimtParams p)
{
    constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, THREADS = Cfg::THREADS, LDA = Cfg::LDA, LDB = Cfg::LDB;
    constexpr int STAGES = Cfg::STAGES, WM = BM / 64;
    extern __shared__ double smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));

    const double* __restrict__ A = static_cast<const double*>(p.A);
    const double* __restrict__ B = static_cast<const double*>(p.B);
    double* __restrict__ C = static_cast<double*>(p.C);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp % WM, wn = warp / WM;  // warp tile 64 x 32
    const int64_t tiles_m = (p.M + BM - 1) / BM;
    const int64_t tiles = tiles_m * ((p.N + BN - 1) / BN);
    const int nk = static_cast<int>((p.K + BK - 1) / BK);
    // Persistent block: tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The copy ring runs over the
    // flat sequence of (tile, K tile) steps, so the gathers of the next tile are already in flight
    // while this one is multiplied and stored.
    const int64_t my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t steps = my_tiles * nk;

    // shared-memory tables
    int64_t* ktabA = reinterpret_cast<int64_t*>(smem + STAGES * Cfg::kStageDoubles);
    int64_t* ktabB = ktabA + Cfg::kMaxKTable;
    int64_t* ctab = ktabB + Cfg::kMaxKTable;  // [STAGES][BM + BN]: offCm then offCn of the tile, -1 = beyond the tensor
    const uint32_t ctab_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ctab));
    const bool k_shared = p.K <= Cfg::kMaxKTable;
    if (k_shared) {
        for (int64_t k = tid; k < p.K; k += THREADS) {
            ktabA[k] = __ldg(p.offAk + k);
            ktabB[k] = __ldg(p.offBk + k);
        }
        __syncthreads();
    }
    const int64_t* offAk = k_shared ? ktabA : p.offAk;
    const int64_t* offBk = k_shared ? ktabB : p.offBk;

    // Row offsets of the tile whose gathers are being issued (modes 0 and 2: one row or row pair per thread).
    int64_t a_row = -1, b_row = -1;
    auto issue = [&](int64_t q) {
        if (q < steps) {
            const int64_t tl = q / nk;
            const int64_t tile = blockIdx.x + tl * gridDim.x;
            const int kt = static_cast<int>(q % nk);
            const int64_t m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
            if (kt == 0) {
                if (p.a_along_k == 0 || p.a_along_k == 2) {
                    const int64_t m = m0 + (p.a_along_k == 2 ? (tid % (BM / 2)) * 2 : tid % BM);
                    a_row = m < p.M ? __ldg(p.offAm + m) : -1;
                }
                if (p.b_along_k == 0 || p.b_along_k == 2) {
                    const int64_t n = n0 + (p.b_along_k == 2 ? (tid % (BN / 2)) * 2 : tid % BN);
                    b_row = n < p.N ? __ldg(p.offBn + n) : -1;
                }
                // C offsets of this tile travel with its first K tile
                const uint32_t ct = ctab_addr + static_cast<uint32_t>((tl % STAGES) * (BM + BN)) * 8u;
                for (int r = tid; r < BM + BN; r += THREADS) {
                    const bool is_m = r < BM;
                    const int64_t g = is_m ? m0 + r : n0 + (r - BM);
                    const bool ok = g < (is_m ? p.M : p.N);
                    if (ok) cp_async_8(ct + static_cast<uint32_t>(r) * 8u, (is_m ? p.offCm : p.offCn) + g, true);
                    else ctab[(tl % STAGES) * (BM + BN) + r] = -1;
                }
            }
            const uint32_t st = smem_base + static_cast<uint32_t>((q % STAGES) * Cfg::kStageDoubles) * 8u;
            gather_tile<BM, BK, LDA, THREADS>(st, A, p.offAm, offAk, k_shared, a_row, m0, p.M, static_cast<int64_t>(kt) * BK, p.K,
                                              p.a_along_k, tid);
            gather_tile<BN, BK, LDB, THREADS>(st + static_cast<uint32_t>(Cfg::kADoubles) * 8u, B, p.offBn, offBk, k_shared, b_row, n0, p.N,
                                              static_cast<int64_t>(kt) * BK, p.K, p.b_along_k, tid);
        }
        cp_async_commit();  // one group per step, empty past the end, so the wait below counts uniformly
    };

    double acc[8][4][2];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    // fragment coordinates of this lane: A(row = lane/4, k = lane%4), B(k = lane%4, col = lane/4)
    const int fr = lane >> 2, fk = lane & 3;
    const bool a_rowmajor = p.a_along_k == 3, b_rowmajor = p.b_along_k == 3;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    int kt = 0;
    int64_t tile = blockIdx.x, tiles_done = 0;
    for (int64_t q = 0; q < steps; ++q) {
        cp_async_wait<STAGES - 2>();  // step q has landed (for this thread's copies)
        __syncthreads();              // ... and for everyone's; the buffer refilled below was read at step q-1
        const double* As = smem + (q % STAGES) * Cfg::kStageDoubles;
        const double* Bs = As + Cfg::kADoubles;
#pragma unroll
        for (int k4 = 0; k4 < BK; k4 += 4) {
            double a[8], b[4];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                a[i] = a_rowmajor ? As[(wm * 64 + i * 8 + fr) * Cfg::LDK + k4 + fk] : As[(k4 + fk) * LDA + wm * 64 + i * 8 + fr];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                b[j] = b_rowmajor ? Bs[(wn * 32 + j * 8 + fr) * Cfg::LDK + k4 + fk] : Bs[(k4 + fk) * LDB + wn * 32 + j * 8 + fr];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) dmma_m8n8k4(acc[i][j], a[i], b[j]);
        }
        // refill the buffer everyone finished reading before the barrier above; issued after this
        // step's MMAs so the tensor path is fed first and the address arithmetic overlaps it
        issue(q + STAGES - 1);
        if (++kt < nk) continue;
        // last K tile of this output tile: store it (accumulator fragment: rows lane/4, columns
        // 2*(lane%4) and 2*(lane%4)+1) and start the next one from zero
        const int64_t* ct = ctab + (tiles_done % STAGES) * (BM + BN);
        int64_t cm[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) cm[i] = ct[wm * 64 + i * 8 + fr];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t cn = ct[BM + wn * 32 + j * 8 + 2 * fk + h];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (cn >= 0 && cm[i] >= 0) __stcs(C + cm[i] + cn, acc[i][j][h]);
                    acc[i][j][h] = 0.0;
                }
            }
        }
        ++tiles_done;
        kt = 0;
        tile += gridDim.x;
    }
    cp_async_wait<0>();
}

// Two shapes: 128 x 128 (8 warps, one block per SM) for long contracted extents, and 128 x 64
// (4 warps, two blocks per SM) for short ones, where a tile is mostly set-up latency and output
// stores and a second resident block hides them.
using CfgBig = DmmaCfg<2, 4, 16, 3>;
using CfgSmall = DmmaCfg<2, 2, 16, 3>;
using CfgSkinny = DmmaCfg<4, 1, 16, 3>;  // 256 x 32: contractions whose N side is a single short mode

cudaError_t dmma_configure()
{
    cudaError_t e = cudaFuncSetAttribute(dmma_contract_kernel<CfgBig>, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgBig::kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(dmma_contract_kernel<CfgSkinny>, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgSkinny::kSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(dmma_contract_kernel<CfgSmall>, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgSmall::kSmemBytes);
}

template <class Cfg>
cudaError_t launch_cfg(const SimtParams& p, int num_sms, cudaStream_t stream)
{
    const int64_t tiles = ((p.M + Cfg::BM - 1) / Cfg::BM) * ((p.N + Cfg::BN - 1) / Cfg::BN);
    if (tiles <= 0) return cudaErrorInvalidValue;
    const int64_t resident = static_cast<int64_t>(num_sms) * Cfg::MIN_BLOCKS;
    dmma_contract_kernel<Cfg><<<static_cast<unsigned>(tiles < resident ? tiles : resident), Cfg::THREADS, Cfg::kSmemBytes, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t dmma_configure_all() { return dmma_configure(); }

cudaError_t launch_dmma_contract(const SimtParams& p, int num_sms, cudaStream_t stream)
{
    int which = p.N <= 48 ? 3 : p.K <= 256 ? 1 : 2;
    if (const char* e = std::getenv("TCONT_DMMA_CFG"))  // tuning switch: 1 = 128x64, 2 = 128x128, 3 = 256x32
        if (e[0] >= '1' && e[0] <= '3') which = e[0] - '0';
    return which == 3 ? launch_cfg<CfgSkinny>(p, num_sms, stream)
         : which == 1 ? launch_cfg<CfgSmall>(p, num_sms, stream)
                      : launch_cfg<CfgBig>(p, num_sms, stream);
}

}  // namespace tcontb
