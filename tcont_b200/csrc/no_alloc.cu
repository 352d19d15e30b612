// no_alloc.cu -- one contraction entry point that never allocates device memory.
//
// Some callers cannot let a library call cudaMalloc on their behalf: a serving process whose
// memory pool reserved the whole GPU at start-up (there is nothing left for the driver to hand
// out), or a latency-critical loop that cannot afford the device-wide synchronisation an
// allocation implies.  The regular run objects allocate (tensors, transpose scratch, the offset
// tables of the CUDA-core kernel).  This entry point runs the same CUDA-core contraction kernel
// on the caller's own A, B and C and keeps the kernel's only scratch -- the six offset tables of
// the GEMM view -- in a fixed array that is part of the library image.
//
// Consequences of the fixed array, all documented in include/tcontb.h:
//   * it costs kNoAllocScratchBytes on every GPU that loads the library, until the process ends;
//   * contractions whose tables do not fit are rejected, never truncated;
//   * all calls share it, so two calls that overlap on the GPU (different streams, or different
//     host threads) race; calls on one stream are safe;
//   * it keeps whatever the previous call left; each call's table kernel overwrites exactly the part
//     its contraction kernel reads, on the same stream, so nothing needs to start at zero.
// The tables are computed on the device from per-mode extents and strides passed as kernel arguments:
// the call copies nothing from host memory and never makes the host wait for the stream.
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/tcontb.h"
#include "kernels.hpp"
#include "planner.hpp"

namespace {

constexpr size_t kNoAllocScratchBytes = size_t(4) << 20;  // 4 MiB
constexpr size_t kNoAllocScratchEntries = kNoAllocScratchBytes / sizeof(long long);

// File-scope device array.  In host code this name is only a handle for the runtime; the device
// address is obtained with cudaGetSymbolAddress below and that pointer is what the kernel gets.
static __device__ __align__(256) long long g_no_alloc_tables[kNoAllocScratchEntries];

// Per-mode description of the three index groups (0: rows of A and C, 1: rows of B and C, 2: contracted),
// passed by value; table entry i of group g is the mixed-radix number i over the group's extents, dotted
// with the group's strides in its two tensors.
struct TableSpec {
    int n_modes[3];
    long long total[3];
    long long extent[3][tcontb::kMaxModes];
    long long stride_x[3][tcontb::kMaxModes];
    long long stride_y[3][tcontb::kMaxModes];
    long long* out_x[3];
    long long* out_y[3];
};

__global__ void __launch_bounds__(256) fill_offset_tables_kernel(const __grid_constant__ TableSpec s)
{
    const int g = blockIdx.y;
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= s.total[g]) return;
    long long rem = i, x = 0, y = 0;
    for (int m = 0; m < s.n_modes[g]; ++m) {
        const long long idx = rem % s.extent[g][m];
        rem /= s.extent[g][m];
        x += idx * s.stride_x[g][m];
        y += idx * s.stride_y[g][m];
    }
    s.out_x[g][i] = x;
    s.out_y[g][i] = y;
}

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
long long* g_tables_on_device[kMaxDevices] = {nullptr};

thread_local std::string g_no_alloc_error;

// Once per device, with that device current: resolve the array's device address.
cudaError_t scratch_for_current_device(long long** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_tables_on_device[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_no_alloc_tables);
        if (e != cudaSuccess) return e;
        g_tables_on_device[dev] = static_cast<long long*>(p);
    }
    *out = g_tables_on_device[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" const char* tcontb_no_alloc_last_error(void) { return g_no_alloc_error.c_str(); }

extern "C" tcontb_status tcontb_contract_no_alloc(const tcontb_desc* d, const void* a_dev, const void* b_dev, void* c_dev,
                                                  void* cuda_stream)
{
    using namespace tcontb;
    auto fail = [](tcontb_status st, const std::string& msg) {
        g_no_alloc_error = msg;
        return st;
    };
    if (!d || !a_dev || !b_dev || !c_dev) return fail(TCONTB_INVALID_ARGUMENT, "Null descriptor or device buffer");

    // Host-side planning only (host memory, no CUDA call); always the direct route, so A and B are
    // read where they lie and no transposed copy is needed.
    Plan plan;
    std::string err;
    const int rc = make_plan(d->modeC, d->nC, d->modeA, d->nA, d->modeB, d->nB, d->op, d->scalar_type, d->ext_mode, d->ext_val,
                             d->n_ext, TCONTB_SELECT_DIRECT, CostTable(), &plan, &err);
    if (rc) return fail(static_cast<tcontb_status>(rc), err);
    const Problem& p = plan.prob;
    const size_t need = 2 * static_cast<size_t>(p.Mtot + p.Ntot + p.Ktot);
    if (need > kNoAllocScratchEntries)
        return fail(TCONTB_UNSUPPORTED,
                    "contraction too large for the allocation-free entry point: its offset tables need " +
                        std::to_string(need * sizeof(long long)) + " bytes, the built-in scratch holds " +
                        std::to_string(kNoAllocScratchBytes) + " (2*(M+N+K) must not exceed " +
                        std::to_string(kNoAllocScratchEntries) + "); use a run object instead");

    long long* scratch = nullptr;
    cudaError_t e = scratch_for_current_device(&scratch);
    if (e != cudaSuccess) return fail(TCONTB_RUNTIME_ERROR, std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));

    // The six tables are written by a small kernel on the caller's stream from the per-mode extents and
    // strides, which travel by value as kernel arguments: no host buffer outlives this call, the host does
    // not wait for earlier work on the stream, and the contraction kernel behind it sees finished tables.
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    TableSpec spec{};
    const std::vector<int>* groups[3] = {&p.M, &p.N, &p.K};
    const int64_t totals[3] = {p.Mtot, p.Ntot, p.Ktot};
    size_t at[6];
    {
        // order in the array: offAm, offAk, offBn, offBk, offCm, offCn
        const size_t len[6] = {size_t(p.Mtot), size_t(p.Ktot), size_t(p.Ntot), size_t(p.Ktot), size_t(p.Mtot), size_t(p.Ntot)};
        size_t pos = 0;
        for (int i = 0; i < 6; ++i) {
            at[i] = pos;
            pos += len[i];
        }
    }
    for (int g = 0; g < 3; ++g) {
        spec.n_modes[g] = static_cast<int>(groups[g]->size());
        spec.total[g] = totals[g];
        for (size_t i = 0; i < groups[g]->size() && i < static_cast<size_t>(kMaxModes); ++i) {
            const Mode& m = p.modes[static_cast<size_t>((*groups[g])[i])];
            spec.extent[g][i] = m.extent;
            // M rows index A and C, N rows index B and C, K indexes A and B
            spec.stride_x[g][i] = g == 0 ? m.sA : g == 1 ? m.sB : m.sA;
            spec.stride_y[g][i] = g == 0 ? m.sC : g == 1 ? m.sC : m.sB;
        }
    }
    spec.out_x[0] = scratch + at[0];  // offAm
    spec.out_y[0] = scratch + at[4];  // offCm
    spec.out_x[1] = scratch + at[2];  // offBn
    spec.out_y[1] = scratch + at[5];  // offCn
    spec.out_x[2] = scratch + at[1];  // offAk
    spec.out_y[2] = scratch + at[3];  // offBk
    const int64_t longest = std::max(p.Mtot, std::max(p.Ntot, p.Ktot));
    const dim3 grid(static_cast<unsigned>((longest + 255) / 256), 3);
    fill_offset_tables_kernel<<<grid, 256, 0, stream>>>(spec);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TCONTB_RUNTIME_ERROR, std::string("table kernel launch failed: ") + cudaGetErrorString(e));

    const int64_t* base = reinterpret_cast<const int64_t*>(scratch);
    SimtParams sp{};
    sp.A = p.swapped ? b_dev : a_dev;
    sp.B = p.swapped ? a_dev : b_dev;
    sp.C = c_dev;
    sp.M = p.Mtot;
    sp.N = p.Ntot;
    sp.K = p.Ktot;
    sp.offAm = base + at[0];
    sp.offAk = base + at[1];
    sp.offBn = base + at[2];
    sp.offBk = base + at[3];
    sp.offCm = base + at[4];
    sp.offCn = base + at[5];
    sp.a_along_k = plan.simt.a_load_along_k;
    sp.b_along_k = plan.simt.b_load_along_k;
    e = launch_simt_contract(sp, plan.scalar_type, stream);
    if (e != cudaSuccess) return fail(TCONTB_RUNTIME_ERROR, std::string("kernel launch failed: ") + cudaGetErrorString(e));
    return TCONTB_OK;
}
