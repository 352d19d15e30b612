// api.cpp -- the C ABI of include/tcontb.h: plan and run objects around the sm_100a kernels.
#include <cuda.h>
#include <cuda_runtime.h>

#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <ctime>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/tcontb.h"
#include "kernels.hpp"
#include "planner.hpp"

using namespace tcontb;

struct tcontb_plan {
    Plan plan;
};

namespace {

thread_local std::string g_last_error;

tcontb_status fail(tcontb_status st, const std::string& msg)
{
    g_last_error = msg;
    return st;
}

#define TC_CUDA(expr)                                                                                     \
    do {                                                                                                  \
        const cudaError_t e_ = (expr);                                                                    \
        if (e_ != cudaSuccess)                                                                            \
            return fail(TCONTB_RUNTIME_ERROR, std::string("CUDA error in " #expr ": ") + cudaGetErrorString(e_)); \
    } while (0)

inline uint64_t splitmix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// The cost table plans are made with: the compiled-in defaults, overridden by the file TCONT_COST_TABLE names;
// without that variable, by `tcont_cost_table.<device name>.txt` beside this library, where
// `python -m tcont_b200.calibrate` writes what it measured on that kind of GPU (spaces in the name become '_').
// The SM count always comes from the current device.  Without a usable device the plan is made for the
// defaults (planning itself needs no GPU).  Cached per device.
CostTable device_cost_table()
{
    static std::mutex mu;
    static std::map<int, CostTable> cache;
    int n = 0, dev = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0 || cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return load_cost_table();
    }
    std::lock_guard<std::mutex> lock(mu);
    const bool from_env = std::getenv("TCONT_COST_TABLE") != nullptr;
    auto it = cache.find(dev);
    if (it != cache.end() && !from_env) return it->second;
    CostTable c = load_cost_table();
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) c.num_sms = sms;
    if (from_env) return c;  // (not cached: tests and tools switch files through the environment)
    cudaDeviceProp prop;
    Dl_info info;
    if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess && dladdr(reinterpret_cast<const void*>(&device_cost_table), &info) && info.dli_fname) {
        std::string name = prop.name, dir = info.dli_fname;
        for (char& ch : name)
            if (ch == ' ' || ch == '/') ch = '_';
        const size_t slash = dir.rfind('/');
        dir = slash == std::string::npos ? "." : dir.substr(0, slash);
        read_cost_table_file(dir + "/tcont_cost_table." + name + ".txt", &c);
        if (sms > 0) c.num_sms = sms;
    } else {
        cudaGetLastError();
    }
    cache[dev] = c;
    return c;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

struct DeviceBuffer {
    void* ptr = nullptr;
    ~DeviceBuffer()
    {
        if (ptr) cudaFree(ptr);
    }
    cudaError_t alloc(size_t bytes) { return cudaMalloc(&ptr, bytes ? bytes : 1); }
};

// Restores the device that was current when a multi-GPU function started, on every way out of it.
struct DeviceGuard {
    int device;
    bool active;
    explicit DeviceGuard(int d, bool on) : device(d), active(on) {}
    ~DeviceGuard()
    {
        if (active) cudaSetDevice(device);
    }
};

}  // namespace

struct tcontb_run {
    Plan plan;
    int device = 0;
    int num_sms = 148;
    cudaStream_t stream = nullptr;
    size_t elt = 8;
    // caller-facing buffers: L (left), R (right), C
    DeviceBuffer ownL, ownR, ownC;
    void *dL = nullptr, *dR = nullptr, *dC = nullptr;
    std::vector<unsigned char> hL, hR;
    bool has_host = false;
    // transpose scratch for role A / role B
    DeviceBuffer tbufA, tbufB;
    // A part of a pipelined host-buffer pass may use the transposed copy another part makes of the operand all
    // parts share (borrowed_tA / borrowed_tB: that part's scratch; this run then neither allocates nor transposes).
    const void *borrowed_tA = nullptr, *borrowed_tB = nullptr;
    TransposeParams tpA{}, tpB{};
    // SIMT tables
    DeviceBuffer tables;
    SimtParams simt{};
    // UMMA
    UmmaParams umma{};
    CUtensorMap tmA{}, tmB{};
    DeviceBuffer status;
    DeviceBuffer splitk;  // partial tensors of a split-K contraction, k_splits copies of C (three times that with tf32x3)
    // Error-compensated Float32 (TCONT_TF32X3=1, tcgen05 kernel only): the part of each operand that
    // narrowing to TF32 drops, its tensor maps, and where the kernel's operands lie.
    bool tf32x3 = false;
    DeviceBuffer loA, loB;
    CUtensorMap tmAlo{}, tmBlo{};
    const void *kernA = nullptr, *kernB = nullptr;
    int64_t kernA_elements = 0, kernB_elements = 0;
    DeviceBuffer prof;  // cycle counters of the tcgen05 kernel, only with TCONT_UMMA_PROF=1
    DeviceBuffer pace;  // progress counters of the tcgen05 kernel's pace keeping (see UmmaParams)
    size_t pace_bytes = 0;
    // C = alpha * (A*B) + beta * C (tcontb_run_set_scalars); the reference's semantics are alpha 1, beta 0.
    // With other values the contraction writes a workspace and the partial-sum pass applies the scalars.
    double alpha = 1.0, beta = 0.0;
    DeviceBuffer scaled_ws;
    // stage timing
    bool stage_timing = false;
    cudaEvent_t ev[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    bool ev_valid = false;
    int64_t kernels_per_launch = 0;
    // Several GPUs of one box behind one run (TCONT_NUM_GPUS > 1): the contraction is cut along an
    // external mode, shard g lives on device first_device + g and is an ordinary run of the
    // smaller contraction; this object then only keeps the global host inputs.
    std::vector<std::unique_ptr<tcontb_run>> shards;
    std::vector<cudaEvent_t> shard_done;
    int first_device = 0;
    bool one_device = false;  // test mode (TCONT_SHARDS_ON_ONE_DEVICE=1): every shard lives on the first device
    char split_mode = 0;
    bool split_contracted = false;        // the shards cut a contracted mode (TCONT_SPLIT=k:<mode>)
    std::vector<cudaEvent_t> shard_kernel;  // shard g's contraction kernel of the current launch has finished
    int shard_device(size_t g) const { return one_device ? first_device : first_device + static_cast<int>(g); }
    // Contracted-mode split (tcontb_run_ksplit_*): this run contracts its slice of a contracted mode into a
    // partial C that never exists as a whole.  C is cut into `world` contiguous ranges along its slowest mode;
    // the kernel stores the tile columns of range o straight into slot [set][rank] of the staging area of the
    // GPU that owns range o (its own, or a peer's over NVLink), and the owner sums its `world` slots.
    // Two sets of slots alternate between launches, so that one barrier per launch (every rank's kernel done
    // before any rank's sum) is all the ordering the ranks need.
    struct KSplit {
        int world = 0, rank = 0;
        int64_t chunk = 0;                    // elements of one range
        DeviceBuffer staging;                 // [2 sets][world slots][chunk]
        void* peer[kMaxOwners] = {nullptr};   // every rank's staging area as this process sees it
        bool opened[kMaxOwners] = {false};    // mapped through an IPC handle (closed with the run)
        int set = 0, last_set = 0;
    } ks;
    // Pipelined host-buffer pass (tcontb_run_contract_host): when C's slowest mode is external and is
    // also the slowest mode of the operand that carries it, a slice of that mode is a contiguous range
    // of the operand and of C.  The contraction is then cut into `parts` along it, each an ordinary
    // run working in place on its ranges of this run's device buffers, so that the upload of slice
    // i+1, the kernels of slice i and the download of slice i-1 overlap (PCIe is full duplex).
    struct HostPipeline {
        bool tried = false;
        bool in_left = false;  // the caller's left operand carries the cut mode
        size_t slice_in = 0, slice_out = 0;  // bytes per part
        // The cut mode is not the slowest mode of the operand that carries it: a part's slice of that operand is
        // `rows` pieces of `width` bytes, `pitch` bytes apart (uploaded by a 2-D copy; the part's plan sees a view).
        bool strided = false;
        size_t width = 0, pitch = 0, rows = 0;
        std::vector<std::unique_ptr<tcontb_run>> parts;
        cudaStream_t s_in = nullptr, s_out = nullptr;
        cudaEvent_t ev_start = nullptr, ev_other = nullptr;
        std::vector<cudaEvent_t> ev_in, ev_done;
    } pipe;

    ~tcontb_run()
    {
        for (int o = 0; o < kMaxOwners; ++o)
            if (ks.opened[o] && ks.peer[o]) cudaIpcCloseMemHandle(ks.peer[o]);
        for (size_t g = 0; g < shards.size(); ++g) {
            cudaSetDevice(shard_device(g));
            shards[g].reset();
            if (g < shard_done.size() && shard_done[g]) cudaEventDestroy(shard_done[g]);
            if (g < shard_kernel.size() && shard_kernel[g]) cudaEventDestroy(shard_kernel[g]);
        }
        if (!shard_done.empty()) cudaSetDevice(first_device);
        if (prof.ptr) {
            // Tuning aid: mean cycles per CTA spent in each role's waits during the last launch.
            std::vector<long long> h(static_cast<size_t>(num_sms) * 8);
            if (cudaMemcpy(h.data(), prof.ptr, h.size() * sizeof(long long), cudaMemcpyDeviceToHost) == cudaSuccess) {
                double s[8] = {0};
                int n = 0;
                for (int b = 0; b < num_sms; ++b)
                    if (h[static_cast<size_t>(b) * 8 + 4] > 0) {
                        ++n;
                        for (int i = 0; i < 8; ++i) s[i] += double(h[static_cast<size_t>(b) * 8 + i]);
                    }
                if (n && plan.kernel == KERNEL_DMMA_F64_TMA)
                    std::fprintf(stderr, "[tcontb prof] ctas=%d group0_total=%.0f wait_stage_full=%.0f main_loop=%.0f tables=%.0f "
                                 "stores=%.0f token_wait=%.0f (cycles, mean per CTA, consumer group 0)\n",
                                 n, s[0] / n, s[1] / n, s[2] / n, s[3] / n, s[4] / n, s[5] / n);
                else if (n)
                    std::fprintf(stderr, "[tcontb prof] ctas=%d mma_total=%.0f mma_wait_acc_empty=%.0f mma_wait_stage_full=%.0f "
                                 "producer_wait_stage_empty=%.0f epilogue_total=%.0f epilogue_wait_acc_full=%.0f pace_cycles=%.0f pace_waits_x2=%.1f "
                                 "(cycles, mean per CTA; MMA figures over issuing CTAs)\n",
                                 n, s[0] / n, s[1] / n, s[2] / n, s[3] / n, s[4] / n, s[5] / n, s[6] / n, s[7] / n);
            }
        }
        for (auto& e : ev)
            if (e) cudaEventDestroy(e);
        pipe.parts.clear();
        for (auto& e : pipe.ev_in) cudaEventDestroy(e);
        for (auto& e : pipe.ev_done) cudaEventDestroy(e);
        if (pipe.ev_start) cudaEventDestroy(pipe.ev_start);
        if (pipe.ev_other) cudaEventDestroy(pipe.ev_other);
        if (pipe.s_in) cudaStreamDestroy(pipe.s_in);
        if (pipe.s_out) cudaStreamDestroy(pipe.s_out);
    }
    const void* roleA_src() const { return plan.prob.swapped ? dR : dL; }
    const void* roleB_src() const { return plan.prob.swapped ? dL : dR; }
};

namespace {

void fill_operand_dev(const UmmaOperand& o, UmmaOperandDev* d)
{
    d->major = o.major;
    d->slab_w = o.slab_w;
    d->slabs_per_tile = o.slabs_per_tile;
    d->n_row_digits = o.n_row_digits;
    d->slab_bytes = o.slab_bytes;
    d->slabs_per_op = o.slabs_per_op;
    d->digit0_scale = o.digit0_scale;
    d->k0_scale = o.k0_scale;
    d->chunk_digit = o.chunk_digit;
    d->oob_coord = o.oob_coord;
    for (int i = 0; i < kMaxTmaRank; ++i) {
        d->row_digit_dim[i] = i < o.n_row_digits ? o.row_digit_dim[i] : -1;
        d->row_digit_ext[i] = i < o.n_row_digits ? static_cast<int>(o.row_digit_ext[i]) : 1;
        d->row_digit_cstride[i] = i < o.n_row_digits ? o.row_digit_cstride[i] : 0;
    }
    d->row_elem_cstride = o.row_elem_cstride;
    d->slab_mode_ext = static_cast<int>(o.slab_mode_ext);
    d->total_slabs = o.total_slabs;
    for (int i = 0; i < 3; ++i) d->k_digit_dim[i] = o.k_digit_dim[i];
    d->split_inner = static_cast<int>(o.split_inner);
    d->split_outer_cstride = o.split_outer_cstride;
}

tcontb_status encode_map(const UmmaOperand& o, const void* base, int elt, CUtensorMap* out)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(TCONTB_RUNTIME_ERROR, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    cuuint64_t dims[kMaxTmaRank];
    cuuint64_t strides[kMaxTmaRank - 1];
    cuuint32_t box[kMaxTmaRank], estr[kMaxTmaRank];
    for (int d = 0; d < kMaxTmaRank; ++d) {
        dims[d] = static_cast<cuuint64_t>(o.ext[d]);
        box[d] = static_cast<cuuint32_t>(o.box[d]);
        estr[d] = 1;
        if (d > 0) strides[d - 1] = static_cast<cuuint64_t>(o.stride[d]) * static_cast<cuuint64_t>(elt);
    }
    const CUresult r = fn(out, elt == 8 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT64 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, kMaxTmaRank, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          // an MN-major 32-bit operand must be swizzled in 32-byte units for tcgen05.mma;
                          // FP64 operands may have 64-byte rows (8 doubles of the k chunk or of the slab mode)
                          (o.major && elt == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                          : (o.box[0] * elt == 64) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TCONTB_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return TCONTB_OK;
}

// Device-side set-up shared by the three run constructors; dL/dR/dC must already be set.
tcontb_status finish_run(tcontb_run* run)
{
    const Plan& pl = run->plan;
    const Problem& p = pl.prob;
    TC_CUDA(cudaGetDevice(&run->device));
    TC_CUDA(cudaDeviceGetAttribute(&run->num_sms, cudaDevAttrMultiProcessorCount, run->device));
    int major = 0;
    TC_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, run->device));
    if (major != 10) return fail(TCONTB_RUNTIME_ERROR, "this library holds sm_100a kernels only; the current device is not a B200-class GPU");

    const void* kA = run->roleA_src();
    const void* kB = run->roleB_src();
    run->kernels_per_launch = 1;
    if (pl.tA.needed && run->borrowed_tA) {
        kA = run->borrowed_tA;
    } else if (pl.tA.needed) {
        if (!make_transpose_params(pl.tA.rank, pl.tA.src_extent, pl.tA.perm, &run->tpA, pl.tA.strided_src ? pl.tA.src_stride : nullptr))
            return fail(TCONTB_RUNTIME_ERROR, "bad transpose plan for A");
        TC_CUDA(run->tbufA.alloc(static_cast<size_t>(pl.tA.elements) * run->elt));
        kA = run->tbufA.ptr;
        run->kernels_per_launch++;
    }
    if (pl.tB.needed && run->borrowed_tB) {
        kB = run->borrowed_tB;
    } else if (pl.tB.needed) {
        if (!make_transpose_params(pl.tB.rank, pl.tB.src_extent, pl.tB.perm, &run->tpB, pl.tB.strided_src ? pl.tB.src_stride : nullptr))
            return fail(TCONTB_RUNTIME_ERROR, "bad transpose plan for B");
        TC_CUDA(run->tbufB.alloc(static_cast<size_t>(pl.tB.elements) * run->elt));
        kB = run->tbufB.ptr;
        run->kernels_per_launch++;
    }
    TC_CUDA(run->status.alloc(sizeof(int)));
    TC_CUDA(cudaMemset(run->status.ptr, 0, sizeof(int)));

    if (pl.kernel == KERNEL_UMMA_TF32 || pl.kernel == KERNEL_DMMA_F64_TMA) {
        const UmmaSpec& u = pl.umma;
        fill_operand_dev(u.a, &run->umma.a);
        fill_operand_dev(u.b, &run->umma.b);
        run->umma.BN = u.BN;
        run->umma.BK = u.BK;
        run->umma.stages = u.stages;
        run->umma.pair = u.pair ? 1 : 0;
        run->umma.producers = u.producers;
        run->umma.store_across_slabs = u.store_across_slabs ? 1 : 0;
        run->umma.n_k_digits = u.n_k_digits;
        for (int i = 0; i < 3; ++i) run->umma.k_digit_ext[i] = static_cast<int>(u.k_digit_ext[i]);
        run->umma.k_iters = static_cast<int>(u.k_iters);
        run->umma.tiles_m = u.tiles_m;
        run->umma.tiles_n = u.tiles_n;
        run->umma.raster_group = u.raster_group;
        run->umma.k_splits = u.k_splits;
        run->umma.k_iters_per_split = static_cast<int>(u.k_iters_per_split);
        run->umma.split_stride = pl.sizeC;
        void* out = run->dC;
        const char* x3 = std::getenv("TCONT_TF32X3");
        run->tf32x3 = pl.kernel == KERNEL_UMMA_TF32 && x3 && x3[0] == '1' && !p.strided;
        if (u.k_splits > 1 || run->tf32x3) {
            TC_CUDA(run->splitk.alloc(static_cast<size_t>(run->tf32x3 ? 3 : 1) * static_cast<size_t>(u.k_splits) *
                                      static_cast<size_t>(pl.sizeC) * run->elt));
            out = run->splitk.ptr;
            run->kernels_per_launch++;
        }
        if (run->tf32x3) {
            // C = hi(A) hi(B) + hi(A) lo(B) + lo(A) hi(B): the tensor core takes hi() itself (it truncates),
            // lo() is computed per launch into these buffers, and the three products are partials of the
            // split-K sum.  Accuracy is that of fp32 accumulation; the cost is three contractions.
            run->kernA = kA;
            run->kernB = kB;
            run->kernA_elements = pl.tA.needed ? pl.tA.elements : (p.swapped ? pl.sizeR : pl.sizeL);
            run->kernB_elements = pl.tB.needed ? pl.tB.elements : (p.swapped ? pl.sizeL : pl.sizeR);
            TC_CUDA(run->loA.alloc(static_cast<size_t>(run->kernA_elements) * run->elt));
            TC_CUDA(run->loB.alloc(static_cast<size_t>(run->kernB_elements) * run->elt));
            run->kernels_per_launch += 4;  // two residual passes, two more contractions
        }
        run->umma.C = static_cast<float*>(out);
        run->umma.C64 = static_cast<double*>(out);
        run->umma.status = static_cast<int*>(run->status.ptr);
        run->umma.prof = nullptr;
        run->umma.wait_limit_ns = 0;
        run->umma.test_skip_iter = -1;
        // Test hooks of the bounded-wait exit (tcgen05 kernel only; see UmmaParams).
        if (const char* e = std::getenv("TCONT_TEST_WAIT_LIMIT_NS")) run->umma.wait_limit_ns = std::strtoull(e, nullptr, 10);
        if (const char* e = std::getenv("TCONT_TEST_SKIP_STAGE")) run->umma.test_skip_iter = std::atoi(e);
        if (const char* pe = std::getenv("TCONT_UMMA_PROF")) {
            if (pe[0] == '1') {
                TC_CUDA(run->prof.alloc(static_cast<size_t>(run->num_sms) * 8 * sizeof(long long)));
                TC_CUDA(cudaMemset(run->prof.ptr, 0, static_cast<size_t>(run->num_sms) * 8 * sizeof(long long)));
                run->umma.prof = static_cast<long long*>(run->prof.ptr);
            }
        }
        run->umma.pace = nullptr;
        if (pl.kernel == KERNEL_UMMA_TF32) {
            // Pace keeping pays where the CTAs walk long panels that do not fit into L2 together: a full grid with
            // several work units each, 32 or more k iterations per unit, operands of 64 MB or more (the large 4-D
            // configuration: 28 -> 21 GB read from DRAM per launch, 2 to 4 % less time; on another GPU 47 GB without).
            // TCONT_UMMA_PACE=0/1 overrides the rule; lead and block size: TCONT_UMMA_PACE_LEAD / _SHIFT.
            const int64_t units = (u.pair ? (u.tiles_m + 1) / 2 : u.tiles_m) * u.tiles_n * u.k_splits;
            const int64_t ctas = std::max<int64_t>(1, std::min<int64_t>(units, u.pair ? run->num_sms / 2 : run->num_sms));
            const int64_t a_elems = pl.tA.needed ? pl.tA.elements : (p.swapped ? pl.sizeR : pl.sizeL);
            const int64_t b_elems = pl.tB.needed ? pl.tB.elements : (p.swapped ? pl.sizeL : pl.sizeR);
            bool pace = units >= 2 * ctas && u.k_iters_per_split >= 32 && (a_elems + b_elems) * static_cast<int64_t>(run->elt) >= (64ll << 20);
            if (const char* pe = std::getenv("TCONT_UMMA_PACE")) pace = pe[0] == '1';
            if (pace) {
                const char* le = std::getenv("TCONT_UMMA_PACE_LEAD");
                const char* se = std::getenv("TCONT_UMMA_PACE_SHIFT");
                run->umma.pace_lead = le ? std::max(1, std::atoi(le)) : 2;
                run->umma.pace_shift = se ? std::min(10, std::max(0, std::atoi(se))) : 4;
                const int64_t iters = ((units + ctas - 1) / ctas) * (u.k_iters_per_split + 1);
                run->pace_bytes = static_cast<size_t>((iters >> run->umma.pace_shift) + 4) * sizeof(unsigned int);
                TC_CUDA(run->pace.alloc(run->pace_bytes));
                run->umma.pace = static_cast<unsigned int*>(run->pace.ptr);
            }
        }
        tcontb_status st = encode_map(u.a, kA, u.elt, &run->tmA);
        if (st != TCONTB_OK) return st;
        st = encode_map(u.b, kB, u.elt, &run->tmB);
        if (st != TCONTB_OK) return st;
        if (run->tf32x3) {
            st = encode_map(u.a, run->loA.ptr, u.elt, &run->tmAlo);
            if (st != TCONTB_OK) return st;
            st = encode_map(u.b, run->loB.ptr, u.elt, &run->tmBlo);
            if (st != TCONTB_OK) return st;
        }
        if (u.smem_bytes > kMaxDynamicSmemBytes) return fail(TCONTB_RUNTIME_ERROR, "plan asks for more shared memory than a block can have");
        if (pl.kernel == KERNEL_UMMA_TF32) TC_CUDA(umma_tf32_configure());
        else TC_CUDA(dmma_tma_configure());
    } else {
        OffsetTables t;
        build_offset_tables(p, &t);
        const size_t n = t.offAm.size() + t.offAk.size() + t.offBn.size() + t.offBk.size() + t.offCm.size() + t.offCn.size();
        std::vector<int64_t> flat;
        flat.reserve(n);
        size_t o[6];
        const std::vector<int64_t>* src[6] = {&t.offAm, &t.offAk, &t.offBn, &t.offBk, &t.offCm, &t.offCn};
        for (int i = 0; i < 6; ++i) {
            o[i] = flat.size();
            flat.insert(flat.end(), src[i]->begin(), src[i]->end());
        }
        TC_CUDA(run->tables.alloc(n * sizeof(int64_t)));
        TC_CUDA(cudaMemcpy(run->tables.ptr, flat.data(), n * sizeof(int64_t), cudaMemcpyHostToDevice));
        const int64_t* base = static_cast<const int64_t*>(run->tables.ptr);
        run->simt.A = kA;
        run->simt.B = kB;
        run->simt.C = run->dC;
        run->simt.M = p.Mtot;
        run->simt.N = p.Ntot;
        run->simt.K = p.Ktot;
        run->simt.offAm = base + o[0];
        run->simt.offAk = base + o[1];
        run->simt.offBn = base + o[2];
        run->simt.offBk = base + o[3];
        run->simt.offCm = base + o[4];
        run->simt.offCn = base + o[5];
        run->simt.a_along_k = pl.simt.a_load_along_k;
        run->simt.b_along_k = pl.simt.b_load_along_k;
        if (pl.kernel == KERNEL_DMMA_F64) {
            TC_CUDA(dmma_configure_all());
            // 16-byte gathers: rows 2r and 2r+1 of the tile must be neighbours in memory, on a
            // 16-byte boundary, for every contracted index.
            auto pairs_ok = [](const std::vector<int64_t>& row, const std::vector<int64_t>& k) {
                if (row.size() % 2) return false;
                for (size_t r = 0; r < row.size(); r += 2)
                    if ((row[r] & 1) || row[r + 1] != row[r] + 1) return false;
                for (int64_t v : k)
                    if (v & 1) return false;
                return true;
            };
            // K-major operand: neighbouring k neighbours in memory, every row offset even
            auto kpairs_ok = [](const std::vector<int64_t>& row, const std::vector<int64_t>& k) {
                if (k.size() % 2) return false;
                for (size_t i = 0; i < k.size(); i += 2)
                    if ((k[i] & 1) || k[i + 1] != k[i] + 1) return false;
                for (int64_t v : row)
                    if (v & 1) return false;
                return true;
            };
            if (run->simt.a_along_k == 1 && kpairs_ok(t.offAm, t.offAk) && reinterpret_cast<uintptr_t>(kA) % 16 == 0) run->simt.a_along_k = 3;
            if (run->simt.b_along_k == 1 && kpairs_ok(t.offBn, t.offBk) && reinterpret_cast<uintptr_t>(kB) % 16 == 0) run->simt.b_along_k = 3;
            if (run->simt.a_along_k == 0 && pairs_ok(t.offAm, t.offAk) && reinterpret_cast<uintptr_t>(kA) % 16 == 0) run->simt.a_along_k = 2;
            if (run->simt.b_along_k == 0 && pairs_ok(t.offBn, t.offBk) && reinterpret_cast<uintptr_t>(kB) % 16 == 0) run->simt.b_along_k = 2;
        }
    }
    const char* st_env = std::getenv("TCONT_STAGE_TIMES");
    run->stage_timing = st_env && std::strcmp(st_env, "1") == 0;
    if (run->stage_timing)
        for (auto& e : run->ev) TC_CUDA(cudaEventCreate(&e));
    return TCONTB_OK;
}

tcontb_status alloc_owned(tcontb_run* run)
{
    const Plan& pl = run->plan;
    TC_CUDA(run->ownL.alloc(static_cast<size_t>(pl.sizeL) * run->elt));
    TC_CUDA(run->ownR.alloc(static_cast<size_t>(pl.sizeR) * run->elt));
    TC_CUDA(run->ownC.alloc(static_cast<size_t>(pl.sizeC) * run->elt));
    run->dL = run->ownL.ptr;
    run->dR = run->ownR.ptr;
    run->dC = run->ownC.ptr;
    TC_CUDA(cudaMemset(run->dC, 0, static_cast<size_t>(pl.sizeC) * run->elt));
    return TCONTB_OK;
}

tcontb_status check_device()
{
    int n = 0;
    const cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(TCONTB_RUNTIME_ERROR, "no usable CUDA device (this engine has no CPU path)");
    }
    return TCONTB_OK;
}

tcontb_status new_run(const tcontb_plan* plan, std::unique_ptr<tcontb_run>* out)
{
    if (!plan) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionPlan is empty");
    const tcontb_status st = check_device();
    if (st != TCONTB_OK) return st;
    out->reset(new tcontb_run());
    (*out)->plan = plan->plan;
    (*out)->elt = plan->plan.scalar_type == TCONTB_F64 ? 8 : 4;
    return TCONTB_OK;
}

// Copies the slice [lo, lo+len) of `mode` out of (or, with scatter = true, back into) a
// column-major tensor: `full` has the global extents, `part` the sliced one.
void slice_mode(unsigned char* full, unsigned char* part, const std::string& modes, const Plan& pl, char mode, int64_t lo,
                int64_t len, size_t elt, bool scatter)
{
    const size_t pos = modes.find(mode);
    auto ext = [&](char c) { return pl.ext_val[pl.ext_mode.find(c)]; };
    int64_t inner = 1, outer = 1;
    for (size_t i = 0; i < modes.size(); ++i) {
        if (i < pos) inner *= ext(modes[i]);
        else if (i > pos) outer *= ext(modes[i]);
    }
    const int64_t e = ext(mode);
    const size_t run_bytes = static_cast<size_t>(len * inner) * elt;
    for (int64_t o = 0; o < outer; ++o) {
        unsigned char* f = full + static_cast<size_t>((o * e + lo) * inner) * elt;
        unsigned char* q = part + static_cast<size_t>(o * len * inner) * elt;
        if (scatter) std::memcpy(f, q, run_bytes);
        else std::memcpy(q, f, run_bytes);
    }
}

int requested_gpus()
{
    const char* e = std::getenv("TCONT_NUM_GPUS");
    const int g = e ? std::atoi(e) : 1;
    return g > 1 ? g : 1;
}

// Builds the shards of a multi-GPU run; `run` already holds the global plan and host inputs.
// Returns TCONTB_OK with run->shards empty when no external mode divides over the GPUs.
tcontb_status make_shards(tcontb_run* run, int gpus)
{
    const Plan& pl = run->plan;
    int have = 0;
    TC_CUDA(cudaGetDeviceCount(&have));
    TC_CUDA(cudaGetDevice(&run->first_device));
    DeviceGuard guard(run->first_device, true);
    // Test mode: every shard on the first device (the slicing, routing, joining and gathering logic then runs on
    // a box with one GPU; the shards' kernels run one after the other, none waits for another).
    if (const char* od = std::getenv("TCONT_SHARDS_ON_ONE_DEVICE")) run->one_device = od[0] == '1';
    if (!run->one_device && run->first_device + gpus > have)
        return fail(TCONTB_RUNTIME_ERROR, "TCONT_NUM_GPUS asks for more devices than the box has from the current device on");
    auto external = [&](char c) {
        return pl.modeC.find(c) != std::string::npos && ((pl.modeA.find(c) != std::string::npos) != (pl.modeB.find(c) != std::string::npos));
    };
    auto ext = [&](char c) { return pl.ext_val[pl.ext_mode.find(c)]; };
    char mode = 0;
    auto contracted = [&](char c) {
        return pl.modeC.find(c) == std::string::npos && pl.modeA.find(c) != std::string::npos && pl.modeB.find(c) != std::string::npos;
    };
    const char* sp = std::getenv("TCONT_SPLIT");
    if (sp && std::strncmp(sp, "k:", 2) == 0) {  // "k:<mode>": cut a contracted mode; partial tiles go straight to their owners
        if (!sp[2] || !contracted(sp[2]) || ext(sp[2]) % gpus || gpus > kMaxOwners)
            return fail(TCONTB_INVALID_ARGUMENT, "TCONT_SPLIT=k:<mode> must name a contracted mode whose extent divides over the GPUs (8 at most)");
        mode = sp[2];
        run->split_contracted = true;
    } else if (sp) {  // "ext:<mode>"
        if (std::strncmp(sp, "ext:", 4) != 0 || !sp[4] || !external(sp[4]) || ext(sp[4]) % gpus)
            return fail(TCONTB_INVALID_ARGUMENT, "TCONT_SPLIT must be ext:<mode> naming an external mode, or k:<mode> naming a contracted one, whose extent divides over the GPUs");
        mode = sp[4];
    } else {
        // slowest mode of C first: its slices are contiguous blocks of C
        for (size_t i = pl.modeC.size(); i-- > 0 && !mode;)
            if (external(pl.modeC[i]) && ext(pl.modeC[i]) % gpus == 0) mode = pl.modeC[i];
        if (!mode) return TCONTB_OK;
    }
    run->split_mode = mode;
    const int64_t len = ext(mode) / gpus;
    std::vector<int64_t> local_ext = pl.ext_val;
    local_ext[pl.ext_mode.find(mode)] = len;
    const bool in_a = pl.modeA.find(mode) != std::string::npos;
    for (int g = 0; g < gpus; ++g) {
        TC_CUDA(cudaSetDevice(run->shard_device(static_cast<size_t>(g))));
        std::unique_ptr<tcontb_run> sh(new tcontb_run());
        std::string err;
        const int rc = make_plan(pl.modeC.data(), static_cast<int>(pl.modeC.size()), pl.modeA.data(), static_cast<int>(pl.modeA.size()),
                                 pl.modeB.data(), static_cast<int>(pl.modeB.size()), pl.op, pl.scalar_type, pl.ext_mode.data(),
                                 local_ext.data(), static_cast<int>(local_ext.size()), pl.backend_selection, device_cost_table(),
                                 &sh->plan, &err);
        if (rc) return fail(static_cast<tcontb_status>(rc), err);
        sh->elt = run->elt;
        const size_t bl = static_cast<size_t>(sh->plan.sizeL) * run->elt, br = static_cast<size_t>(sh->plan.sizeR) * run->elt;
        sh->hL.resize(bl);
        sh->hR.resize(br);
        if (run->split_contracted) {  // both inputs carry the cut mode
            slice_mode(run->hL.data(), sh->hL.data(), pl.modeA, pl, mode, g * len, len, run->elt, false);
            slice_mode(run->hR.data(), sh->hR.data(), pl.modeB, pl, mode, g * len, len, run->elt, false);
        } else if (in_a) {
            slice_mode(run->hL.data(), sh->hL.data(), pl.modeA, pl, mode, g * len, len, run->elt, false);
            sh->hR = run->hR;
        } else {
            sh->hL = run->hL;
            slice_mode(run->hR.data(), sh->hR.data(), pl.modeB, pl, mode, g * len, len, run->elt, false);
        }
        tcontb_status st = alloc_owned(sh.get());
        if (st != TCONTB_OK) return st;
        TC_CUDA(cudaMemcpy(sh->dL, sh->hL.data(), bl, cudaMemcpyHostToDevice));
        TC_CUDA(cudaMemcpy(sh->dR, sh->hR.data(), br, cudaMemcpyHostToDevice));
        sh->hL.clear();
        sh->hL.shrink_to_fit();
        sh->hR.clear();
        sh->hR.shrink_to_fit();
        st = finish_run(sh.get());
        if (st != TCONTB_OK) return st;
        cudaEvent_t ev = nullptr;
        TC_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        run->shard_done.push_back(ev);
        if (run->split_contracted) {
            st = tcontb_run_ksplit_enable(sh.get(), gpus, g);
            if (st != TCONTB_OK) return st;
            cudaEvent_t ek = nullptr;
            TC_CUDA(cudaEventCreateWithFlags(&ek, cudaEventDisableTiming));
            run->shard_kernel.push_back(ek);
        }
        run->shards.push_back(std::move(sh));
    }
    if (run->split_contracted) {
        // every shard stores into every other shard's staging area: peer access both ways, then the pointers
        for (int g = 0; g < gpus; ++g) {
            TC_CUDA(cudaSetDevice(run->shard_device(static_cast<size_t>(g))));
            for (int h = 0; h < gpus; ++h) {
                if (h == g) continue;
                if (!run->one_device) {
                    const cudaError_t pe = cudaDeviceEnablePeerAccess(run->shard_device(static_cast<size_t>(h)), 0);
                    if (pe == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                    else if (pe != cudaSuccess) return fail(TCONTB_RUNTIME_ERROR, std::string("peer access between the GPUs of the split is not available: ") + cudaGetErrorString(pe));
                }
                const tcontb_status as = tcontb_run_ksplit_attach(run->shards[static_cast<size_t>(g)].get(), h, run->shards[static_cast<size_t>(h)].get());
                if (as != TCONTB_OK) return as;
            }
        }
    }
    TC_CUDA(cudaSetDevice(run->first_device));
    run->kernels_per_launch = 0;
    for (auto& sh : run->shards) run->kernels_per_launch += sh->kernels_per_launch;
    return TCONTB_OK;
}

// Builds the parts of the pipelined host-buffer pass, if the descriptor allows it (see HostPipeline).
// TCONT_HOST_CHUNKS=<n> forces the number of parts (0 or 1: one pass, no overlap).
tcontb_status build_host_pipeline(tcontb_run* run)
{
    auto& pp = run->pipe;
    pp.tried = true;
    const Plan& pl = run->plan;
    if (!run->shards.empty() || pl.modeC.empty()) return TCONTB_OK;
    const char mode = pl.modeC.back();
    const bool left = pl.modeA.find(mode) != std::string::npos, right = pl.modeB.find(mode) != std::string::npos;
    if (left == right) return TCONTB_OK;
    const std::string& carrier = left ? pl.modeA : pl.modeB;
    const int64_t ext = pl.ext_val[pl.ext_mode.find(mode)];
    // Where the cut mode is not the carrier's slowest mode, a part's slice of the carrier is a sub-tensor view:
    // `rows` pieces (one per index of the modes behind the cut mode) of `width` bytes each, `pitch` bytes apart.
    const bool strided = carrier.back() != mode;
    std::vector<int64_t> carrier_parent;
    int64_t inner = 1, outer = 1;
    {
        const size_t pos = carrier.find(mode);
        for (size_t i = 0; i < carrier.size(); ++i) {
            const int64_t e = pl.ext_val[pl.ext_mode.find(carrier[i])];
            carrier_parent.push_back(e);
            if (i < pos) inner *= e;
            else if (i > pos) outer *= e;
        }
    }
    const size_t in_bytes = static_cast<size_t>(left ? pl.sizeL : pl.sizeR) * run->elt, out_bytes = static_cast<size_t>(pl.sizeC) * run->elt;
    int64_t n = 0;
    if (const char* e = std::getenv("TCONT_HOST_CHUNKS")) {
        n = std::atoll(e);
        if (n < 2 || ext % n) return TCONTB_OK;
    } else {
        // as many parts as leave 16 MB of C per part, 16 at most (the first upload and the last download
        // are the only transfers nothing overlaps)
        for (int64_t c : {16, 12, 8, 6, 4, 3, 2})
            if (!n && ext % c == 0 && out_bytes / static_cast<size_t>(c) >= (size_t(16) << 20)) n = c;
        if (!n) return TCONTB_OK;
    }
    pp.slice_in = in_bytes / static_cast<size_t>(n);
    pp.slice_out = out_bytes / static_cast<size_t>(n);
    pp.strided = strided;
    pp.width = static_cast<size_t>(inner * (ext / n)) * run->elt;
    pp.pitch = static_cast<size_t>(inner * ext) * run->elt;
    pp.rows = static_cast<size_t>(outer);
    if (pp.slice_in % 16 || pp.slice_out % 16 || (strided && pp.width % 16)) return TCONTB_OK;
    std::vector<int64_t> local_ext = pl.ext_val;
    local_ext[pl.ext_mode.find(mode)] = ext / n;
    std::vector<std::unique_ptr<tcontb_run>> parts;
    for (int64_t i = 0; i < n; ++i) {
        std::unique_ptr<tcontb_run> part(new tcontb_run());
        std::string err;
        const int rc = make_plan(pl.modeC.data(), static_cast<int>(pl.modeC.size()), pl.modeA.data(), static_cast<int>(pl.modeA.size()),
                                 pl.modeB.data(), static_cast<int>(pl.modeB.size()), pl.op, pl.scalar_type, pl.ext_mode.data(),
                                 local_ext.data(), static_cast<int>(local_ext.size()), pl.backend_selection, device_cost_table(),
                                 &part->plan, &err, nullptr, strided && left ? carrier_parent.data() : nullptr,
                                 strided && !left ? carrier_parent.data() : nullptr);
        if (rc) return fail(static_cast<tcontb_status>(rc), err);
        part->elt = run->elt;
        part->stream = run->stream;
        // contiguous slices lie one after the other; a view starts (i * ext / n) indices of the cut mode into the carrier
        const size_t in_offset = strided ? static_cast<size_t>(i) * pp.width : static_cast<size_t>(i) * pp.slice_in;
        unsigned char* in = static_cast<unsigned char*>(left ? run->dL : run->dR) + in_offset;
        part->dL = left ? static_cast<void*>(in) : run->dL;
        part->dR = left ? run->dR : static_cast<void*>(in);
        part->dC = static_cast<unsigned char*>(run->dC) + static_cast<size_t>(i) * pp.slice_out;
        // the operand every part shares is transposed once, by the first part; the others read its copy
        if (!parts.empty()) {
            const bool carrier_is_role_a = part->plan.prob.swapped ? !left : left;
            if (carrier_is_role_a && part->plan.tB.needed && parts[0]->plan.tB.needed) part->borrowed_tB = parts[0]->tbufB.ptr;
            if (!carrier_is_role_a && part->plan.tA.needed && parts[0]->plan.tA.needed) part->borrowed_tA = parts[0]->tbufA.ptr;
        }
        const tcontb_status st = finish_run(part.get());
        if (st != TCONTB_OK) return st;
        parts.push_back(std::move(part));
    }
    TC_CUDA(cudaStreamCreateWithFlags(&pp.s_in, cudaStreamNonBlocking));
    TC_CUDA(cudaStreamCreateWithFlags(&pp.s_out, cudaStreamNonBlocking));
    TC_CUDA(cudaEventCreateWithFlags(&pp.ev_start, cudaEventDisableTiming));
    TC_CUDA(cudaEventCreateWithFlags(&pp.ev_other, cudaEventDisableTiming));
    for (int64_t i = 0; i < n; ++i) {
        cudaEvent_t a = nullptr, b = nullptr;
        TC_CUDA(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        pp.ev_in.push_back(a);
        TC_CUDA(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        pp.ev_done.push_back(b);
    }
    pp.in_left = left;
    pp.parts = std::move(parts);
    return TCONTB_OK;
}

#define TC_NOT_SHARDED(run, what)                                                                              \
    if (!(run)->shards.empty()) return fail(TCONTB_UNSUPPORTED, what " is not available on a multi-GPU run")

}  // namespace

// A bounded device-side wait that gave up leaves C partly written and only raises the run's status word.
// The entry points that hand results to the caller synchronise anyway; they read the word there (of the
// run, its shards and its parts), so that no caller of this C ABI or of the C++ surface above it takes a
// partial result for a good one.
static tcontb_status fail_if_device_gave_up(tcontb_run* run)
{
    int status = 0;
    const tcontb_status st = tcontb_run_device_status(run, &status);
    if (st != TCONTB_OK) return st;
    if (status != 0)
        return fail(TCONTB_RUNTIME_ERROR, "a bounded device wait gave up (device status " + std::to_string(status) +
                                              "): the output tensor is incomplete");
    return TCONTB_OK;
}

extern "C" {

const char* tcontb_last_error(void) { return g_last_error.c_str(); }

tcontb_status tcontb_plan_create(const tcontb_desc* d, tcontb_plan** out)
{
    if (!d || !out) return fail(TCONTB_INVALID_ARGUMENT, "Null descriptor or output pointer");
    std::unique_ptr<tcontb_plan> pl(new tcontb_plan());
    std::string err;
    const int rc = make_plan(d->modeC, d->nC, d->modeA, d->nA, d->modeB, d->nB, d->op, d->scalar_type, d->ext_mode, d->ext_val,
                             d->n_ext, d->backend_selection, device_cost_table(), &pl->plan, &err);
    if (rc) return fail(static_cast<tcontb_status>(rc), err);
    *out = pl.release();
    return TCONTB_OK;
}

tcontb_status tcontb_plan_create_strided(const tcontb_desc* d, const int64_t* parent_c, const int64_t* parent_a, const int64_t* parent_b,
                                         tcontb_plan** out)
{
    if (!d || !out) return fail(TCONTB_INVALID_ARGUMENT, "Null descriptor or output pointer");
    std::unique_ptr<tcontb_plan> pl(new tcontb_plan());
    std::string err;
    const int rc = make_plan(d->modeC, d->nC, d->modeA, d->nA, d->modeB, d->nB, d->op, d->scalar_type, d->ext_mode, d->ext_val,
                             d->n_ext, d->backend_selection, device_cost_table(), &pl->plan, &err, parent_c, parent_a, parent_b);
    if (rc) return fail(static_cast<tcontb_status>(rc), err);
    *out = pl.release();
    return TCONTB_OK;
}

void tcontb_plan_destroy(tcontb_plan* plan) { delete plan; }

int tcontb_plan_backend(const tcontb_plan* plan) { return plan ? plan->plan.backend : -1; }

double tcontb_plan_flops(const tcontb_plan* plan) { return plan ? plan->plan.flops : 0.0; }

tcontb_status tcontb_plan_describe(const tcontb_plan* plan, char* buf, size_t n)
{
    if (!plan || !buf || n == 0) return fail(TCONTB_INVALID_ARGUMENT, "Null plan or buffer");
    const std::string s = describe_plan(plan->plan);
    if (s.size() + 1 > n) return fail(TCONTB_INVALID_ARGUMENT, "Buffer too small for the plan description");
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return TCONTB_OK;
}

tcontb_status tcontb_fill_uniform(void* dst, int scalar_type, int64_t n, uint64_t seed, uint64_t offset, double lo, double hi)
{
    if (!dst || n < 0 || (scalar_type != TCONTB_F32 && scalar_type != TCONTB_F64))
        return fail(TCONTB_INVALID_ARGUMENT, "Bad arguments to tcontb_fill_uniform");
    const uint64_t base = seed * 0x9E3779B97F4A7C15ull + offset;
    for (int64_t i = 0; i < n; ++i) {
        const double u = static_cast<double>(splitmix64(base + static_cast<uint64_t>(i)) >> 11) * (1.0 / 9007199254740992.0);
        const double v = lo + (hi - lo) * u;
        if (scalar_type == TCONTB_F64) static_cast<double*>(dst)[i] = v;
        else static_cast<float*>(dst)[i] = static_cast<float>(v);
    }
    return TCONTB_OK;
}

tcontb_status tcontb_run_create_with_inputs(const tcontb_plan* plan, const void* a_host, const void* b_host, tcontb_run** out)
{
    if (!out) return fail(TCONTB_INVALID_ARGUMENT, "Null output pointer");
    if (!a_host || !b_host) return fail(TCONTB_INVALID_ARGUMENT, "Null input buffer");
    if (plan && plan->plan.prob.strided)
        return fail(TCONTB_UNSUPPORTED, "a plan over sub-tensor views runs on caller-owned device buffers (tcontb_run_create_on_device)");
    std::unique_ptr<tcontb_run> run;
    tcontb_status st = new_run(plan, &run);
    if (st != TCONTB_OK) return st;
    const Plan& pl = run->plan;
    const size_t bl = static_cast<size_t>(pl.sizeL) * run->elt, br = static_cast<size_t>(pl.sizeR) * run->elt;
    run->hL.assign(static_cast<const unsigned char*>(a_host), static_cast<const unsigned char*>(a_host) + bl);
    run->hR.assign(static_cast<const unsigned char*>(b_host), static_cast<const unsigned char*>(b_host) + br);
    run->has_host = true;
    if (requested_gpus() > 1) {
        st = make_shards(run.get(), requested_gpus());
        if (st != TCONTB_OK) return st;
        if (!run->shards.empty()) {
            *out = run.release();
            return TCONTB_OK;
        }
    }
    st = alloc_owned(run.get());
    if (st != TCONTB_OK) return st;
    TC_CUDA(cudaMemcpy(run->dL, run->hL.data(), bl, cudaMemcpyHostToDevice));
    TC_CUDA(cudaMemcpy(run->dR, run->hR.data(), br, cudaMemcpyHostToDevice));
    st = finish_run(run.get());
    if (st != TCONTB_OK) return st;
    *out = run.release();
    return TCONTB_OK;
}

tcontb_status tcontb_run_create(const tcontb_plan* plan, tcontb_run** out)
{
    if (!plan) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionPlan is empty");
    if (!out) return fail(TCONTB_INVALID_ARGUMENT, "Null output pointer");
    const Plan& pl = plan->plan;
    const size_t elt = pl.scalar_type == TCONTB_F64 ? 8 : 4;
    uint64_t seed = static_cast<uint64_t>(std::time(nullptr));
    if (const char* s = std::getenv("TCONT_SEED")) seed = std::strtoull(s, nullptr, 10);
    double lo = 0.0, hi = 1.0;
    if (const char* r = std::getenv("TCONT_INPUT_RANGE")) {
        if (std::sscanf(r, "%lf:%lf", &lo, &hi) != 2) return fail(TCONTB_INVALID_ARGUMENT, "TCONT_INPUT_RANGE must look like lo:hi");
    }
    std::vector<unsigned char> a(static_cast<size_t>(pl.sizeL) * elt), b(static_cast<size_t>(pl.sizeR) * elt);
    tcontb_fill_uniform(a.data(), pl.scalar_type, pl.sizeL, seed, 0, lo, hi);
    tcontb_fill_uniform(b.data(), pl.scalar_type, pl.sizeR, seed, static_cast<uint64_t>(pl.sizeL), lo, hi);
    return tcontb_run_create_with_inputs(plan, a.data(), b.data(), out);
}

tcontb_status tcontb_run_create_on_device(const tcontb_plan* plan, const void* a_dev, const void* b_dev, void* c_dev,
                                          tcontb_run** out)
{
    if (!out) return fail(TCONTB_INVALID_ARGUMENT, "Null output pointer");
    if (!a_dev || !b_dev || !c_dev) return fail(TCONTB_INVALID_ARGUMENT, "Null device buffer");
    if ((reinterpret_cast<uintptr_t>(a_dev) | reinterpret_cast<uintptr_t>(b_dev) | reinterpret_cast<uintptr_t>(c_dev)) & 15)
        return fail(TCONTB_INVALID_ARGUMENT, "Device buffers must be 16-byte aligned");
    std::unique_ptr<tcontb_run> run;
    tcontb_status st = new_run(plan, &run);
    if (st != TCONTB_OK) return st;
    run->dL = const_cast<void*>(a_dev);
    run->dR = const_cast<void*>(b_dev);
    run->dC = c_dev;
    st = finish_run(run.get());
    if (st != TCONTB_OK) return st;
    *out = run.release();
    return TCONTB_OK;
}

void tcontb_run_destroy(tcontb_run* run) { delete run; }

tcontb_status tcontb_run_set_stream(tcontb_run* run, void* cuda_stream)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    TC_NOT_SHARDED(run, "a caller stream");
    run->stream = static_cast<cudaStream_t>(cuda_stream);
    for (auto& part : run->pipe.parts) part->stream = run->stream;
    return TCONTB_OK;
}

tcontb_status tcontb_run_upload_inputs(tcontb_run* run, const void* a_host, const void* b_host)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    if (!a_host || !b_host) return fail(TCONTB_INVALID_ARGUMENT, "Null input buffer");
    TC_NOT_SHARDED(run, "replacing the inputs");
    if (run->plan.prob.strided) return fail(TCONTB_UNSUPPORTED, "replacing the inputs is not available on sub-tensor views");
    const Plan& pl = run->plan;
    TC_CUDA(cudaMemcpyAsync(run->dL, a_host, static_cast<size_t>(pl.sizeL) * run->elt, cudaMemcpyHostToDevice, run->stream));
    TC_CUDA(cudaMemcpyAsync(run->dR, b_host, static_cast<size_t>(pl.sizeR) * run->elt, cudaMemcpyHostToDevice, run->stream));
    return TCONTB_OK;
}

tcontb_status tcontb_run_set_scalars(tcontb_run* run, double alpha, double beta)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    if (!std::isfinite(alpha) || !std::isfinite(beta)) return fail(TCONTB_INVALID_ARGUMENT, "alpha and beta must be finite");
    TC_NOT_SHARDED(run, "alpha and beta");
    const bool scaled = alpha != 1.0 || beta != 0.0;
    if (scaled && run->plan.prob.c_strided) return fail(TCONTB_UNSUPPORTED, "alpha and beta are not available when C is a sub-tensor view");
    if (scaled && !run->splitk.ptr && !run->scaled_ws.ptr) {
        // allocated here, once, so that launches stay free of allocations
        TC_CUDA(run->scaled_ws.alloc(static_cast<size_t>(run->plan.sizeC) * run->elt));
    }
    const bool was = run->alpha != 1.0 || run->beta != 0.0;
    if (!run->splitk.ptr) run->kernels_per_launch += (scaled ? 1 : 0) - (was ? 1 : 0);
    run->alpha = alpha;
    run->beta = beta;
    // the parts of a pipelined host-buffer pass work on ranges of this run's C
    for (auto& part : run->pipe.parts) {
        const tcontb_status st = tcontb_run_set_scalars(part.get(), alpha, beta);
        if (st != TCONTB_OK) return st;
    }
    return TCONTB_OK;
}

tcontb_status tcontb_run_launch(tcontb_run* run)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    if (!run->shards.empty()) {
        DeviceGuard guard(run->first_device, true);
        // Every shard runs on its own device's NULL stream; the first device's NULL stream then waits
        // for all of them, so events the caller records there bracket the whole multi-GPU launch.
        const size_t G = run->shards.size();
        for (size_t g = 0; g < G; ++g) {
            TC_CUDA(cudaSetDevice(run->shard_device(g)));
            if (run->split_contracted)  // the sums of the previous launch read what this launch's peers are about to overwrite two launches on
                for (size_t h = 0; h < G; ++h)
                    if (h != g) TC_CUDA(cudaStreamWaitEvent(nullptr, run->shard_done[h], 0));
            const tcontb_status st = tcontb_run_launch(run->shards[g].get());
            if (st != TCONTB_OK) {
                cudaSetDevice(run->first_device);
                return st;
            }
            if (run->split_contracted) TC_CUDA(cudaEventRecord(run->shard_kernel[g], nullptr));
            else TC_CUDA(cudaEventRecord(run->shard_done[g], nullptr));
        }
        if (run->split_contracted) {
            // every shard's kernel has stored its partial tiles into the owners' slots: each owner adds its slots up
            for (size_t g = 0; g < G; ++g) {
                TC_CUDA(cudaSetDevice(run->shard_device(g)));
                for (size_t h = 0; h < G; ++h)
                    if (h != g) TC_CUDA(cudaStreamWaitEvent(nullptr, run->shard_kernel[h], 0));
                const tcontb_status st = tcontb_run_ksplit_reduce(run->shards[g].get());
                if (st != TCONTB_OK) return st;
                TC_CUDA(cudaEventRecord(run->shard_done[g], nullptr));
            }
        }
        TC_CUDA(cudaSetDevice(run->first_device));
        for (size_t g = 1; g < run->shards.size(); ++g) TC_CUDA(cudaStreamWaitEvent(nullptr, run->shard_done[g], 0));
        return TCONTB_OK;
    }
    const Plan& pl = run->plan;
    const bool t = run->stage_timing;
    // Other scalars than (1, 0): the kernel writes the workspace instead of C (a split-K run does anyway)
    const bool scaled = run->alpha != 1.0 || run->beta != 0.0;
    const bool redirect = scaled && !run->splitk.ptr;
    UmmaParams umma = run->umma;
    SimtParams simt = run->simt;
    if (redirect) {
        umma.C = static_cast<float*>(run->scaled_ws.ptr);
        umma.C64 = static_cast<double*>(run->scaled_ws.ptr);
        simt.C = run->scaled_ws.ptr;
    }
    if (t) TC_CUDA(cudaEventRecord(run->ev[0], run->stream));
    if (pl.tA.needed && !run->borrowed_tA) TC_CUDA(launch_transpose(run->roleA_src(), run->tbufA.ptr, run->tpA, static_cast<int>(run->elt), run->stream));
    if (t) TC_CUDA(cudaEventRecord(run->ev[1], run->stream));
    if (pl.tB.needed && !run->borrowed_tB) TC_CUDA(launch_transpose(run->roleB_src(), run->tbufB.ptr, run->tpB, static_cast<int>(run->elt), run->stream));
    if (t) TC_CUDA(cudaEventRecord(run->ev[2], run->stream));
    if (pl.kernel == KERNEL_UMMA_TF32 && run->tf32x3) {
        TC_CUDA(launch_tf32_residual(static_cast<const float*>(run->kernA), static_cast<float*>(run->loA.ptr), run->kernA_elements, run->stream));
        TC_CUDA(launch_tf32_residual(static_cast<const float*>(run->kernB), static_cast<float*>(run->loB.ptr), run->kernB_elements, run->stream));
        const CUtensorMap* maps[3][2] = {{&run->tmA, &run->tmB}, {&run->tmA, &run->tmBlo}, {&run->tmAlo, &run->tmB}};
        for (int pass = 0; pass < 3; ++pass) {
            UmmaParams q = umma;
            q.C = static_cast<float*>(run->splitk.ptr) + static_cast<long long>(pass) * pl.umma.k_splits * pl.sizeC;
            if (q.pace) TC_CUDA(cudaMemsetAsync(q.pace, 0, run->pace_bytes, run->stream));   // (a copy-engine node, not a kernel)
            TC_CUDA(launch_umma_tf32(q, maps[pass][0], maps[pass][1], pl.umma.smem_bytes, run->num_sms, run->stream));
        }
    } else if (pl.kernel == KERNEL_UMMA_TF32) {
        if (run->ks.world > 1) {
            // contracted-mode split: tile columns of range o go to slot [set][rank] of owner o's staging area
            auto& ks = run->ks;
            if (scaled) return fail(TCONTB_UNSUPPORTED, "alpha and beta are not available with a contracted-mode split");
            umma.owners = ks.world;
            umma.tn_per_owner = static_cast<int>(pl.umma.tiles_n / ks.world);
            umma.tn_rotate = ((ks.rank + 1) % ks.world) * umma.tn_per_owner;
            for (int o = 0; o < ks.world; ++o) {
                if (!ks.peer[o]) return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split: the staging area of rank " + std::to_string(o) + " was never attached");
                umma.owner_base[o] = static_cast<float*>(ks.peer[o]) + (static_cast<int64_t>(ks.set) * ks.world + ks.rank) * ks.chunk -
                                     static_cast<int64_t>(o) * ks.chunk;
            }
            ks.last_set = ks.set;
            ks.set ^= 1;
        }
        if (umma.pace) TC_CUDA(cudaMemsetAsync(umma.pace, 0, run->pace_bytes, run->stream));
        TC_CUDA(launch_umma_tf32(umma, &run->tmA, &run->tmB, pl.umma.smem_bytes, run->num_sms, run->stream));
    }
    else if (pl.kernel == KERNEL_DMMA_F64_TMA)
        TC_CUDA(launch_dmma_tma(umma, &run->tmA, &run->tmB, pl.umma.smem_bytes, run->num_sms, run->stream));
    else if (pl.kernel == KERNEL_DMMA_F64)
        TC_CUDA(launch_dmma_contract(simt, run->num_sms, run->stream));
    else
        TC_CUDA(launch_simt_contract(simt, pl.scalar_type, run->stream));
    if (run->splitk.ptr)
        TC_CUDA(launch_splitk_reduce(run->splitk.ptr, run->dC, pl.sizeC, pl.umma.k_splits * (run->tf32x3 ? 3 : 1), pl.sizeC,
                                     static_cast<int>(run->elt), run->stream, run->alpha, run->beta));
    else if (redirect)
        TC_CUDA(launch_splitk_reduce(run->scaled_ws.ptr, run->dC, pl.sizeC, 1, pl.sizeC, static_cast<int>(run->elt), run->stream,
                                     run->alpha, run->beta));
    if (t) {
        TC_CUDA(cudaEventRecord(run->ev[3], run->stream));
        run->ev_valid = true;
    }
    return TCONTB_OK;
}

tcontb_status tcontb_run_warmup(tcontb_run* run, int iterations)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    for (int i = 0; i < iterations; ++i) {
        const tcontb_status st = tcontb_run_launch(run);
        if (st != TCONTB_OK) return st;
    }
    DeviceGuard guard(run->first_device, !run->shards.empty());
    for (size_t g = 0; g < run->shards.size(); ++g) {
        TC_CUDA(cudaSetDevice(run->shard_device(g)));
        TC_CUDA(cudaDeviceSynchronize());
    }
    if (!run->shards.empty()) TC_CUDA(cudaSetDevice(run->first_device));
    TC_CUDA(cudaDeviceSynchronize());
    return TCONTB_OK;
}

tcontb_status tcontb_run_zero_output(tcontb_run* run)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    if (!run->shards.empty()) {
        DeviceGuard guard(run->first_device, true);
        for (size_t g = 0; g < run->shards.size(); ++g) {
            TC_CUDA(cudaSetDevice(run->shard_device(g)));
            const tcontb_status st = tcontb_run_zero_output(run->shards[g].get());
            if (st != TCONTB_OK) return st;
        }
        TC_CUDA(cudaSetDevice(run->first_device));
        return TCONTB_OK;
    }
    if (run->plan.prob.c_strided) return fail(TCONTB_UNSUPPORTED, "zero_output is not available when C is a sub-tensor view (the caller owns the parent tensor)");
    TC_CUDA(cudaMemsetAsync(run->dC, 0, static_cast<size_t>(run->plan.sizeC) * run->elt, run->stream));
    return TCONTB_OK;
}

tcontb_status tcontb_run_stage_times(tcontb_run* run, float out[6])
{
    if (!run || !out) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    for (int i = 0; i < 6; ++i) out[i] = 0.0f;
    if (!run->shards.empty()) return tcontb_run_stage_times(run->shards[0].get(), out);  // the first device's stages
    if (!run->stage_timing || !run->ev_valid) return TCONTB_OK;
    TC_CUDA(cudaEventSynchronize(run->ev[3]));
    float ta = 0, tb = 0, tc = 0;
    TC_CUDA(cudaEventElapsedTime(&ta, run->ev[0], run->ev[1]));
    TC_CUDA(cudaEventElapsedTime(&tb, run->ev[1], run->ev[2]));
    TC_CUDA(cudaEventElapsedTime(&tc, run->ev[2], run->ev[3]));
    // a route without a transpose reports zero for it (the few microseconds between two events that bracket
    // nothing are not a stage)
    if (!run->plan.tA.needed) ta = 0.0f;
    if (!run->plan.tB.needed) tb = 0.0f;
    out[0] = 1.0f;
    out[1] = ta + tb + tc;
    out[2] = run->plan.prob.swapped ? tb : ta;  // reported per caller operand: left, right
    out[3] = run->plan.prob.swapped ? ta : tb;
    out[4] = tc;
    out[5] = 0.0f;  // C is written in its final order by the contraction kernel
    return TCONTB_OK;
}

const void* tcontb_run_host_input(const tcontb_run* run, int which)
{
    if (!run || !run->has_host) return nullptr;
    return which == 0 ? static_cast<const void*>(run->hL.data()) : static_cast<const void*>(run->hR.data());
}

tcontb_status tcontb_run_copy_output(tcontb_run* run, void* dst, size_t bytes)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    if (!dst) return fail(TCONTB_INVALID_ARGUMENT, "Destination buffer is null");
    if (run->plan.prob.c_strided) return fail(TCONTB_UNSUPPORTED, "copy_output is not available when C is a sub-tensor view (the caller owns the parent tensor)");
    const size_t have = static_cast<size_t>(run->plan.sizeC) * run->elt;
    if (bytes > have) return fail(TCONTB_INVALID_ARGUMENT, "Requested more bytes than the output tensor holds");
    if (!run->shards.empty()) {
        // gather: every shard's C goes back to its slice of the global tensor
        if (bytes != have) return fail(TCONTB_INVALID_ARGUMENT, "A multi-GPU run copies the whole output tensor or nothing");
        DeviceGuard guard(run->first_device, true);
        const Plan& pl = run->plan;
        if (run->split_contracted) {
            // shard g owns the g-th contiguous range of C (cut along C's slowest mode) and holds it at the start of its C buffer
            const size_t chunk_bytes = have / run->shards.size();
            for (size_t g = 0; g < run->shards.size(); ++g) {
                TC_CUDA(cudaSetDevice(run->shard_device(g)));
                TC_CUDA(cudaMemcpy(static_cast<unsigned char*>(dst) + g * chunk_bytes, run->shards[g]->dC, chunk_bytes, cudaMemcpyDeviceToHost));
            }
            TC_CUDA(cudaSetDevice(run->first_device));
            return fail_if_device_gave_up(run);
        }
        const int64_t len = pl.ext_val[pl.ext_mode.find(run->split_mode)] / static_cast<int64_t>(run->shards.size());
        std::vector<unsigned char> part;
        for (size_t g = 0; g < run->shards.size(); ++g) {
            tcontb_run* sh = run->shards[g].get();
            part.resize(static_cast<size_t>(sh->plan.sizeC) * run->elt);
            TC_CUDA(cudaSetDevice(run->shard_device(g)));
            TC_CUDA(cudaMemcpy(part.data(), sh->dC, part.size(), cudaMemcpyDeviceToHost));
            slice_mode(static_cast<unsigned char*>(dst), part.data(), pl.modeC, pl, run->split_mode, static_cast<int64_t>(g) * len, len,
                       run->elt, true);
        }
        TC_CUDA(cudaSetDevice(run->first_device));
        return fail_if_device_gave_up(run);
    }
    TC_CUDA(cudaMemcpyAsync(dst, run->dC, bytes, cudaMemcpyDeviceToHost, run->stream));
    TC_CUDA(cudaStreamSynchronize(run->stream));
    return fail_if_device_gave_up(run);
}

tcontb_status tcontb_run_time_launches(tcontb_run* run, int iterations, float* elapsed_ms, int64_t* kernel_launches)
{
    if (!run || !elapsed_ms || iterations <= 0) return fail(TCONTB_INVALID_ARGUMENT, "Bad arguments to tcontb_run_time_launches");
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    TC_CUDA(cudaEventCreate(&e0));
    TC_CUDA(cudaEventCreate(&e1));
    tcontb_status st = TCONTB_OK;
    cudaError_t ce = cudaEventRecord(e0, run->stream);
    for (int i = 0; i < iterations && st == TCONTB_OK && ce == cudaSuccess; ++i) st = tcontb_run_launch(run);
    if (ce == cudaSuccess) ce = cudaEventRecord(e1, run->stream);
    if (ce == cudaSuccess) ce = cudaEventSynchronize(e1);
    if (ce == cudaSuccess) ce = cudaEventElapsedTime(elapsed_ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (st != TCONTB_OK) return st;
    if (ce != cudaSuccess) return fail(TCONTB_RUNTIME_ERROR, std::string("CUDA error while timing launches: ") + cudaGetErrorString(ce));
    if (kernel_launches) *kernel_launches = run->kernels_per_launch * iterations;
    return TCONTB_OK;
}

tcontb_status tcontb_run_contract_host(tcontb_run* run, const void* a_host, const void* b_host, void* c_host, int64_t* h2d,
                                       int64_t* d2h)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    if (!c_host) return fail(TCONTB_INVALID_ARGUMENT, "Destination buffer is null");
    TC_NOT_SHARDED(run, "the host-buffer pass");
    if (!a_host || !b_host) return fail(TCONTB_INVALID_ARGUMENT, "Null input buffer");
    if (run->plan.prob.strided) return fail(TCONTB_UNSUPPORTED, "the host-buffer pass is not available on sub-tensor views");
    if (!run->pipe.tried) {
        const tcontb_status bs = build_host_pipeline(run);
        if (bs != TCONTB_OK) return bs;
    }
    if (!run->pipe.parts.empty()) {
        auto& pp = run->pipe;
        const Plan& pl = run->plan;
        const size_t n = pp.parts.size();
        const unsigned char* cut_host = static_cast<const unsigned char*>(pp.in_left ? a_host : b_host);
        unsigned char* cut_dev = static_cast<unsigned char*>(pp.in_left ? run->dL : run->dR);
        // uploads start once everything queued on the run's stream so far is done with the buffers
        TC_CUDA(cudaEventRecord(pp.ev_start, run->stream));
        TC_CUDA(cudaStreamWaitEvent(pp.s_in, pp.ev_start, 0));
        TC_CUDA(cudaStreamWaitEvent(pp.s_out, pp.ev_start, 0));
        if (pp.in_left) TC_CUDA(cudaMemcpyAsync(run->dR, b_host, static_cast<size_t>(pl.sizeR) * run->elt, cudaMemcpyHostToDevice, pp.s_in));
        else TC_CUDA(cudaMemcpyAsync(run->dL, a_host, static_cast<size_t>(pl.sizeL) * run->elt, cudaMemcpyHostToDevice, pp.s_in));
        TC_CUDA(cudaEventRecord(pp.ev_other, pp.s_in));
        for (size_t i = 0; i < n; ++i) {
            if (pp.strided)
                TC_CUDA(cudaMemcpy2DAsync(cut_dev + i * pp.width, pp.pitch, cut_host + i * pp.width, pp.pitch, pp.width, pp.rows,
                                          cudaMemcpyHostToDevice, pp.s_in));
            else
                TC_CUDA(cudaMemcpyAsync(cut_dev + i * pp.slice_in, cut_host + i * pp.slice_in, pp.slice_in, cudaMemcpyHostToDevice, pp.s_in));
            TC_CUDA(cudaEventRecord(pp.ev_in[i], pp.s_in));
        }
        TC_CUDA(cudaStreamWaitEvent(run->stream, pp.ev_other, 0));
        for (size_t i = 0; i < n; ++i) {
            TC_CUDA(cudaStreamWaitEvent(run->stream, pp.ev_in[i], 0));
            if (pp.parts[i]->alpha != run->alpha || pp.parts[i]->beta != run->beta) {
                const tcontb_status ss = tcontb_run_set_scalars(pp.parts[i].get(), run->alpha, run->beta);
                if (ss != TCONTB_OK) return ss;
            }
            const tcontb_status ls = tcontb_run_launch(pp.parts[i].get());
            if (ls != TCONTB_OK) return ls;
            TC_CUDA(cudaEventRecord(pp.ev_done[i], run->stream));
            TC_CUDA(cudaStreamWaitEvent(pp.s_out, pp.ev_done[i], 0));
            TC_CUDA(cudaMemcpyAsync(static_cast<unsigned char*>(c_host) + i * pp.slice_out, static_cast<unsigned char*>(run->dC) + i * pp.slice_out,
                                    pp.slice_out, cudaMemcpyDeviceToHost, pp.s_out));
        }
        TC_CUDA(cudaStreamSynchronize(pp.s_out));
        TC_CUDA(cudaStreamSynchronize(run->stream));
        if (h2d) *h2d = (pl.sizeL + pl.sizeR) * static_cast<int64_t>(run->elt);
        if (d2h) *d2h = static_cast<int64_t>(pl.sizeC) * static_cast<int64_t>(run->elt);
        return fail_if_device_gave_up(run);
    }
    tcontb_status st = tcontb_run_upload_inputs(run, a_host, b_host);
    if (st != TCONTB_OK) return st;
    st = tcontb_run_launch(run);
    if (st != TCONTB_OK) return st;
    const size_t cb = static_cast<size_t>(run->plan.sizeC) * run->elt;
    st = tcontb_run_copy_output(run, c_host, cb);
    if (st != TCONTB_OK) return st;
    if (h2d) *h2d = (run->plan.sizeL + run->plan.sizeR) * static_cast<int64_t>(run->elt);
    if (d2h) *d2h = static_cast<int64_t>(cb);
    return TCONTB_OK;
}

tcontb_status tcontb_run_device_status(tcontb_run* run, int* status)
{
    if (!run || !status) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    if (!run->shards.empty()) {
        *status = 0;
        DeviceGuard guard(run->first_device, true);
        for (size_t g = 0; g < run->shards.size(); ++g) {
            int s1 = 0;
            TC_CUDA(cudaSetDevice(run->shard_device(g)));
            const tcontb_status st = tcontb_run_device_status(run->shards[g].get(), &s1);
            if (st != TCONTB_OK) return st;
            if (s1 > *status) *status = s1;
        }
        TC_CUDA(cudaSetDevice(run->first_device));
        return TCONTB_OK;
    }
    TC_CUDA(cudaMemcpyAsync(status, run->status.ptr, sizeof(int), cudaMemcpyDeviceToHost, run->stream));
    TC_CUDA(cudaStreamSynchronize(run->stream));
    for (auto& part : run->pipe.parts) {
        int s1 = 0;
        const tcontb_status st = tcontb_run_device_status(part.get(), &s1);
        if (st != TCONTB_OK) return st;
        if (s1 > *status) *status = s1;
    }
    return TCONTB_OK;
}

tcontb_status tcontb_run_ksplit_enable(tcontb_run* run, int world, int rank)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    TC_NOT_SHARDED(run, "tcontb_run_ksplit_enable");
    if (world < 2 || world > kMaxOwners || rank < 0 || rank >= world) return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split: need 2..8 ranks and 0 <= rank < ranks");
    if (run->ks.world) return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split is already enabled on this run");
    const Plan& pl = run->plan;
    const Problem& p = pl.prob;
    const UmmaSpec& u = pl.umma;
    if (p.strided) return fail(TCONTB_UNSUPPORTED, "contracted-mode split is not available on sub-tensor views");
    if (pl.kernel != KERNEL_UMMA_TF32 || u.k_splits != 1 || run->tf32x3)
        return fail(TCONTB_UNSUPPORTED, "contracted-mode split needs the tcgen05 kernel without split-K (Float32 operands TMA can stage; TCONT_SPLITK=1)");
    // C's slowest mode must be a column mode of the kernel (role B), the most significant digit of the column
    // slab index, and its ranges must fall on tile-column boundaries: a tile then has exactly one owner.
    if (p.C.empty() || p.N.empty() || p.C.back() != p.N.back())
        return fail(TCONTB_UNSUPPORTED, "contracted-mode split: C's slowest mode must belong to the operand that does not hold C's stride-1 mode");
    const Mode& slow = p.modes[static_cast<size_t>(p.C.back())];
    const int64_t sb = u.b.slabs_per_tile;
    const bool single = p.N.size() == 1;
    if (slow.extent % world || u.b.total_slabs % world || (u.b.total_slabs / world) % sb || u.tiles_n % world || pl.sizeC % world ||
        (single && (slow.extent / world) % u.b.slab_w))
        return fail(TCONTB_UNSUPPORTED, "contracted-mode split: the extent of C's slowest mode does not cut into whole tile columns per rank");
    auto& ks = run->ks;
    ks.chunk = pl.sizeC / world;
    if ((static_cast<size_t>(ks.chunk) * run->elt) % 16) return fail(TCONTB_UNSUPPORTED, "contracted-mode split: a rank's range of C is not a multiple of 16 bytes");
    TC_CUDA(ks.staging.alloc(static_cast<size_t>(2) * world * static_cast<size_t>(ks.chunk) * run->elt));
    ks.world = world;
    ks.rank = rank;
    ks.peer[rank] = ks.staging.ptr;
    return TCONTB_OK;
}

int64_t tcontb_run_ksplit_range_elements(const tcontb_run* run) { return run ? run->ks.chunk : 0; }

tcontb_status tcontb_run_ksplit_export(tcontb_run* run, void* handle, size_t handle_bytes)
{
    if (!run || !handle) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun or handle buffer is empty");
    if (!run->ks.world) return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split is not enabled on this run");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return fail(TCONTB_INVALID_ARGUMENT, "handle buffer is smaller than a CUDA IPC memory handle (64 bytes)");
    cudaIpcMemHandle_t h;
    TC_CUDA(cudaIpcGetMemHandle(&h, run->ks.staging.ptr));
    std::memcpy(handle, &h, sizeof(h));
    return TCONTB_OK;
}

tcontb_status tcontb_run_ksplit_import(tcontb_run* run, int peer_rank, const void* handle, size_t handle_bytes)
{
    if (!run || !handle) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun or handle is empty");
    auto& ks = run->ks;
    if (!ks.world || peer_rank < 0 || peer_rank >= ks.world || peer_rank == ks.rank) return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split: bad peer rank");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return fail(TCONTB_INVALID_ARGUMENT, "handle is smaller than a CUDA IPC memory handle (64 bytes)");
    if (ks.peer[peer_rank]) return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split: this peer is already attached");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    TC_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    ks.peer[peer_rank] = p;
    ks.opened[peer_rank] = true;
    return TCONTB_OK;
}

tcontb_status tcontb_run_ksplit_attach(tcontb_run* run, int peer_rank, tcontb_run* peer)
{
    if (!run || !peer) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    auto& ks = run->ks;
    if (!ks.world || peer_rank < 0 || peer_rank >= ks.world || peer_rank == ks.rank || peer->ks.world != ks.world || peer->ks.rank != peer_rank ||
        peer->ks.chunk != ks.chunk)
        return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split: the peer run is not rank " + std::to_string(peer_rank) + " of the same split");
    ks.peer[peer_rank] = peer->ks.staging.ptr;
    return TCONTB_OK;
}

tcontb_status tcontb_run_ksplit_reduce(tcontb_run* run)
{
    if (!run) return fail(TCONTB_INVALID_ARGUMENT, "ExecutionRun is empty");
    auto& ks = run->ks;
    if (!ks.world) return fail(TCONTB_INVALID_ARGUMENT, "contracted-mode split is not enabled on this run");
    const unsigned char* slots = static_cast<const unsigned char*>(ks.staging.ptr) +
                                 static_cast<size_t>(ks.last_set) * ks.world * static_cast<size_t>(ks.chunk) * run->elt;
    TC_CUDA(launch_splitk_reduce(slots, run->dC, ks.chunk, ks.world, ks.chunk, static_cast<int>(run->elt), run->stream, 1.0, 0.0));
    return TCONTB_OK;
}

tcontb_status tcontb_transpose(const void* src, void* dst, int rank, const int64_t* src_extent, const int* perm, int elem_bytes,
                               void* cuda_stream)
{
    if (!src || !dst || !src_extent || !perm) return fail(TCONTB_INVALID_ARGUMENT, "Null argument to tcontb_transpose");
    if (elem_bytes != 4 && elem_bytes != 8) return fail(TCONTB_INVALID_ARGUMENT, "Element size must be 4 or 8 bytes");
    const tcontb_status st = check_device();
    if (st != TCONTB_OK) return st;
    TransposeParams tp{};
    if (!make_transpose_params(rank, src_extent, perm, &tp)) return fail(TCONTB_INVALID_ARGUMENT, "Not a permutation, or a non-positive extent");
    TC_CUDA(launch_transpose(src, dst, tp, elem_bytes, static_cast<cudaStream_t>(cuda_stream)));
    return TCONTB_OK;
}

}  // extern "C"
