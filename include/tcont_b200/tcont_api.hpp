// tcont_api.hpp -- the C++ surface `namespace TconT` of the B200 contraction engine.
//
// Source- and ABI-compatible with the reference's include/tcont.hpp (types at :12-135, free
// functions at :138-148): same names, same member order, same mangled symbols, so the reference's
// own harness (benchmarks/tccg/bench_tccg.cpp) links against libtcont.so of this repository
// without a change.  Behind it sits the C ABI of include/tcontb.h; every function below says
// which C entry point it forwards to.
//
// Semantics (identical to what the reference's two GPU backends actually do): C = A * B,
// alpha = 1, beta = 0; TCEquation::op is carried but not applied.  Tensors are column-major:
// the first mode of each list is the fastest one.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace TconT {

// ---- scalar types -------------------------------------------------------------------------
enum class ScalarType { Float32, Float64 };  // Float32 = fp32 storage, TF32 multiply, fp32 accumulate

constexpr size_t scalar_type_size(ScalarType t)
{
    return t == ScalarType::Float32 ? 4 : t == ScalarType::Float64 ? 8 : 0;
}

constexpr const char* scalar_type_name(ScalarType t)
{
    return t == ScalarType::Float32 ? "FLOAT" : t == ScalarType::Float64 ? "DOUBLE" : "unknown";
}

// ---- backends -----------------------------------------------------------------------------
// The two names are the reference's; here COGENT means "direct contraction kernel" and
// TTGT_CUTT means "transpose the inputs, then the direct kernel" (no cuTT, no cuBLAS).
enum class Backend { COGENT, TTGT_CUTT };
enum class BackendSelection { MODEL, COGENT, TTGT_CUTT };  // MODEL = let the planner's cost table decide

constexpr const char* backend_name(Backend b)
{
    return b == Backend::COGENT ? "cogent" : b == Backend::TTGT_CUTT ? "ttgt" : "unknown";
}

constexpr const char* backend_selection_name(BackendSelection s)
{
    return s == BackendSelection::MODEL    ? "model"
           : s == BackendSelection::COGENT ? "cogent"
           : s == BackendSelection::TTGT_CUTT ? "ttgt"
                                              : "unknown";
}

// ---- the contraction descriptor -------------------------------------------------------------
struct TCEquation {
    std::vector<char> modeC;  // output modes, fastest first
    std::vector<char> modeA;  // left input
    std::vector<char> modeB;  // right input
    char op = '?';            // '+', '-': printed by callers, not applied (C is overwritten)
    ScalarType scalar_type = ScalarType::Float64;

    std::unordered_map<char, int64_t> extent;  // one entry per mode name
    BackendSelection backend_selection = BackendSelection::MODEL;
};

struct ContractionResult {
    float avg_ms;
    double gflops;
    bool coorect;  // (sic) spelled as in the reference so aggregate initialisers keep compiling
};

struct RunOptions {
    int warmup = 3;
    int repeats = 10;
};

// Per-stage device times of the most recent launch; filled only when the environment has
// TCONT_STAGE_TIMES=1.  transpose_c_ms is always 0: C is written in place in its final order.
struct ExecutionStageTimes {
    bool available = false;
    float total_ms = 0.0f;
    float transpose_a_ms = 0.0f;
    float transpose_b_ms = 0.0f;
    float gemm_ms = 0.0f;
    float transpose_c_ms = 0.0f;
};

// ---- implementation interfaces (kept so that code holding these pointers keeps compiling) --
struct RunImpl;

struct PlanImpl {
    virtual ~PlanImpl() = default;
    virtual Backend backend() const = 0;
    virtual std::shared_ptr<RunImpl> prepare() const = 0;
};

struct RunImpl {
    virtual ~RunImpl() = default;
    virtual Backend backend() const = 0;
    virtual void launch() = 0;
    virtual bool warmup(int iterations)
    {
        (void)iterations;
        return false;
    }
    virtual void zero_output() {}
    virtual const void* input_left_host_data() const = 0;
    virtual const void* input_right_host_data() const = 0;
    virtual void copy_output_to_host(void* destination, size_t bytes) const = 0;
    virtual ExecutionStageTimes stage_times() const { return {}; }
};

struct ExecutionPlan {
    Backend backend = Backend::COGENT;
    TCEquation equation;
    std::shared_ptr<PlanImpl> impl;
};

struct ExecutionRun {
    Backend backend = Backend::COGENT;
    TCEquation equation;
    std::shared_ptr<RunImpl> impl;
};

// ---- free functions ---------------------------------------------------------------------------
// Throws std::runtime_error("CUDA error in <expr>: <text>") unless status is cudaSuccess.
void check_cuda(cudaError_t status, const char* expr);
// 2*sqrt(|A||B||C|) / (avg_ms * 1e6); 0 when avg_ms <= 0; std::invalid_argument for a missing extent.
double compute_gflops(const TCEquation& equation, float avg_ms);

// tcontb_plan_create. std::invalid_argument for a malformed descriptor (missing extent, ...),
// std::runtime_error for one the engine cannot express (batch modes).  Prints the same
// "[TconT] Cogent selected" / "[TconT] TTGT selected" line as the reference.
ExecutionPlan plan(const TCEquation& desc);
// tcontb_run_create: allocates device tensors, generates and uploads inputs.
ExecutionRun prepare(const ExecutionPlan& plan);
// tcontb_run_launch (asynchronous, legacy NULL stream).
void launch(const ExecutionRun& run);
// tcontb_run_warmup: `iterations` launches, then cudaDeviceSynchronize.
void warmup(const ExecutionRun& run, int iterations);
// tcontb_run_zero_output.
void zero_output(const ExecutionRun& run);
// tcontb_run_stage_times.
ExecutionStageTimes stage_times(const ExecutionRun& run);
// tcontb_run_host_input: the inputs the run generated, |A| / |B| elements of the scalar type.
const void* input_left_host_data(const ExecutionRun& run);
const void* input_right_host_data(const ExecutionRun& run);
// tcontb_run_copy_output (blocking).
void copy_output_to_host(const ExecutionRun& run, void* destination, size_t bytes);

}  // namespace TconT
