// tcont_shim.cpp -- `namespace TconT` (include/tcont.hpp) implemented over the C ABI.
//
// Mirrors the orchestration and the error behaviour of the reference's src/tcont.cpp:
// std::invalid_argument for empty plans/runs, null destinations and malformed descriptors
// (:91-93, :103-105, :162-164), std::runtime_error for CUDA failures (:25-31).  Nothing here
// exits the process.
#include <cuda_runtime.h>

#include <cmath>
#include <iostream>
#include <stdexcept>
#include <string>

#include "tcont.hpp"
#include "tcontb.h"

namespace TconT {
namespace {

[[noreturn]] void raise(tcontb_status st)
{
    const std::string msg = tcontb_last_error();
    if (st == TCONTB_INVALID_ARGUMENT) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

void ok(tcontb_status st)
{
    if (st != TCONTB_OK) raise(st);
}

struct PlanHandle {
    tcontb_plan* p = nullptr;
    ~PlanHandle() { tcontb_plan_destroy(p); }
};

class EngineRun final : public RunImpl {
   public:
    EngineRun(std::shared_ptr<PlanHandle> plan, Backend backend) : plan_(std::move(plan)), backend_(backend)
    {
        ok(tcontb_run_create(plan_->p, &run_));
    }
    ~EngineRun() override { tcontb_run_destroy(run_); }
    Backend backend() const override { return backend_; }
    void launch() override { ok(tcontb_run_launch(run_)); }
    bool warmup(int iterations) override
    {
        ok(tcontb_run_warmup(run_, iterations));
        return true;
    }
    void zero_output() override { ok(tcontb_run_zero_output(run_)); }
    const void* input_left_host_data() const override { return tcontb_run_host_input(run_, 0); }
    const void* input_right_host_data() const override { return tcontb_run_host_input(run_, 1); }
    void copy_output_to_host(void* destination, size_t bytes) const override
    {
        ok(tcontb_run_copy_output(run_, destination, bytes));
    }
    ExecutionStageTimes stage_times() const override
    {
        float t[6];
        ok(tcontb_run_stage_times(run_, t));
        ExecutionStageTimes s;
        s.available = t[0] != 0.0f;
        s.total_ms = t[1];
        s.transpose_a_ms = t[2];
        s.transpose_b_ms = t[3];
        s.gemm_ms = t[4];
        s.transpose_c_ms = t[5];
        return s;
    }

   private:
    std::shared_ptr<PlanHandle> plan_;  // keeps the plan alive for as long as a run exists
    Backend backend_;
    tcontb_run* run_ = nullptr;
};

class EnginePlan final : public PlanImpl {
   public:
    EnginePlan(std::shared_ptr<PlanHandle> h, Backend b) : handle_(std::move(h)), backend_(b) {}
    Backend backend() const override { return backend_; }
    std::shared_ptr<RunImpl> prepare() const override { return std::make_shared<EngineRun>(handle_, backend_); }

   private:
    std::shared_ptr<PlanHandle> handle_;
    Backend backend_;
};

void require(const ExecutionRun& run)
{
    if (!run.impl) throw std::invalid_argument("ExecutionRun is empty");
}

}  // namespace

void check_cuda(cudaError_t status, const char* expr)
{
    if (status != cudaSuccess)
        throw std::runtime_error(std::string("CUDA error in ") + expr + ": " + cudaGetErrorString(status));
}

double compute_gflops(const TCEquation& eq, float avg_ms)
{
    if (avg_ms <= 0.0f) return 0.0;
    double prod = 1.0;
    for (const std::vector<char>* modes : {&eq.modeA, &eq.modeB, &eq.modeC}) {
        for (char m : *modes) {
            const auto it = eq.extent.find(m);
            if (it == eq.extent.end()) throw std::invalid_argument(std::string("Missing extent for mode: ") + m);
            prod *= static_cast<double>(it->second);
        }
    }
    return 2.0 * std::sqrt(prod) / (static_cast<double>(avg_ms) * 1.0e6);
}

ExecutionPlan plan(const TCEquation& desc)
{
    std::string ext_mode;
    std::vector<int64_t> ext_val;
    for (const auto& kv : desc.extent) {
        ext_mode.push_back(kv.first);
        ext_val.push_back(kv.second);
    }
    tcontb_desc d{};
    d.nC = static_cast<int>(desc.modeC.size());
    d.nA = static_cast<int>(desc.modeA.size());
    d.nB = static_cast<int>(desc.modeB.size());
    d.modeC = desc.modeC.data();
    d.modeA = desc.modeA.data();
    d.modeB = desc.modeB.data();
    d.op = desc.op;
    d.scalar_type = desc.scalar_type == ScalarType::Float64 ? TCONTB_F64 : TCONTB_F32;
    d.n_ext = static_cast<int>(ext_mode.size());
    d.ext_mode = ext_mode.data();
    d.ext_val = ext_val.data();
    d.backend_selection = desc.backend_selection == BackendSelection::MODEL    ? TCONTB_SELECT_MODEL
                          : desc.backend_selection == BackendSelection::COGENT ? TCONTB_SELECT_DIRECT
                                                                               : TCONTB_SELECT_TTGT;
    auto handle = std::make_shared<PlanHandle>();
    ok(tcontb_plan_create(&d, &handle->p));
    const Backend backend = tcontb_plan_backend(handle->p) == TCONTB_BACKEND_TTGT ? Backend::TTGT_CUTT : Backend::COGENT;
    std::cout << (backend == Backend::COGENT ? "[TconT] Cogent selected" : "[TconT] TTGT selected") << std::endl;

    ExecutionPlan out;
    out.backend = backend;
    out.equation = desc;
    out.impl = std::make_shared<EnginePlan>(handle, backend);
    return out;
}

ExecutionRun prepare(const ExecutionPlan& plan)
{
    if (!plan.impl) throw std::invalid_argument("ExecutionPlan is empty");
    ExecutionRun run;
    run.backend = plan.backend;
    run.equation = plan.equation;
    run.impl = plan.impl->prepare();
    return run;
}

void launch(const ExecutionRun& run)
{
    require(run);
    run.impl->launch();
}

void warmup(const ExecutionRun& run, int iterations)
{
    require(run);
    if (iterations <= 0) return;
    if (run.impl->warmup(iterations)) return;
    for (int i = 0; i < iterations; ++i) run.impl->launch();
    check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize(warmup)");
}

void zero_output(const ExecutionRun& run)
{
    require(run);
    run.impl->zero_output();
}

ExecutionStageTimes stage_times(const ExecutionRun& run)
{
    require(run);
    return run.impl->stage_times();
}

const void* input_left_host_data(const ExecutionRun& run)
{
    require(run);
    return run.impl->input_left_host_data();
}

const void* input_right_host_data(const ExecutionRun& run)
{
    require(run);
    return run.impl->input_right_host_data();
}

void copy_output_to_host(const ExecutionRun& run, void* destination, size_t bytes)
{
    require(run);
    if (destination == nullptr) throw std::invalid_argument("Destination buffer is null");
    run.impl->copy_output_to_host(destination, bytes);
}

}  // namespace TconT
