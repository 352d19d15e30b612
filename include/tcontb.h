/*
 * tcontb.h -- C ABI of the B200 tensor-contraction engine (libtcontb.so).
 *
 * One binary contraction  C[modeC] = sum_K A[modeA] * B[modeB]  on column-major tensors (first
 * mode fastest), FP64 or "Float32 = TF32 multiply, FP32 accumulate", executed by hand-written
 * sm_100a kernels.  The semantics are the reference's effective ones: alpha = 1, beta = 0, the
 * descriptor's sign character is carried but ignored, so every launch overwrites C
 * (reference: backends/ttgt_cutt/src/ttgt_cutt.cpp:742-743, benchmarks/tccg/tccg_verify.cpp:35-37).
 *
 * Each entry point names the piece of the reference's C++ surface (include/tcont.hpp,
 * src/tcont.cpp) it stands behind; include/tcont.hpp of this repository re-creates that C++
 * surface on top of these functions.  There is no CPU fallback: every compute entry point fails
 * with TCONTB_RUNTIME_ERROR when no CUDA device is usable.
 *
 * Threading: plans and runs are independent objects; a run must be used by one thread at a
 * time.  All device work of a run is issued to the run's stream, by default the legacy NULL
 * stream of the device that was current at tcontb_run_create (the reference launches
 * everything on the NULL stream, benchmarks/tccg/bench_tccg.cpp:132-136).
 */
#ifndef TCONTB_H
#define TCONTB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    TCONTB_OK = 0,
    TCONTB_INVALID_ARGUMENT = 1, /* maps to std::invalid_argument in the C++ surface */
    TCONTB_RUNTIME_ERROR = 2,    /* maps to std::runtime_error (CUDA failures, no device) */
    TCONTB_UNSUPPORTED = 3       /* a descriptor the engine cannot express (batch modes ...) */
} tcontb_status;

enum { TCONTB_F32 = 0, TCONTB_F64 = 1 };                 /* TconT::ScalarType, tcont.hpp:12-15 */
enum { TCONTB_SELECT_MODEL = 0, TCONTB_SELECT_DIRECT = 1, TCONTB_SELECT_TTGT = 2 }; /* BackendSelection, tcont.hpp:44-48 */
enum { TCONTB_BACKEND_DIRECT = 0, TCONTB_BACKEND_TTGT = 1 };  /* Backend {COGENT, TTGT_CUTT}, tcont.hpp:39-42 */

/* Plain-C image of TconT::TCEquation (tcont.hpp:74-83). Mode names are single characters;
 * ext_mode[i] has extent ext_val[i]. */
typedef struct tcontb_desc {
    int nC, nA, nB;
    const char* modeC;
    const char* modeA;
    const char* modeB;
    char op;              /* '+', '-', ... : carried, ignored (see above) */
    int scalar_type;      /* TCONTB_F32 | TCONTB_F64 */
    int n_ext;
    const char* ext_mode;
    const int64_t* ext_val;
    int backend_selection; /* TCONTB_SELECT_* */
} tcontb_desc;

typedef struct tcontb_plan tcontb_plan; /* behind TconT::ExecutionPlan / PlanImpl, tcont.hpp:105-131 */
typedef struct tcontb_run tcontb_run;   /* behind TconT::ExecutionRun / RunImpl, tcont.hpp:111-135 */

/* Last error text of the calling thread ("" when none). */
const char* tcontb_last_error(void);

/* ---- planning (host only, needs no GPU) ------------------------------------------------- */

/* TconT::plan (src/tcont.cpp:58-88): validates the descriptor, classifies modes into the
 * GEMM-like M/N/K groups, fuses adjacent modes, picks backend, kernel family and tile shape.
 * Replaces the reference's LightGBM selector, Python planner and NVRTC step; nothing is
 * compiled at run time. */
tcontb_status tcontb_plan_create(const tcontb_desc* desc, tcontb_plan** out);
/* Beyond the reference, whose descriptor has no strides (backends/cogent/plan/base/index_mapping.py:211 takes
 * dense column-major tensors): each tensor may be a sub-tensor VIEW of a larger column-major tensor.  parent_x[i] is the
 * extent of mode i of tensor x in its parent (at least the view's extent; NULL = that tensor is dense).  Strides come from
 * the parents, everything else from the view's extents; modes fuse only where the view leaves no gap between them.  A
 * plan over views runs on caller-owned device buffers (tcontb_run_create_on_device), with the pointers at the views'
 * first elements, 16-byte aligned; split-K, alpha/beta, the compensated Float32 mode, zero_output and copy_output are not
 * available when C is a view. */
tcontb_status tcontb_plan_create_strided(const tcontb_desc* desc, const int64_t* parent_c, const int64_t* parent_a,
                                         const int64_t* parent_b, tcontb_plan** out);
void tcontb_plan_destroy(tcontb_plan* plan);
/* ExecutionPlan::backend (tcont.hpp:126): TCONTB_BACKEND_DIRECT prints as "cogent",
 * TCONTB_BACKEND_TTGT as "ttgt". */
int tcontb_plan_backend(const tcontb_plan* plan);
/* Planner decisions as one JSON object (groups, fusion, kernel, tiles); for tests and logs. */
tcontb_status tcontb_plan_describe(const tcontb_plan* plan, char* buf, size_t buf_bytes);
/* 2*sqrt(|A||B||C|), the reference's operation count (src/tcont.cpp:51-55). */
double tcontb_plan_flops(const tcontb_plan* plan);

/* ---- runs (device) ---------------------------------------------------------------------- */

/* TconT::prepare (src/tcont.cpp:90-100): allocates A, B, C (and transpose scratch) on the
 * current device, generates host inputs and uploads them.  The reference fills inputs with
 * rand() in [0,1] seeded by time (backends/cogent/src/cogent.cpp:284-288); here the stream is
 * tcontb_fill_uniform with seed TCONT_SEED (default: time based) and range TCONT_INPUT_RANGE
 * "lo:hi" (default 0:1). */
tcontb_status tcontb_run_create(const tcontb_plan* plan, tcontb_run** out);
/* Same, but with caller-provided host inputs (|A| and |B| elements of the scalar type), which
 * the run copies and keeps. */
tcontb_status tcontb_run_create_with_inputs(const tcontb_plan* plan, const void* a_host, const void* b_host,
                                            tcontb_run** out);
/* Same, but on caller-owned DEVICE buffers (no host copies are kept, tcontb_run_host_input
 * returns NULL): the form a caller uses whose tensors already live in HBM. */
tcontb_status tcontb_run_create_on_device(const tcontb_plan* plan, const void* a_dev, const void* b_dev, void* c_dev,
                                          tcontb_run** out);
void tcontb_run_destroy(tcontb_run* run);

/* Stream all later work of the run is issued to (a cudaStream_t; NULL = legacy NULL stream). */
tcontb_status tcontb_run_set_stream(tcontb_run* run, void* cuda_stream);
/* Replaces the run's inputs by an asynchronous host-to-device copy on the run's stream. */
tcontb_status tcontb_run_upload_inputs(tcontb_run* run, const void* a_host, const void* b_host);

/* Beyond the reference, whose backends always overwrite (alpha = 1, beta = 0: cublasGemmEx scalars at
 * backends/ttgt_cutt/src/ttgt_cutt.cpp:742-743, generated kernels store a zeroed accumulator): later
 * launches compute C = alpha * (A*B) + beta * C.  With other values than (1, 0) the contraction
 * writes a workspace of the size of C (allocated by this call, not by the launches) and the
 * partial-sum pass applies the scalars; C is read only when beta is not zero.  Not available on a
 * run that spans several GPUs. */
tcontb_status tcontb_run_set_scalars(tcontb_run* run, double alpha, double beta);

/* TconT::launch (src/tcont.cpp:102-108): one contraction, asynchronous. */
tcontb_status tcontb_run_launch(tcontb_run* run);
/* TconT::warmup (src/tcont.cpp:110-124): `iterations` launches, then a device synchronize. */
tcontb_status tcontb_run_warmup(tcontb_run* run, int iterations);
/* TconT::zero_output (src/tcont.cpp:126-132): memset of C on the run's stream. */
tcontb_status tcontb_run_zero_output(tcontb_run* run);
/* TconT::stage_times (tcont.hpp:96-103): out = {available, total, transpose_a, transpose_b,
 * contraction, transpose_c} in ms for the most recent launch; measured only when the
 * environment has TCONT_STAGE_TIMES=1 (otherwise available = 0). */
tcontb_status tcontb_run_stage_times(tcontb_run* run, float out[6]);
/* TconT::input_left_host_data / input_right_host_data (tcont.hpp:144-145): which = 0 (A), 1 (B). */
const void* tcontb_run_host_input(const tcontb_run* run, int which);
/* TconT::copy_output_to_host (src/tcont.cpp:158-167): blocking device-to-host copy of C. */
tcontb_status tcontb_run_copy_output(tcontb_run* run, void* dst, size_t bytes);

/* `iterations` launches bracketed by CUDA events on the run's stream; returns the elapsed
 * milliseconds (the reference harness's timing loop, benchmarks/tccg/bench_tccg.cpp:125-138).
 * If kernel_launches is not NULL it receives the number of kernels the engine launched. */
tcontb_status tcontb_run_time_launches(tcontb_run* run, int iterations, float* elapsed_ms, int64_t* kernel_launches);
/* One pass through the caller-facing path with HOST buffers: upload A and B, launch, download
 * C, synchronize.  Bytes moved are reported. */
tcontb_status tcontb_run_contract_host(tcontb_run* run, const void* a_host, const void* b_host, void* c_host,
                                       int64_t* h2d_bytes, int64_t* d2h_bytes);

/* Device status word of the most recent launch: 0, or a non-zero code when a bounded wait
 * inside a kernel gave up (the kernel then returns instead of hanging). */
tcontb_status tcontb_run_device_status(tcontb_run* run, int* status);

/* ---- contracted-mode split over the GPUs of one box ------------------------------------------
 *
 * No counterpart in the reference, which has no multi-GPU code.  The sharding that needs no exchange cuts an
 * external mode (TCONT_NUM_GPUS / TCONT_SPLIT=ext:<mode>, or one run per process on a descriptor with the
 * smaller extent).  Cutting a CONTRACTED mode instead gives every GPU a partial sum of the whole C; here the
 * partial C never exists as a whole: C is cut into `ranks` contiguous ranges along its slowest mode, range o
 * belongs to rank o, and the contraction kernel of rank r stores every finished tile of range o straight
 * into rank o's memory (its own, or the peer's over NVLink: plain peer stores, no collective library, no
 * remote loads).  After a barrier among the ranks each owner adds up its `ranks` slots.
 *
 * Per rank: create the run on the descriptor with the contracted extent divided by `ranks` (its slice of A
 * and B); the run's C buffer receives only this rank's range (|C| / ranks elements).  Then
 *   tcontb_run_ksplit_enable(run, ranks, rank)            allocates the staging area (2 * |C| elements)
 *   tcontb_run_ksplit_export / _import                    one process per GPU: CUDA IPC handle of the staging
 *                                                         area, sent to every other rank by the caller's own means
 *   tcontb_run_ksplit_attach(run, peer_rank, peer_run)    the same between runs of one process
 *   per step:  tcontb_run_launch(run);  <barrier among the ranks, ordered on the run's stream>;
 *              tcontb_run_ksplit_reduce(run)
 * Two sets of slots alternate between launches, so one barrier per step is enough.  Needs the tcgen05
 * kernel without split-K, C's slowest mode in the operand that does not hold C's stride-1 mode, and an extent
 * of that mode that cuts into whole tile columns per rank; otherwise TCONTB_UNSUPPORTED.
 * Within one process TCONT_NUM_GPUS=<n> with TCONT_SPLIT=k:<mode> does all of this behind one run object. */
tcontb_status tcontb_run_ksplit_enable(tcontb_run* run, int ranks, int rank);
tcontb_status tcontb_run_ksplit_export(tcontb_run* run, void* handle, size_t handle_bytes);   /* 64 bytes */
tcontb_status tcontb_run_ksplit_import(tcontb_run* run, int peer_rank, const void* handle, size_t handle_bytes);
tcontb_status tcontb_run_ksplit_attach(tcontb_run* run, int peer_rank, tcontb_run* peer_run);
tcontb_status tcontb_run_ksplit_reduce(tcontb_run* run);
int64_t tcontb_run_ksplit_range_elements(const tcontb_run* run);

/* ---- utilities ---------------------------------------------------------------------------- */

/* Counter-based uniform fill (host): element i = lo + (hi-lo)*u_i, u_i = top 53 bits of
 * splitmix64(seed*0x9E3779B97F4A7C15 + offset + i) * 2^-53, rounded to float for TCONTB_F32.
 * A uses offset 0, B uses offset |A|.  Stands in for the reference's rand() fill
 * (backends/cogent/helper/tcl_helper.h:14-29) so that tests can regenerate identical inputs. */
tcontb_status tcontb_fill_uniform(void* dst, int scalar_type, int64_t n, uint64_t seed, uint64_t offset, double lo,
                                  double hi);

/* Stand-alone tensor permutation on the device (the engine's replacement for the cuTT calls of
 * backends/ttgt_cutt/src/ttgt_cutt.cpp:732-760): dst mode i = src mode perm[i]; column-major;
 * elem_bytes 4 or 8; pointers are device pointers; asynchronous on `cuda_stream`. */
tcontb_status tcontb_transpose(const void* src_dev, void* dst_dev, int rank, const int64_t* src_extent, const int* perm,
                               int elem_bytes, void* cuda_stream);

/* Arithmetic-peak microbenchmarks on the current device, for roofline denominators (no
 * counterpart in the reference): which = 0 TF32 tensor cores (tcgen05.mma kind::tf32 128x256x8
 * issued back to back on resident operands), 1 = FP64 DFMA, 2 = FP64 mma.sync m8n8k4.
 * Result in TFLOP/s, all SMs busy at once. */
tcontb_status tcontb_measure_peak(int which, double* tflops);
const char* tcontb_peak_last_error(void);

/* ---- allocation-free contraction ------------------------------------------------------------
 *
 * No counterpart in the reference.  For callers that must not trigger a device allocation: a
 * process whose own memory pool has claimed the whole GPU, or a latency-critical loop that cannot
 * take the device-wide synchronisation of cudaMalloc.  One contraction C = A*B on the caller's
 * DEVICE buffers, asynchronous on `cuda_stream`, computed by the CUDA-core kernel (FP64, or plain
 * FP32 arithmetic for TCONTB_F32 -- not the TF32 tensor-core path).  It calls no cudaMalloc /
 * cudaFree and no allocating library routine: the kernel's scratch (its offset tables) lives in
 * a 4 MiB array built into the library, resident on every GPU that loads the library until the
 * process exits.
 *
 *  - Limit: 2*(M+N+K) <= 524288, with M, N, K the products of the external-left, external-right
 *    and contracted extents; larger contractions return TCONTB_UNSUPPORTED with a message that
 *    states the need and the limit.  d->backend_selection is ignored (always the direct route).
 *  - The first call on each device resolves the array's device address (cudaGetSymbolAddress);
 *    make that first call outside any stream capture.
 *  - All calls share the one array and it keeps the previous call's contents; every call
 *    overwrites the part it uses before its kernel reads it.  Calls whose GPU work can overlap
 *    (different streams, concurrent host threads) race on it: keep them on one stream or
 *    serialise them yourself.
 *  - Errors of this entry point are reported by tcontb_no_alloc_last_error().
 */
tcontb_status tcontb_contract_no_alloc(const tcontb_desc* desc, const void* a_dev, const void* b_dev, void* c_dev,
                                       void* cuda_stream);
const char* tcontb_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* TCONTB_H */
