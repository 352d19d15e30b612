// kernels.hpp -- host-callable launchers of the sm_100a kernels (implemented in the .cu files).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "planner.hpp"

namespace tcontb {

// ---- generic SIMT contraction (simt_contract.cu) -----------------------------------------
// GEMM view with offset tables: C[offCm[m] + offCn[n]] = sum_k A[offAm[m] + offAk[k]] * B[offBn[n] + offBk[k]].
struct SimtParams {
    const void* A;
    const void* B;
    void* C;
    int64_t M, N, K;
    const int64_t* offAm;
    const int64_t* offAk;
    const int64_t* offBn;
    const int64_t* offBk;
    const int64_t* offCm;
    const int64_t* offCn;
    int a_along_k, b_along_k;  // 0: threads run along the rows, 1: along k, 2 / 3 (FP64 tensor kernel only): along the rows / along k, two at a time
};
cudaError_t launch_simt_contract(const SimtParams& p, int scalar_type, cudaStream_t stream);

// ---- FP64 tensor-core contraction (dmma_f64.cu), same GEMM view ----------------------------
cudaError_t launch_dmma_contract(const SimtParams& p, int num_sms, cudaStream_t stream);
cudaError_t dmma_configure_all();  // once per device before the first launch

// ---- tensor permutation (transpose.cu) ------------------------------------------------------
struct TransposeParams {
    int rank;                      // after merging, <= kMaxModes
    int64_t ext[kMaxModes];        // source extents
    int64_t src_stride[kMaxModes]; // element strides of source mode i in the source
    int64_t dst_stride[kMaxModes]; // element strides of source mode i in the destination
    int64_t elements;
};
// Builds merged params for dst mode i = src mode perm[i]; returns false for a bad permutation.
// `src_stride` (optional): element strides of the source modes when the source is a view into a larger tensor.
bool make_transpose_params(int rank, const int64_t* src_extent, const int* perm, TransposeParams* out, const int64_t* src_stride = nullptr);
cudaError_t launch_transpose(const void* src, void* dst, const TransposeParams& p, int elem_bytes, cudaStream_t stream);

// ---- TF32 tcgen05 contraction (umma_tf32.cu) -------------------------------------------------
constexpr int kMaxOwners = 8;  // GPUs of one box

struct UmmaOperandDev {
    int major, slab_w, slabs_per_tile, n_row_digits, slab_bytes;
    int slabs_per_op, digit0_scale, oob_coord;
    int chunk_digit;  // which row digit is the chunk of the slab mode (scaled by digit0_scale, out-of-range past the tensor)
    int k0_scale;  // TMA coordinate of k digit 0 = k iteration * this
    int row_digit_dim[kMaxTmaRank];
    int row_digit_ext[kMaxTmaRank];
    long long row_digit_cstride[kMaxTmaRank];
    long long row_elem_cstride;
    int slab_mode_ext;
    long long total_slabs;
    int k_digit_dim[3];
    int split_inner;                // operand-level row fusion: see UmmaOperand (0 = none)
    long long split_outer_cstride;
};
struct UmmaParams {
    UmmaOperandDev a, b;
    int BN, BK, stages, n_k_digits;
    int pair;  // 1: two-CTA clusters, 256 x BN tiles (cta_group::2); 0: one CTA per 128 x BN tile
    int producers;  // tcgen05 kernel: 2 = two producer warps taking turns stage by stage (needs an even number of stages)
    int k_digit_ext[3];
    int k_iters;
    // Split-K: every tile is computed k_splits times over consecutive ranges of k_iters_per_split
    // iterations; split s writes its partial tile at C + s * split_stride (a workspace laid out like
    // C, summed afterwards by launch_splitk_reduce).  k_splits = 1: the kernel writes C itself.
    int k_splits, k_iters_per_split;
    long long split_stride;
    long long tiles_m, tiles_n;
    int raster_group;
    float* C;       // tcgen05 TF32 kernel
    double* C64;    // TMA-fed FP64 kernel
    int* status;  // device status word: set non-zero when a bounded wait gives up
    long long* prof;  // optional per-CTA cycle counters [grid][8] (TCONT_UMMA_PROF=1), else null
    // Test hooks of the bounded-wait exit (tcgen05 kernel): a shorter wait limit (0 = the default 2 s), and
    // the index of one k iteration per CTA whose stage the producer leaves unfilled and unannounced
    // (-1 = none), so that the MMA warp's wait on it runs out with nothing in flight for that stage.
    unsigned long long wait_limit_ns;
    int test_skip_iter;
    // Contracted-mode split over several GPUs (tcgen05 kernel): this GPU's partial C is cut into `owners`
    // contiguous ranges along C's slowest mode, `tn_per_owner` tile columns each, and range o is stored straight
    // into the memory of the GPU that owns it, over NVLink: element i of the full C (i inside range o) goes to
    // owner_base[o][i].  owners = 0 or 1: everything goes to C.  `tn_rotate` shifts the order in which a GPU
    // visits the tile columns, so that the GPUs of a job write to different owners at any one time.
    int store_across_slabs;  // FP64 kernel: see UmmaSpec
    // tcgen05 kernel, pace keeping: the CTAs (pairs) of a launch walk their panels along k at about the same
    // pace, so that a panel one of them fetched is still in L2 when the others of its tile row or column ask for
    // it.  pace[0] counts the producers that have ended, pace[1 + g] those that have started their block g of
    // 2^pace_shift k iterations; a producer starts block g only when all have started block g - pace_lead
    // (bounded wait; after one time-out it stops looking).  Zeroed before every launch.  nullptr = off.
    unsigned int* pace;
    int pace_shift, pace_lead;
    int owners, tn_per_owner, tn_rotate;
    float* owner_base[kMaxOwners];
};
// tmapA / tmapB are 128-byte CUtensorMap objects passed by value as kernel parameters.
cudaError_t launch_umma_tf32(const UmmaParams& p, const void* tmapA, const void* tmapB, int smem_bytes, int num_sms,
                             cudaStream_t stream);
// Opt-in maximum of dynamic shared memory per block on sm_100 (227 KB); set once per function and device.
constexpr int kMaxDynamicSmemBytes = 227 * 1024;
cudaError_t umma_tf32_configure();

// ---- TMA-fed FP64 tensor-path contraction (dmma_tma_f64.cu), same parameter block ------------
cudaError_t launch_dmma_tma(const UmmaParams& p, const void* tmapA, const void* tmapB, int smem_bytes, int num_sms,
                            cudaStream_t stream);
cudaError_t dmma_tma_configure();

// ---- split-K: C[e] = sum over s of partial[s * stride + e], s ascending (splitk_reduce.cu) ----
// With alpha != 1 or beta != 0: C[e] = alpha * sum + beta * C[e] (C is read only when beta != 0).
cudaError_t launch_splitk_reduce(const void* partial, void* C, long long elements, int splits, long long stride, int elt_bytes,
                                 cudaStream_t stream, double alpha = 1.0, double beta = 0.0);

// ---- error-compensated Float32 (splitk_reduce.cu): lo = x - truncate_to_tf32(x), exact in fp32 ----
cudaError_t launch_tf32_residual(const float* x, float* lo, long long elements, cudaStream_t stream);

}  // namespace tcontb
