// planner.hpp -- host-side planning of one tensor contraction (no CUDA dependency).
//
// Stands where the reference has three pieces: the LightGBM backend selector
// (src/backend_model_selector.cpp:365-403), the Python COGENT planner
// (backends/cogent/plan/tc_plan.py:5-98 and base/*.py) and the TTGT permutation search
// (backends/ttgt_cutt/src/ttgt_cutt.cpp:220-687).  The plan is a pure function of the
// descriptor and the cost table, so it can be unit-tested without a GPU.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace tcontb {

constexpr int kMaxModes = 16;
constexpr int kMaxTmaRank = 5;

enum ModeGroup { GROUP_M = 0, GROUP_N = 1, GROUP_K = 2 };
enum KernelKind { KERNEL_SIMT = 0, KERNEL_UMMA_TF32 = 1, KERNEL_DMMA_F64 = 2, KERNEL_DMMA_F64_TMA = 3 };

struct Mode {
    std::string names;  // the caller's mode letters fused into this mode, fastest first
    int64_t extent = 1;
    int64_t sA = 0, sB = 0, sC = 0;  // element strides (0 = mode absent from that tensor)
    int group = GROUP_K;
};

// The contraction the kernels see: roles A/B may be exchanged relative to the caller's
// left/right operands so that the M group always owns C's stride-1 mode (the reference makes
// the same exchange through its swap_flag, backends/cogent/plan/tc_gen_inner_group.py:450, but
// keyed on the letter "a"; here it is keyed on position).
struct Problem {
    int scalar_type = 1;
    bool swapped = false;
    std::vector<Mode> modes;
    std::vector<int> A, B, C;  // mode ids in memory order, fastest first
    std::vector<int> M, N, K;  // M and N in C's order; K in the order the kernels iterate it
    int64_t Mtot = 1, Ntot = 1, Ktot = 1;
    int64_t sizeA = 1, sizeB = 1, sizeC = 1;  // elements of the (sub-)tensors
    int64_t spanA = 1, spanB = 1, spanC = 1;  // elements the strides cover: the same for dense tensors, the parent's for views
    bool strided = false;    // some tensor is a view into a larger parent
    bool c_strided = false;  // C is
};

// A permutation of one caller tensor: dst mode i = src mode perm[i].
struct TransposeSpec {
    bool needed = false;
    int rank = 0;
    int64_t src_extent[kMaxModes] = {0};
    int perm[kMaxModes] = {0};
    int64_t elements = 0;
    bool strided_src = false;              // the source is a view: src_stride holds its element strides
    int64_t src_stride[kMaxModes] = {0};
};

// How one operand's tile is staged into shared memory for tcgen05.mma: a tile is a run of
// "slabs", each slab one 2-D TMA box (rows x 128 bytes, 128-byte swizzle).
struct UmmaOperand {
    int rank = 0;
    int64_t ext[kMaxTmaRank] = {1, 1, 1, 1, 1};
    int64_t stride[kMaxTmaRank] = {0, 0, 0, 0, 0};  // elements
    int box[kMaxTmaRank] = {1, 1, 1, 1, 1};
    int major = 0;         // 0: K-major (stride-1 mode is the chunked K mode), 1: MN-major
    int slab_w = 32;       // rows (K-major) or contiguous elements (MN-major) of the slab mode per slab
    int slab_dim = 0;      // tensor dim the slab runs along
    int kc_dim = 0;        // tensor dim of the chunked K mode
    int slabs_per_tile = 4;
    int slabs_per_op = 1;    // consecutive slabs fetched by one TMA copy (merged boxes, MN-major only)
    int digit0_scale = 32;   // TMA coordinate of row digit 0 = chunk index * this
    int k0_scale = 32;       // TMA coordinate of k digit 0 = k iteration * this (BK; BK / 32 for a K-major operand chunked in 32s)
    int oob_coord = 0;       // coordinate (in row digit 0's dim) that lies past the tensor: zero fill
    int n_row_digits = 1;  // slab index = mixed radix number; digit `chunk_digit` = chunk of the slab mode
    int chunk_digit = 0;   // 0 normally; 1 when C's stride-1 mode leads the digits (rows of a tile run across slabs)
    int row_digit_dim[kMaxTmaRank] = {0};
    int64_t row_digit_ext[kMaxTmaRank] = {1};
    int64_t row_digit_cstride[kMaxTmaRank] = {0};  // C offset per unit of the digit
    int64_t row_elem_cstride = 1;                  // C stride of one element inside a slab
    int64_t slab_mode_ext = 1;
    int64_t total_slabs = 1;
    int k_digit_dim[3] = {-1, -1, -1};
    int slab_bytes = 0;
    // Operand-level row fusion (FP64 kernel): the slab mode is two row modes that lie one after the other in
    // the operand but not in C (a short stride-1 mode and the next one), shown to TMA as one dimension.
    // Position q of the fused mode sits at (q % split_inner) * row_elem_cstride + (q / split_inner) *
    // split_outer_cstride in C.  0 = not fused.
    int64_t split_inner = 0;
    int64_t split_outer_cstride = 0;
};

struct UmmaSpec {
    bool eligible = false;
    std::string why_not;
    std::string kc_names;  // the contracted mode that is cut into BK-sized chunks
    int BM = 128, BN = 256, BK = 32, stages = 4;
    UmmaOperand a, b;
    int n_k_digits = 1;
    int64_t k_digit_ext[3] = {1, 1, 1};  // digit 0 = chunks of the chunked K mode
    int64_t k_iters = 1, tiles_m = 1, tiles_n = 1;
    int k_splits = 1;               // ranges of the k iterations computed as separate work units (split-K)
    int64_t k_iters_per_split = 1;
    double far_fraction = 0;  // share of a stage's bytes whose K rows are 64 KB or more apart in memory
    int raster_group = 16;
    bool pair = false;  // two-CTA clusters working on 256-row tiles (tcgen05 cta_group::2)
    int producers = 1;  // tcgen05 kernel: producer warps taking turns stage by stage (2 needs an even number of stages)
    // FP64 kernel: the slabs of an A tile are consecutive indices of C's stride-1 mode (which is not A's stride-1
    // mode); a thread stores the same row of four neighbouring slabs as one 32-byte piece
    bool store_across_slabs = false;
    int smem_bytes = 0;
    int elt = 4;  // element bytes: 4 = tcgen05 TF32 kernel, 8 = TMA-fed FP64 tensor-path kernel
};

struct SimtSpec {
    int a_load_along_k = 0;  // 0: threads run along m when loading A (m contiguous), 1: along k
    int b_load_along_k = 0;
    int tile = 64;           // BM = BN
};

struct CostTable {
    // Defaults: what `python -m tcont_b200.calibrate` measured on a B200 (the file it writes,
    // tcont_cost_table.NVIDIA_B200.txt beside the library, holds the same figures and is read when the current
    // device has that name; TCONT_COST_TABLE names another "key value" file).
    double hbm_gbs = 6178.9;                // copy through the permutation kernel, read + write
    double umma_tf32_tflops = 674.4;        // tcgen05 kernel, 8192 x 8192 x 4096, CTA pairs with a k chunk of 64
    double simt_f32_tflops = 23.7;
    double simt_f64_tflops = 16.4;
    double dmma_f64_tflops = 33.5;          // TMA-fed tensor-path kernel
    double dmma_f64_gather_tflops = 20.8;   // gather tensor-path kernel, 16-byte gathers
    double dmma_f64_gather8_tflops = 15.5;  // gather tensor-path kernel, an operand on 8-byte gathers
    double dmma_f64_gather_narrow_tflops = 6.5;  // gather tensor-path kernel, 256 x 32 tiles (N <= 48)
    double scatter_store_ps = 27.6;         // per element of C stored on its own (TMA-fed FP64 kernel)
    double scatter_store_f32_ps = 17.6;     // the same for the tcgen05 kernel's 4-byte elements
    double launch_us = 6.9;                 // one more launch through the library (a contraction too small to matter, in a loop)
    // Fraction of the tcgen05 rate lost per unit of staged bytes whose K rows lie 2 MB or more apart, i.e. every row
    // of a TMA box in another 2 MB page (the calibration probe: the large 4-D configuration with f = 64, A's rows 8 MB
    // apart, half of a pair's bytes; the configuration itself: 18.7 ms where A lies against 14.1 ms through the
    // transpose that brings the rows together, i.e. 0.53; with rows 1 MB apart there is no loss: 701 / 689 TFLOP/s).
    double far_row_penalty = 0.47;
    // Least time per stage of the tcgen05 kernel's ring, whatever the stage holds: one pass of the producer's
    // wait-announce-copy sequence (700 to 900 cycles in the main-loop probes).
    double umma_stage_us = 0.45;
    // What one SM's epilogue stores per second (GB/s): a 128 x 256 fp32 tile takes 3.7 us to leave (cfg4).
    double umma_store_gbs_per_sm = 35.5;
    int num_sms = 148;  // SMs of the device the plan is made for (api.cpp fills it in from the current device)
};

struct Plan {
    // caller's descriptor, owned copies
    std::string modeC, modeA, modeB, ext_mode;
    std::vector<int64_t> ext_val;
    char op = '?';
    int scalar_type = 1;
    int backend_selection = 0;
    // Sub-tensor views: extents of each tensor's modes in the parent it is a view of (empty = dense)
    std::vector<int64_t> parentC, parentA, parentB;

    int backend = 0;        // TCONTB_BACKEND_*
    Problem prob;           // what the contraction kernel sees (after the transposes, if any)
    TransposeSpec tA, tB;   // transposes feeding role A / role B (src = the caller's tensor of that role)
    int kernel = KERNEL_SIMT;
    SimtSpec simt;
    UmmaSpec umma;
    double est_direct_us = 0, est_ttgt_us = 0;
    double flops = 0;
    int64_t sizeL = 1, sizeR = 1, sizeC = 1;  // caller's left, right, output element counts
};

// Returns 0 (ok), 1 (invalid argument), 3 (unsupported); `err` receives the message.
// parentC / parentA / parentB (optional): the tensor is a view into a larger column-major tensor whose extents, mode
// by mode, these are; strides come from them, everything else from the view's extents.
int make_plan(const char* modeC, int nC, const char* modeA, int nA, const char* modeB, int nB, char op, int scalar_type,
              const char* ext_mode, const int64_t* ext_val, int n_ext, int backend_selection, const CostTable& cost,
              Plan* plan, std::string* err, const int64_t* parentC = nullptr, const int64_t* parentA = nullptr,
              const int64_t* parentB = nullptr);

std::string describe_plan(const Plan& plan);
// Defaults, overridden by the "key value" file TCONT_COST_TABLE names, if any.
CostTable load_cost_table();
// Reads "key value" lines into `table` (unknown keys are ignored); false when the file cannot be opened.
bool read_cost_table_file(const std::string& path, CostTable* table);

// Offset tables of the GEMM view: address(A, m, k) = offAm[m] + offAk[k] and so on.
struct OffsetTables {
    std::vector<int64_t> offAm, offAk, offBn, offBk, offCm, offCn;
};
void build_offset_tables(const Problem& p, OffsetTables* t);

}  // namespace tcontb
