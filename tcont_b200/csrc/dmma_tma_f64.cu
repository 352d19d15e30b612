// dmma_tma_f64.cu -- FP64 direct contraction: TMA-staged operand tiles feeding mma.sync m8n8k4.
//
// tcgen05 has no FP64 kind, so the arithmetic is warp-level DMMA (37.0 TFLOP/s measured on B200).
// What the gather kernel (dmma_f64.cu) spends on address arithmetic is done here by the copy
// engine: the planner's slab machinery, the same as for the tcgen05 kernel but with 16 doubles per
// 128-byte row, describes every operand tile as a few multi-mode TMA boxes.
//
// One block per SM, three warpgroups; setmaxnreg moves the register budget from the first (56 per
// thread) to the other two (224):
//   warps 0, 1  producers, one per consumer group: lane i issues copy i of a stage (5-D tensor
//               maps, 128-byte swizzle, no multicast) into the group's own ring of stages,
//               full/empty mbarriers per stage, the ring runs across tile boundaries
//   warps 2, 3  table builders: for every tile, ahead of time, the C offset of each of its 128 rows
//               and 64 columns (mixed-radix slab arithmetic, the same as the tcgen05 epilogue),
//               double-buffered per group behind mbarriers
//   warps 4-7   consumer group 0, warps 8-11 consumer group 1.  A group is 2 x 2 warps with a
//               64 x 32 warp tile (8 x 4 accumulator fragments; 64 x 16 in the 128 x 32 variant for
//               narrow N) and takes every other tile of the block.  Group 1 starts half a main loop late, so one group's stores fall into the
//               other's main loop instead of both storing with the FP64 pipe idle.
// Fragment rows are permuted so that one 16-byte shared load of an MN-major operand feeds two
// fragments (rows 2 r and 2 r + 1 of a 16-row slab) without bank conflicts, and the MMA is issued
// transposed (B fragment as the row operand): a thread then owns four consecutive elements of C's
// stride-1 mode per fragment pair and a warp store instruction writes eight whole 128-byte lines.
// The loads of the next k step are issued between the MMAs of the current one.
// Every wait is bounded and raises the run's status word instead of hanging.
//
// Stands where the reference runs its generated FP64 WMMA kernels
// (backends/cogent/plan/generators/kernels/kernel_compute.py:127-850) and its cublasGemmEx FP64
// call (backends/ttgt_cutt/src/ttgt_cutt.cpp:764-809).
#include <cuda.h>

#include "kernels.hpp"
#include "tile_common.cuh"

namespace tcontb {
namespace {

constexpr int kThreads64 = 384;
constexpr int kBM = 128, kMaxBN = 64;
constexpr uint32_t kTabBytes = (kBM + kMaxBN) * 8u;  // one tile's row and column offsets

__device__ __forceinline__ double ld_shared_f64(uint32_t addr)
{
    double v;
    asm volatile("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void ld_shared_v2f64(uint32_t addr, double& x, double& y)
{
    asm volatile("ld.shared.v2.f64 {%0, %1}, [%2];" : "=d"(x), "=d"(y) : "r"(addr));
}

__device__ __forceinline__ void dmma_m8n8k4(double (&c)[2], double a, double b)
{
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                 : "+d"(c[0]), "+d"(c[1])
                 : "d"(a), "d"(b));
}

__device__ __forceinline__ void st_global_cs_v4f64(double* p, double a, double b, double c, double d)
{
    asm volatile("st.global.cs.v4.f64 [%0], {%1, %2, %3, %4};" ::"l"(p), "d"(a), "d"(b), "d"(c), "d"(d) : "memory");
}

// Which k a lane feeds into step t of a stage: k = 8 (t / 2) + 2 fk + ((fk ^ (fk >> 1) ^ t) & 1), fk = lane % 4.
// Any assignment works as long as both operands use the same one.  With this one
//  * the four rows an MN-major 16-byte load touches per quarter warp differ in k / 2, which after the
//    XOR swizzle puts the quarter's eight 16-byte chunks into eight different bank groups;
//  * the two lanes of a half warp that meet in the same 16-byte chunk of a K-major operand (rows
//    2 fr + par with fr two apart in the swizzle) take different halves of it.
__device__ __forceinline__ uint32_t step_k(uint32_t t, uint32_t fk) { return 8u * (t >> 1) + 2u * fk + ((fk ^ (fk >> 1) ^ t) & 1u); }

// Where a thread finds its fragments of one operand for one k:
//   MN-major (rows of the stage are k, 16 consecutive m per 128-byte row, slabs of 16 m one slab apart;
//   or 8 m per 64-byte row, two slabs per 16 m):
//     one 16-byte load at  q0 + pair * pitch  holds fragments 2 pair and 2 pair + 1
//   K-major (rows of the stage are m, BK consecutive k per row: 128 bytes, or 64 with a k chunk of 8):
//     fragment i at  (i odd ? q1 : q0) + (i / 2) * pitch,  pitch = 16 rows
// The 16-byte chunk index inside a row is XORed with (row % 8) (128-byte rows, 128-byte swizzle) or
// with (row / 2) % 4 (64-byte rows, 64-byte swizzle).
struct FragAddr {
    uint32_t q0, q1;
};

// `rows64`: K-major rows of 64 bytes (k chunk of 8); `slabs8`: MN-major rows of 64 bytes (slabs of 8)
template <bool MN>
__device__ __forceinline__ FragAddr frag_addr(uint32_t thread_base, uint32_t k, uint32_t fr, bool rows64, bool slabs8)
{
    FragAddr f;
    if (MN) {
        // (with slabs of 8 the thread's slab, fr / 4, is already part of thread_base)
        f.q0 = slabs8 ? thread_base + k * 64u + (((fr & 3u) ^ ((k >> 1) & 3u)) << 4) : thread_base + k * 128u + ((fr ^ (k & 7u)) << 4);
        f.q1 = 0;
    } else {
        const uint32_t kk = (k & 1u) * 8u, kc = k >> 1;
        if (rows64) {
            f.q0 = thread_base + kk + ((kc ^ (fr & 3u)) << 4);  // rows 2 fr and 2 fr + 1 share (row / 2) % 4
            f.q1 = f.q0 + 64u;
        } else {
            f.q0 = thread_base + kk + ((kc ^ ((2u * fr) & 7u)) << 4);
            f.q1 = thread_base + 128u + kk + ((kc ^ ((2u * fr + 1u) & 7u)) << 4);
        }
    }
    return f;
}

// load `n` fragments (n = 8 for A, 4 for B), all at once
template <bool MN, int N>
__device__ __forceinline__ void load_all(double (&f)[N], const FragAddr& q, uint32_t pitch)
{
#pragma unroll
    for (int i = 0; i < N; ++i) {
        if (MN) {
            if ((i & 1) == 0) ld_shared_v2f64(q.q0 + static_cast<uint32_t>(i >> 1) * pitch, f[i], f[i + 1]);
        } else {
            f[i] = ld_shared_f64(((i & 1) ? q.q1 : q.q0) + static_cast<uint32_t>(i >> 1) * pitch);
        }
    }
}

// One k4 step of a warp: 8 NF MMAs on the current fragments (NF = 4 or 2 column fragments); with PF the fragment loads of the next
// step are issued between them, where the FP64 tensor pipe leaves issue slots free.
// acc[i][j][h]: row m = 16 (i / 2) + 4 (lane % 4) + 2 h + (i % 2), column n = 16 (j / 2) + 2 (lane / 4) + (j % 2).
template <bool PF, bool AMN, bool BMN, int NF>
__device__ __forceinline__ void mma_step(double (&acc)[8][NF][2], const double (&ac)[8], const double (&bc)[NF], double (&an)[8],
                                         double (&bn)[NF], const FragAddr& qa, const FragAddr& qb, uint32_t a_pitch, uint32_t b_pitch)
{
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int j = 0; j < NF; ++j) dmma_m8n8k4(acc[i][j], bc[j], ac[i]);
        if (PF) {
            if (AMN) {
                if ((i & 1) == 0) ld_shared_v2f64(qa.q0 + static_cast<uint32_t>(i >> 1) * a_pitch, an[i], an[i + 1]);
            } else {
                an[i] = ld_shared_f64(((i & 1) ? qa.q1 : qa.q0) + static_cast<uint32_t>(i >> 1) * a_pitch);
            }
            if (BMN) {
                if ((i == 1 || i == 3) && i < NF) ld_shared_v2f64(qb.q0 + static_cast<uint32_t>(i >> 1) * b_pitch, bn[i - 1], bn[i]);
            } else {
                if (i < NF) bn[i] = ld_shared_f64(((i & 1) ? qb.q1 : qb.q0) + static_cast<uint32_t>(i >> 1) * b_pitch);
            }
        }
    }
}

template <bool AMN, bool BMN, int NF>
__global__ void __launch_bounds__(kThreads64, 1)
dmma_tma_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                const __grid_constant__ UmmaParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // 1024-byte aligned
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int SA = p.a.slabs_per_tile, SB = p.b.slabs_per_tile;
    const uint32_t a_tile_bytes = static_cast<uint32_t>(SA * p.a.slab_bytes);
    const uint32_t stage_bytes = a_tile_bytes + static_cast<uint32_t>(SB * p.b.slab_bytes);

    uint8_t* aux = smem + static_cast<size_t>(p.stages) * stage_bytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(aux);  // [8]
    uint64_t* bar_empty = bar_full + 8;                     // [8]
    const uint32_t abort_flag = smem_u32(bar_empty + 8);
    uint64_t* tab_full = bar_empty + 10;   // [group][buffer]
    uint64_t* tab_empty = tab_full + 4;    // [group][buffer]
    const uint32_t tabs = smem_u32(aux + 256);  // [group][buffer]: long long [128] row offsets, [64] column offsets (-1 = beyond C)

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bar_full + s), 1);
            mbar_init(smem_u32(bar_empty + s), 4);  // one arrival per consumer warp
        }
        for (int s = 0; s < 4; ++s) {
            mbar_init(smem_u32(tab_full + s), 64);  // every builder thread
            mbar_init(smem_u32(tab_empty + s), 4);  // one arrival per consumer warp
        }
        st_shared_u32(abort_flag, 0u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const uint32_t tiles_m = static_cast<uint32_t>(p.tiles_m), tiles_n = static_cast<uint32_t>(p.tiles_n);
    const uint32_t total_tiles = tiles_m * tiles_n * static_cast<uint32_t>(p.k_splits);  // work units (tile, k range)
    const uint32_t my_tiles = blockIdx.x < total_tiles ? (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t ring = static_cast<uint32_t>(p.stages) / 2u;  // stages per group

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp < 2) {
            // ---------------- TMA producer of group `warp`: lane i owns copy i of the stage ----------------
            const uint32_t first = static_cast<uint32_t>(warp) * ring;  // first stage of this group's ring
            const int OA = SA / p.a.slabs_per_op, OB = SB / p.b.slabs_per_op;
            const bool is_a = lane < OA;
            const bool active = lane < OA + OB;
            const UmmaOperandDev& o = is_a ? p.a : p.b;
            const void* tmap = is_a ? static_cast<const void*>(&tmapA) : static_cast<const void*>(&tmapB);
            const int slab = is_a ? lane * p.a.slabs_per_op : (lane - OA) * p.b.slabs_per_op;
            const uint32_t my_off = is_a ? static_cast<uint32_t>(slab * p.a.slab_bytes)
                                         : a_tile_bytes + static_cast<uint32_t>(slab * p.b.slab_bytes);
            if (lane == 0) {
                asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmapA)) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmapB)) : "memory");
            }
            uint32_t stage = 0, phase = 0;
            uint32_t issued_mask = 0, issued_parity = 0;
            for (uint32_t i = static_cast<uint32_t>(warp); i < my_tiles; i += 2) {
                const WorkUnit w = decode_unit(blockIdx.x + i * gridDim.x, p, tiles_m, tiles_n);
                const uint32_t tm = w.tm, tn = w.tn;
                int base[kMaxTmaRank] = {0, 0, 0, 0, 0};
                if (active) {
                    const uint32_t s = (is_a ? tm * SA : tn * SB) + slab;
                    if (s < static_cast<uint32_t>(o.total_slabs)) {
                        uint32_t rem = s;
    #pragma unroll
                        for (int d = 0; d < kMaxTmaRank; ++d) {
                            if (d < o.n_row_digits) {
                                const uint32_t e = static_cast<uint32_t>(o.row_digit_ext[d]);
                                const int idx = static_cast<int>(rem % e);
                                rem /= e;
                                const int v = d == o.chunk_digit ? idx * o.digit0_scale : idx;
    #pragma unroll
                                for (int t = 0; t < kMaxTmaRank; ++t)
                                    if (o.row_digit_dim[d] == t) base[t] = v;
                            }
                        }
                    } else {
                        // Slab beyond the tensor: start the box past the slab mode's end, TMA fills zeros.
    #pragma unroll
                        for (int t = 0; t < kMaxTmaRank; ++t)
                            if (o.row_digit_dim[o.chunk_digit] == t) base[t] = o.oob_coord;
                    }
                }
                int kd0 = w.it0 % p.k_digit_ext[0], kd1 = (w.it0 / p.k_digit_ext[0]) % p.k_digit_ext[1];
                int kd2 = w.it0 / (p.k_digit_ext[0] * p.k_digit_ext[1]);
                for (int it = 0; it < w.n_it; ++it) {
                    const uint32_t ps = first + stage;
                    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar_empty + ps), phase ^ 1u, abort_flag, 200u));
                    if (ok) {
                        if (lane == 0) mbar_arrive_expect_tx(smem_u32(bar_full + ps), stage_bytes);
                        __syncwarp();
                        if (active) {
                            int c[kMaxTmaRank];
    #pragma unroll
                            for (int t = 0; t < kMaxTmaRank; ++t) {
                                c[t] = base[t];
                                if (o.k_digit_dim[0] == t) c[t] = kd0 * p.BK;
                                if (o.k_digit_dim[1] == t) c[t] = kd1;
                                if (o.k_digit_dim[2] == t) c[t] = kd2;
                            }
                            tma_load_5d(smem_u32(smem + static_cast<size_t>(ps) * stage_bytes + my_off), tmap,
                                        smem_u32(bar_full + ps), c[0], c[1], c[2], c[3], c[4]);
                        }
                        issued_mask |= 1u << ps;
                        issued_parity = (issued_parity & ~(1u << ps)) | (phase << ps);
                    }
                    if (++kd0 == p.k_digit_ext[0]) {
                        kd0 = 0;
                        if (++kd1 == p.k_digit_ext[1]) {
                            kd1 = 0;
                            ++kd2;
                        }
                    }
                    if (++stage == ring) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (ld_shared_u32(abort_flag) && lane == 0) {
                // Give the bulk copies issued into these barriers a bounded time to land before the block ends.
                for (int s = 0; s < p.stages; ++s) {
                    if (!(issued_mask & (1u << s))) continue;
                    const unsigned long long t0 = global_timer();
                    while (!mbar_try_wait(smem_u32(bar_full + s), (issued_parity >> s) & 1u))
                        if (global_timer() - t0 > 100000000ull) break;
                }
            }
        } else {
            // ---------------- table builders: 64 threads, three entries each per tile ----------------
            const int bt = threadIdx.x - 64;
            for (uint32_t i = 0; i < my_tiles; ++i) {
                const WorkUnit w = decode_unit(blockIdx.x + i * gridDim.x, p, tiles_m, tiles_n);
                const uint32_t tm = w.tm, tn = w.tn;
                const uint32_t slot = (i & 1u) * 2u + ((i >> 1) & 1u);  // group, buffer
                const uint32_t use = i >> 2;                            // how often this slot was filled before
                if (!mbar_wait(smem_u32(tab_empty + slot), (use & 1u) ^ 1u, abort_flag, 500u)) break;
                const uint32_t tab = tabs + slot * kTabBytes;
#pragma unroll
                for (int e3 = 0; e3 < 3; ++e3) {
                    const int e = bt + e3 * 64;
                    const bool is_row = e < kBM;
                    if (!is_row && e - kBM >= NF * 16) continue;
                    const UmmaOperandDev& o = is_row ? p.a : p.b;
                    const int idx = is_row ? e : e - kBM;
                    const int sl = idx / o.slab_w, in = idx % o.slab_w;
                    bool ok;
                    int d0 = 0;
                    const long long off = slab_c_offset(o, (is_row ? tm * SA : tn * SB) + sl, &d0, &ok);
                    ok = ok && (d0 * o.slab_w + in < o.slab_mode_ext);
                    st_shared_s64(tab + static_cast<uint32_t>(e) * 8u, ok ? off + slab_elem_offset(o, d0, in) : -1);
                }
                mbar_arrive(smem_u32(tab_full + slot));
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---------------- consumers: two groups of 2 x 2 warps, warp tile 64 x 32 ----------------
        const int cw = warp & 3, grp = (warp >> 2) - 1, wm = cw & 1, wn = cw >> 1;
        const uint32_t fr = static_cast<uint32_t>(lane >> 2), fk = static_cast<uint32_t>(lane & 3);
        const uint32_t first = static_cast<uint32_t>(grp) * ring;
        // pitch between fragment pairs: one 16-wide slab (MN-major) or 16 rows (K-major)
        const bool rows64 = p.BK == 8;
        const uint32_t k_row = rows64 ? 64u : 128u;
        const bool a8 = AMN && p.a.slab_w == 8, b8 = BMN && p.b.slab_w == 8;  // 16 m = two slabs of 8
        const uint32_t a_pitch = AMN ? static_cast<uint32_t>(p.a.slab_bytes) * (a8 ? 2u : 1u) : 16u * k_row;
        const uint32_t b_pitch = BMN ? static_cast<uint32_t>(p.b.slab_bytes) * (b8 ? 2u : 1u) : 16u * k_row;
        const uint32_t a_thread = AMN ? static_cast<uint32_t>(wm * 4) * a_pitch + (a8 ? (fr >> 2) * static_cast<uint32_t>(p.a.slab_bytes) : 0u)
                                      : (static_cast<uint32_t>(wm * 64) + 2u * fr) * k_row;
        const uint32_t b_thread = a_tile_bytes + (BMN ? static_cast<uint32_t>(wn * (NF / 2)) * b_pitch + (b8 ? (fr >> 2) * static_cast<uint32_t>(p.b.slab_bytes) : 0u)
                                                      : (static_cast<uint32_t>(wn * NF * 8) + 2u * fr) * k_row);

        double acc[8][NF][2];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < NF; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

        uint32_t stage = 0, phase = 0;
        const bool prof = p.prof != nullptr && (threadIdx.x & 127) == 0 && grp == 0;
        long long t_all = prof ? clock64() : 0, t_full = 0, t_main = 0, t_tab = 0, t_store = 0;

        for (uint32_t i = static_cast<uint32_t>(grp); i < my_tiles; i += 2) {
            long long t0 = prof ? clock64() : 0;
            // group 1 starts half a main loop behind group 0 (named barrier 1: 128 waiting, 128 arriving)
            if (i == 1) asm volatile("bar.sync 1, 256;" ::: "memory");

            const WorkUnit w = decode_unit(blockIdx.x + i * gridDim.x, p, tiles_m, tiles_n);
            double* __restrict__ C = p.C64 + static_cast<long long>(w.split) * p.split_stride;
            bool tile_ok = true;
            // fa0/fb0 may already hold the first fragments of the stage about to be worked on: the last step
            // of a stage fetches them when the next stage has landed by then, instead of ending with a
            // step without loads and starting the next stage with loads nothing overlaps
            bool have_first = false;
            double fa0[8], fb0[NF], fa1[8], fb1[NF];
            for (int it = 0; it < w.n_it; ++it) {
                if (i == 0 && my_tiles > 1 && it == w.n_it / 2) asm volatile("bar.arrive 1, 256;" ::: "memory");
                const uint32_t ps = first + stage;
                bool ok = true;
                if (!have_first) {
                    const long long tw = prof ? clock64() : 0;
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar_full + ps), phase, abort_flag));
                    if (prof) t_full += clock64() - tw;
                }
                tile_ok = tile_ok && ok;
                const uint32_t next_stage = stage + 1 == ring ? 0u : stage + 1u, next_phase = stage + 1 == ring ? phase ^ 1u : phase;
                bool next_first = false;
                if (ok) {
                    const uint32_t sb = smem_u32(smem) + ps * stage_bytes;
                    FragAddr qa, qb;
                    if (!have_first) {
                        qa = frag_addr<AMN>(sb + a_thread, step_k(0, fk), fr, rows64, a8), qb = frag_addr<BMN>(sb + b_thread, step_k(0, fk), fr, rows64, b8);
                        load_all<AMN, 8>(fa0, qa, a_pitch);
                        load_all<BMN, NF>(fb0, qb, b_pitch);
                    }
                    qa = frag_addr<AMN>(sb + a_thread, step_k(1, fk), fr, rows64, a8), qb = frag_addr<BMN>(sb + b_thread, step_k(1, fk), fr, rows64, b8);
                    mma_step<true, AMN, BMN, NF>(acc, fa0, fb0, fa1, fb1, qa, qb, a_pitch, b_pitch);
                    if (p.BK == 16) {
                        qa = frag_addr<AMN>(sb + a_thread, step_k(2, fk), fr, rows64, a8), qb = frag_addr<BMN>(sb + b_thread, step_k(2, fk), fr, rows64, b8);
                        mma_step<true, AMN, BMN, NF>(acc, fa1, fb1, fa0, fb0, qa, qb, a_pitch, b_pitch);
                        qa = frag_addr<AMN>(sb + a_thread, step_k(3, fk), fr, rows64, a8), qb = frag_addr<BMN>(sb + b_thread, step_k(3, fk), fr, rows64, b8);
                        mma_step<true, AMN, BMN, NF>(acc, fa0, fb0, fa1, fb1, qa, qb, a_pitch, b_pitch);
                    }
                    // last step: one look at the next stage's barrier; if its data is there, fetch from it
                    if (it + 1 < w.n_it)
                        next_first = __all_sync(0xffffffffu, mbar_test_wait(smem_u32(bar_full + first + next_stage), next_phase));
                    if (next_first) {
                        const uint32_t nb = smem_u32(smem) + (first + next_stage) * stage_bytes;
                        qa = frag_addr<AMN>(nb + a_thread, step_k(0, fk), fr, rows64, a8), qb = frag_addr<BMN>(nb + b_thread, step_k(0, fk), fr, rows64, b8);
                        mma_step<true, AMN, BMN, NF>(acc, fa1, fb1, fa0, fb0, qa, qb, a_pitch, b_pitch);
                    } else {
                        mma_step<false, AMN, BMN, NF>(acc, fa1, fb1, fa0, fb0, qa, qb, a_pitch, b_pitch);
                    }
                }
                have_first = next_first;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(bar_empty + ps));  // this warp is done reading the stage
                stage = next_stage;
                phase = next_phase;
            }
            if (prof) { const long long t1 = clock64(); t_main += t1 - t0; t0 = t1; }

            // the tile's offset tables were built while it was being computed
            const uint32_t slot = static_cast<uint32_t>(grp) * 2u + ((i >> 1) & 1u);
            tile_ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(tab_full + slot), (i >> 2) & 1u, abort_flag)) && tile_ok;
            const uint32_t row_tab = tabs + slot * kTabBytes, col_tab = row_tab + kBM * 8u;
            if (prof) { const long long t1 = clock64(); t_tab += t1 - t0; t0 = t1; }

            // store: four consecutive rows per (fragment pair, column fragment), 32 bytes when aligned
            long long cn[NF];
#pragma unroll
            for (int j = 0; j < NF; ++j)
                cn[j] = ld_shared_s64(col_tab + (static_cast<uint32_t>(wn * NF * 8 + 16 * (j >> 1) + (j & 1)) + 2u * fr) * 8u);
            if (p.store_across_slabs) {
                // The warp's 64 rows are four slabs of 16; slab q is index a0 + q of C's stride-1 mode and the rows
                // of a slab run along another mode.  Row (4 fk + dd) of the four slabs is four neighbouring
                // elements of C: acc[2 q + (dd & 1)][j][dd >> 1], q = 0..3.
#pragma unroll
                for (int dd = 0; dd < 4; ++dd) {
                    const int par = dd & 1, h = dd >> 1;
                    const uint32_t r = static_cast<uint32_t>(wm * 64) + 4u * fk + static_cast<uint32_t>(dd);
                    const long long cm0 = ld_shared_s64(row_tab + r * 8u), cm1 = ld_shared_s64(row_tab + (r + 16u) * 8u);
                    const long long cm2 = ld_shared_s64(row_tab + (r + 32u) * 8u), cm3 = ld_shared_s64(row_tab + (r + 48u) * 8u);
                    const bool run4 = cm0 >= 0 && cm1 == cm0 + 1 && cm2 == cm0 + 2 && cm3 == cm0 + 3;
#pragma unroll
                    for (int j = 0; j < NF; ++j) {
                        if (tile_ok && cn[j] >= 0) {
                            double* dst = C + cm0 + cn[j];
                            if (run4 && (reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
                                st_global_cs_v4f64(dst, acc[par][j][h], acc[2 + par][j][h], acc[4 + par][j][h], acc[6 + par][j][h]);
                            } else {
                                if (cm0 >= 0) __stcs(dst, acc[par][j][h]);
                                if (cm1 >= 0) __stcs(C + cm1 + cn[j], acc[2 + par][j][h]);
                                if (cm2 >= 0) __stcs(C + cm2 + cn[j], acc[4 + par][j][h]);
                                if (cm3 >= 0) __stcs(C + cm3 + cn[j], acc[6 + par][j][h]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < NF; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;
            } else
#pragma unroll
            for (int pr = 0; pr < 4; ++pr) {
                const uint32_t r = static_cast<uint32_t>(wm * 64 + 16 * pr) + 4u * fk;
                const long long cm0 = ld_shared_s64(row_tab + r * 8u), cm1 = ld_shared_s64(row_tab + r * 8u + 8u);
                const long long cm2 = ld_shared_s64(row_tab + r * 8u + 16u), cm3 = ld_shared_s64(row_tab + r * 8u + 24u);
                const bool run4 = cm0 >= 0 && cm1 == cm0 + 1 && cm2 == cm0 + 2 && cm3 == cm0 + 3;
#pragma unroll
                for (int j = 0; j < NF; ++j) {
                    if (tile_ok && cn[j] >= 0) {
                        double* dst = C + cm0 + cn[j];
                        if (run4 && (reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
                            st_global_cs_v4f64(dst, acc[2 * pr][j][0], acc[2 * pr + 1][j][0], acc[2 * pr][j][1], acc[2 * pr + 1][j][1]);
                        } else {
                            // ragged or odd-aligned runs: 16 bytes where two rows are neighbours, else one by one
                            if (cm0 >= 0 && cm1 == cm0 + 1 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                                __stcs(reinterpret_cast<double2*>(dst), make_double2(acc[2 * pr][j][0], acc[2 * pr + 1][j][0]));
                            } else {
                                if (cm0 >= 0) __stcs(dst, acc[2 * pr][j][0]);
                                if (cm1 >= 0) __stcs(C + cm1 + cn[j], acc[2 * pr + 1][j][0]);
                            }
                            double* dst2 = C + cm2 + cn[j];
                            if (cm2 >= 0 && cm3 == cm2 + 1 && (reinterpret_cast<uintptr_t>(dst2) & 15u) == 0) {
                                __stcs(reinterpret_cast<double2*>(dst2), make_double2(acc[2 * pr][j][1], acc[2 * pr + 1][j][1]));
                            } else {
                                if (cm2 >= 0) __stcs(dst2, acc[2 * pr][j][1]);
                                if (cm3 >= 0) __stcs(C + cm3 + cn[j], acc[2 * pr + 1][j][1]);
                            }
                        }
                    }
                    acc[2 * pr][j][0] = acc[2 * pr][j][1] = acc[2 * pr + 1][j][0] = acc[2 * pr + 1][j][1] = 0.0;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(tab_empty + slot));  // this warp is done with the tables
            if (prof) t_store += clock64() - t0;
        }
        if (prof) {
            long long* q = p.prof + static_cast<size_t>(blockIdx.x) * 8;
            q[0] = clock64() - t_all;
            q[1] = t_full;
            q[2] = t_main;
            q[3] = t_tab;
            q[4] = t_store;
            q[5] = 0;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && ld_shared_u32(abort_flag)) atomicMax(p.status, 1);
}

template <bool AMN, bool BMN, int NF>
cudaError_t launch_variant(const UmmaParams& p, const void* tmapA, const void* tmapB, int smem_bytes, unsigned grid, cudaStream_t stream)
{
    dmma_tma_kernel<AMN, BMN, NF><<<grid, kThreads64, smem_bytes, stream>>>(*static_cast<const CUtensorMap*>(tmapA),
                                                                             *static_cast<const CUtensorMap*>(tmapB), p);
    return cudaGetLastError();
}

template <int NF>
cudaError_t launch_width(const UmmaParams& p, const void* tmapA, const void* tmapB, int smem_bytes, unsigned grid, cudaStream_t stream)
{
    if (p.a.major && p.b.major) return launch_variant<true, true, NF>(p, tmapA, tmapB, smem_bytes, grid, stream);
    if (p.a.major) return launch_variant<true, false, NF>(p, tmapA, tmapB, smem_bytes, grid, stream);
    if (p.b.major) return launch_variant<false, true, NF>(p, tmapA, tmapB, smem_bytes, grid, stream);
    return launch_variant<false, false, NF>(p, tmapA, tmapB, smem_bytes, grid, stream);
}

template <int NF>
cudaError_t configure_width()
{
    const int smem_bytes = kMaxDynamicSmemBytes;  // the same opt-in maximum for every run (the cap is per function and device)
    cudaError_t e = cudaFuncSetAttribute(dmma_tma_kernel<false, false, NF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dmma_tma_kernel<false, true, NF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dmma_tma_kernel<true, false, NF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dmma_tma_kernel<true, true, NF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    return e;
}

}  // namespace

cudaError_t dmma_tma_configure()
{
    const cudaError_t e = configure_width<4>();
    return e == cudaSuccess ? configure_width<2>() : e;
}

cudaError_t launch_dmma_tma(const UmmaParams& p, const void* tmapA, const void* tmapB, int smem_bytes, int num_sms, cudaStream_t stream)
{
    const long long total = p.tiles_m * p.tiles_n * p.k_splits;
    if (total <= 0 || p.k_splits < 1 || p.stages < 2 || (p.stages & 1) || (p.BN != 64 && p.BN != 32)) return cudaErrorInvalidValue;
    const unsigned grid = static_cast<unsigned>(total < num_sms ? total : num_sms);
    return p.BN == 64 ? launch_width<4>(p, tmapA, tmapB, smem_bytes, grid, stream) : launch_width<2>(p, tmapA, tmapB, smem_bytes, grid, stream);
}

}  // namespace tcontb
