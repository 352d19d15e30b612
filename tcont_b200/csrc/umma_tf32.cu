// umma_tf32.cu -- direct TF32 contraction on the 5th-generation tensor cores (sm_100a only).
//
// One persistent CTA per SM, three roles:
//   warp 0      TMA producer.  An operand tile is a run of "slabs"; each slab is one 2-D box of a
//               5-D tensor map laid over the operand's own (strided, multi-mode) layout, written
//               with a 128-byte swizzle so that it is already a UMMA canonical tile.  Lane i owns
//               slab i and issues its own cp.async.bulk.tensor per K step (no cluster multicast).
//   warp 1      allocates tensor memory, and its lane 0 issues tcgen05.mma kind::tf32
//               (M = 128, N = BN, K = 8 per instruction) into one of two TMEM accumulators.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (lane = row), scatter it to C's final,
//               permuted position; with C's stride-1 mode on the slab rows a warp writes 128
//               contiguous bytes per column.
// Every wait is bounded: when one gives up the CTA raises a status word, stops issuing work,
// lets the remaining loops run empty, waits (bounded) for its outstanding bulk copies, frees its
// tensor memory and returns.
//
// Stands where the reference runs its generated TF32 WMMA kernels
// (backends/cogent/plan/generators/kernels/kernel_compute.py:851-1833, kernel_load.py:687-868,
// kernel_store.py:280-507): same contract (C overwritten with the fp32-accumulated TF32
// products; raw fp32 bits are handed to the tensor core, which ignores the low mantissa bits).
#include <cuda.h>
#include <cstdlib>

#include "kernels.hpp"
#include "tile_common.cuh"

namespace tcontb {
namespace {

constexpr int kThreads = 224;   // warp 0 producer, 1 MMA issue, 2-5 epilogue, 6 second producer (launched only with two producers)
// The same copy for a CTA pair: the destination is this CTA's shared memory, the mbarrier may live
// in the partner CTA (address in the cluster window).  No multicast.
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster, int c0, int c1, int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

__device__ __forceinline__ void red_add_relaxed(unsigned int* addr, unsigned int v)
{
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_relaxed(const unsigned int* addr)
{
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}

// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// One commit that arrives on the barrier at the same offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair_both(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(static_cast<unsigned short>(3)) : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// Shared-memory matrix descriptor, descriptor version 1 (Blackwell).
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 version      bits 61-63 layout type
// Layout types used here: 2 = 128-byte swizzle in 16-byte units (K-major operands);
// 1 = 128-byte swizzle in 32-byte units, the only layout the tensor core accepts for an MN-major
// operand of a 32-bit type (TMA writes it with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(layout_type) << 61;
    return d;
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// PAIR = false: one CTA per 128 x BN tile (cta_group::1).
// PAIR = true : a cluster of two CTAs per 256 x BN tile (cta_group::2).  CTA r of the pair stages its own
//               128 rows of A and half of the B tile (no multicast; every copy is a plain TMA load into
//               the issuing CTA), CTA 0 issues the MMAs for both, each CTA drains its own 128 x BN
//               accumulator.  B traffic per flop halves, which is what the operand-fetch-bound 1-CTA
//               kernel lacks.
// NP = producer warps (1, or 2 taking turns stage by stage); a template parameter so that the one-producer loop,
// whose pass per stage is the tightest thing in the pair kernel, carries none of the two-producer bookkeeping
// (with it as a run-time value the pair kernel lost 8 %).
template <bool PAIR, int NP>
__global__ void __launch_bounds__(kThreads, 1)
umma_tf32_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                 const __grid_constant__ UmmaParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // 1024-byte aligned
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_rank() : 0u;        // 0 = the CTA that issues the MMAs
    const int SA = p.a.slabs_per_tile, SB = p.b.slabs_per_tile;
    const int SBL = PAIR ? SB / 2 : SB;                       // B slabs this CTA stages itself
    const uint32_t a_tile_bytes = static_cast<uint32_t>(SA * p.a.slab_bytes);
    const uint32_t stage_bytes = a_tile_bytes + static_cast<uint32_t>(SBL * p.b.slab_bytes);

    uint8_t* aux = smem + static_cast<size_t>(p.stages) * stage_bytes;
    uint64_t* bar_full = reinterpret_cast<uint64_t*>(aux);  // [8]
    uint64_t* bar_empty = bar_full + 8;                     // [8]
    uint64_t* bar_tfull = bar_empty + 8;                    // [2]
    uint64_t* bar_tempty = bar_tfull + 2;                   // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tempty + 2);
    const uint32_t abort_flag = smem_u32(tmem_slot + 1);
    const uint32_t col_off = smem_u32(aux + 256);  // long long [2][256], -1 = column not stored

    uint32_t tmem_cols = 32;
    while (tmem_cols < static_cast<uint32_t>(2 * p.BN)) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(bar_full + s), 1);
            mbar_init(smem_u32(bar_empty + s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(bar_tfull + a), 1);
            mbar_init(smem_u32(bar_tempty + a), PAIR ? 256 : 128);
        }
        st_shared_u32(abort_flag, 0u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // the partner's barriers exist before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Work units: 128-row tiles, or 256-row tile pairs; unit u of a pair covers row tiles 2u and 2u+1.
    const uint32_t tiles_m = PAIR ? (static_cast<uint32_t>(p.tiles_m) + 1u) / 2u : static_cast<uint32_t>(p.tiles_m);
    const uint32_t tiles_n = static_cast<uint32_t>(p.tiles_n);
    const uint32_t total_tiles = tiles_m * tiles_n * static_cast<uint32_t>(p.k_splits);  // work units (tile, k range)
    const uint32_t first_unit = PAIR ? blockIdx.x / 2u : blockIdx.x;
    const uint32_t unit_step = PAIR ? gridDim.x / 2u : gridDim.x;

    if (warp == 0 || (warp == 6 && NP == 2)) {
        // ---------------- TMA producer: lane i owns slab i of the stage ----------------
        // With two producers (p.producers == 2, an even number of stages) warp 0 fills the even k iterations of the
        // CTA and warp 6 the odd ones: the wait-announce-copy round trip of one warp may then take two stages' worth
        // of MMA time, which is what lets stages be half as large and the ring twice as deep.
        constexpr int np = NP;
        const int pi = warp == 0 ? 0 : 1;
        // lane i owns copy i of the stage; a copy brings slabs_per_op consecutive slabs
        const int OA = SA / p.a.slabs_per_op, OBL = SBL / p.b.slabs_per_op;
        const bool is_a = lane < OA;
        const bool active = lane < OA + OBL;
        const UmmaOperandDev& o = is_a ? p.a : p.b;
        const void* tmap = is_a ? static_cast<const void*>(&tmapA) : static_cast<const void*>(&tmapB);
        const int slab = is_a ? lane * p.a.slabs_per_op : (lane - OA) * p.b.slabs_per_op;   // first slab of the copy, inside this CTA's part
        const uint32_t my_off = is_a ? static_cast<uint32_t>(slab * p.a.slab_bytes)
                                     : a_tile_bytes + static_cast<uint32_t>(slab * p.b.slab_bytes);
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmapA)) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmapB)) : "memory");
        }
        int stage = 0;
        uint32_t phase = 0;
        uint32_t issued_mask = 0, issued_parity = 0;
        long long t_empty = 0;
        int cta_iter = 0;  // k iterations this CTA has gone through (test hook: one of them may be left out)
        // pace keeping (see UmmaParams): one producer per work unit takes part
        const bool pacing = p.pace != nullptr && rank == 0 && pi == 0;
        bool pace_live = pacing;
        const unsigned int pace_peers = PAIR ? gridDim.x / 2u : gridDim.x;
        long long pace_waits = 0, pace_clk = 0;
        // One look at the next stage's empty barrier is issued right behind the copies of the current one, so
        // that its latency overlaps theirs; `have_slot` says that look found the stage free.
        bool have_slot = false;

        // TMA coordinates of this lane's copy for the rows / columns of a work unit (the k coordinates come on top);
        // worked out one unit ahead, so that the first copies of a unit do not wait for the divisions
        auto unit_base = [&](const WorkUnit& u, int (&base)[kMaxTmaRank]) {
#pragma unroll
            for (int t = 0; t < kMaxTmaRank; ++t) base[t] = 0;
            if (!active) return;
            const uint32_t s = is_a ? (PAIR ? 2u * u.tm + rank : u.tm) * SA + slab
                                    : u.tn * SB + (PAIR ? rank * SBL : 0u) + slab;
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
        };
        WorkUnit w_next{};
        int base_next[kMaxTmaRank] = {0, 0, 0, 0, 0};
        if (first_unit < total_tiles) {
            w_next = decode_unit(first_unit, p, tiles_m, tiles_n);
            unit_base(w_next, base_next);
        }

        for (uint32_t tile = first_unit; tile < total_tiles; tile += unit_step) {
            const WorkUnit w = w_next;
            int base[kMaxTmaRank];
#pragma unroll
            for (int t = 0; t < kMaxTmaRank; ++t) base[t] = base_next[t];
            const bool have_next = tile + unit_step < total_tiles;
            if (have_next) {
                w_next = decode_unit(tile + unit_step, p, tiles_m, tiles_n);
                unit_base(w_next, base_next);
            }
            // K digits: chunk of the chunked mode, then the other K modes
            int kd0 = w.it0 % p.k_digit_ext[0], kd1 = (w.it0 / p.k_digit_ext[0]) % p.k_digit_ext[1];
            int kd2 = w.it0 / (p.k_digit_ext[0] * p.k_digit_ext[1]);
            for (int it = 0; it < w.n_it; ++it, ++cta_iter) {
                const bool mine = np == 1 || (cta_iter & 1) == pi;
                if (mine && pace_live && (cta_iter & ((1 << p.pace_shift) - 1)) == 0) {
                    const int blk = cta_iter >> p.pace_shift;
                    int go = 1;
                    if (lane == 0) {
                        red_add_relaxed(p.pace + 1 + blk, 1u);
                        if (blk >= p.pace_lead) {
                            const long long tp = p.prof ? clock64() : 0;
                            const unsigned int* behind = p.pace + 1 + blk - p.pace_lead;
                            unsigned long long t_start = 0;
                            while (ld_relaxed(behind) + ld_relaxed(p.pace) < pace_peers) {
                                const unsigned long long now = global_timer();
                                if (t_start == 0) { t_start = now; ++pace_waits; }
                                else if (now - t_start > 50000ull) { go = 0; break; }   // 50 us: somebody is not running; stop keeping pace
                            }
                            if (p.prof) pace_clk += clock64() - tp;
                        }
                    }
                    pace_live = __shfl_sync(0xffffffffu, go, 0) != 0;
                }
                const long long t0 = p.prof ? clock64() : 0;
                const bool ok = mine && (have_slot || __all_sync(0xffffffffu, mbar_wait(smem_u32(bar_empty + stage), phase ^ 1u, abort_flag, 0, p.wait_limit_ns)));
                if (p.prof) t_empty += clock64() - t0;
                if (ok && cta_iter != p.test_skip_iter) {
                    // one arrival with the byte count of the whole stage; in a pair the MMA-issuing CTA
                    // accounts for both CTAs' copies, which all signal its barrier
                    if (lane == 0 && rank == 0) mbar_arrive_expect_tx(smem_u32(bar_full + stage), PAIR ? 2u * stage_bytes : stage_bytes);
                    __syncwarp();
                    if (active) {
                        int c[kMaxTmaRank];
#pragma unroll
                        for (int t = 0; t < kMaxTmaRank; ++t) {
                            c[t] = base[t];
                            if (o.k_digit_dim[0] == t) c[t] = kd0 * o.k0_scale;
                            if (o.k_digit_dim[1] == t) c[t] = kd1;
                            if (o.k_digit_dim[2] == t) c[t] = kd2;
                        }
                        const uint32_t dst = smem_u32(smem + static_cast<size_t>(stage) * stage_bytes + my_off);
                        if (PAIR) tma_load_5d_pair(dst, tmap, map_to_cta(smem_u32(bar_full + stage), 0u), c[0], c[1], c[2], c[3], c[4]);
                        else tma_load_5d(dst, tmap, smem_u32(bar_full + stage), c[0], c[1], c[2], c[3], c[4]);
                    }
                    issued_mask |= 1u << stage;
                    issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
                }
                if (++kd0 == p.k_digit_ext[0]) {
                    kd0 = 0;
                    if (++kd1 == p.k_digit_ext[1]) {
                        kd1 = 0;
                        ++kd2;
                    }
                }
                if (++stage == p.stages) {
                    stage = 0;
                    phase ^= 1u;
                }
                // a look at the stage of this warp's next iteration (the next one, or the one after it)
                if (np == 1) {
                    have_slot = __all_sync(0xffffffffu, mbar_test_wait(smem_u32(bar_empty + stage), phase ^ 1u));
                } else if (mine) {
                    const int s2 = stage + 1 == p.stages ? 0 : stage + 1;
                    const uint32_t ph2 = stage + 1 == p.stages ? phase ^ 1u : phase;
                    have_slot = __all_sync(0xffffffffu, mbar_test_wait(smem_u32(bar_empty + s2), ph2 ^ 1u));
                }
            }
        }
        if (pacing && lane == 0) red_add_relaxed(p.pace, 1u);
        if (p.prof && lane == 0 && pi == 0) {
            p.prof[blockIdx.x * 8 + 3] = t_empty;
            p.prof[blockIdx.x * 8 + 6] = pace_clk;
            p.prof[blockIdx.x * 8 + 7] = pace_waits * 2 + (pacing && !pace_live ? 1 : 0);
        }
        if (ld_shared_u32(abort_flag) && lane == 0 && rank == 0) {
            // Give the bulk copies issued into this barrier a bounded time to land before the CTA ends.
            for (int s = 0; s < p.stages; ++s) {
                if (!(issued_mask & (1u << s))) continue;
                const unsigned long long t0 = global_timer();
                while (!mbar_try_wait(smem_u32(bar_full + s), (issued_parity >> s) & 1u))
                    if (global_timer() - t0 > 100000000ull) break;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(p.a.major) << 15) |
                                   (static_cast<uint32_t>(p.b.major) << 16) | (static_cast<uint32_t>(p.BN >> 3) << 17) |
                                   (static_cast<uint32_t>((PAIR ? 256 : 128) >> 4) << 24);
            // MN-major: slabs sit one leading-byte-offset apart; the 8 K rows of one MMA are two
            //           4-row groups 512 bytes apart (stride byte offset), 1024 bytes per MMA.
            // K-major : 8-row groups sit 1024 bytes apart, 8 K elements per MMA = 32 bytes.
            const uint32_t a_lbo = p.a.major ? static_cast<uint32_t>(p.a.slab_bytes) : 16u;
            const uint32_t b_lbo = p.b.major ? static_cast<uint32_t>(p.b.slab_bytes) : 16u;
            const uint32_t a_sbo = p.a.major ? 512u : 1024u, b_sbo = p.b.major ? 512u : 1024u;
            const uint32_t a_type = p.a.major ? 1u : 2u, b_type = p.b.major ? 1u : 2u;
            // Byte offset of MMA k step kk inside an operand's part of the stage.  MN-major: 1 024 bytes per step
            // (eight k rows of 128 bytes).  K-major: 32 bytes per step inside a 128-byte row of 32 k, and with a
            // k chunk of 64 the second 32 k lie one whole slab image (slab rows x 128 bytes) further on.
            const uint32_t a_chunk = static_cast<uint32_t>(p.a.slab_w) * 128u, b_chunk = static_cast<uint32_t>(p.b.slab_w) * 128u;
            const int ksteps = p.BK / 8;
            int stage = 0;
            uint32_t phase = 0;
            long long iter = 0;
            long long t_tempty = 0, t_full = 0, t_all = clock64();
            for (uint32_t tile = first_unit; tile < total_tiles; tile += unit_step, ++iter) {
                const int acc = static_cast<int>(iter & 1);
                const uint32_t acc_parity = static_cast<uint32_t>((iter >> 1) & 1);
                long long t0 = p.prof ? clock64() : 0;
                bool ok = mbar_wait(smem_u32(bar_tempty + acc), acc_parity ^ 1u, abort_flag, 0, p.wait_limit_ns);
                if (p.prof) t_tempty += clock64() - t0;
                tcgen05_fence_after();
                const uint32_t tmem_c = tmem_base + static_cast<uint32_t>(acc * p.BN);
                const int n_it = decode_unit(tile, p, tiles_m, tiles_n).n_it;
                for (int it = 0; it < n_it; ++it) {
                    t0 = p.prof ? clock64() : 0;
                    ok = ok && mbar_wait(smem_u32(bar_full + stage), phase, abort_flag, 0, p.wait_limit_ns);
                    if (p.prof) t_full += clock64() - t0;
                    if (ok) {
                        tcgen05_fence_after();
                        const uint32_t a_base = smem_u32(smem + static_cast<size_t>(stage) * stage_bytes);
                        const uint32_t b_base = a_base + a_tile_bytes;
                        for (int kk = 0; kk < ksteps; ++kk) {
                            const uint32_t ukk = static_cast<uint32_t>(kk);
                            const uint32_t a_off = p.a.major ? ukk * 1024u : (ukk >> 2) * a_chunk + (ukk & 3u) * 32u;
                            const uint32_t b_off = p.b.major ? ukk * 1024u : (ukk >> 2) * b_chunk + (ukk & 3u) * 32u;
                            const uint64_t da = smem_desc(a_base + a_off, a_lbo, a_sbo, a_type);
                            const uint64_t db = smem_desc(b_base + b_off, b_lbo, b_sbo, b_type);
                            if (PAIR) umma_tf32_pair(tmem_c, da, db, idesc, (it | kk) != 0 ? 1u : 0u);
                            else umma_tf32(tmem_c, da, db, idesc, (it | kk) != 0 ? 1u : 0u);
                        }
                        // frees the stage (in both CTAs of a pair) once the MMAs have read it
                        if (PAIR) {
                            umma_commit_pair_both(smem_u32(bar_empty + stage));
                        } else {
                            umma_commit(smem_u32(bar_empty + stage));
                        }
                    }
                    if (++stage == p.stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) {  // accumulator complete
                    if (PAIR) {
                        umma_commit_pair_both(smem_u32(bar_tfull + acc));
                    } else {
                        umma_commit(smem_u32(bar_tfull + acc));
                    }
                }
            }
            if (p.prof) {
                p.prof[blockIdx.x * 8 + 0] = clock64() - t_all;
                p.prof[blockIdx.x * 8 + 1] = t_tempty;
                p.prof[blockIdx.x * 8 + 2] = t_full;
            }
        }
    } else if (warp < 6) {
        // ---------------- epilogue: 4 warps, warp w reads TMEM lanes 32*(w%4).. ----------------
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int et = threadIdx.x - 64;
        long long iter = 0;
        long long t_tfull = 0, t_epi = clock64();
        for (uint32_t tile = first_unit; tile < total_tiles; tile += unit_step, ++iter) {
            const WorkUnit w = decode_unit(tile, p, tiles_m, tiles_n);
            const uint32_t tm = w.tm, tn = w.tn;
            const int acc = static_cast<int>(iter & 1);
            const uint32_t acc_parity = static_cast<uint32_t>((iter >> 1) & 1);
            // this thread's row of C
            bool row_ok;
            int digit0 = 0;
            const int a_slab = row / p.a.slab_w, a_in = row % p.a.slab_w;
            long long row_off = slab_c_offset(p.a, (PAIR ? 2u * tm + rank : tm) * SA + a_slab, &digit0, &row_ok);
            row_ok = row_ok && (digit0 * p.a.slab_w + a_in < p.a.slab_mode_ext);
            row_off += a_in * p.a.row_elem_cstride;
            // Column offsets of this tile.  A 32-column chunk of the accumulator never straddles a
            // B slab when slabs are 32 or more columns wide, so one base offset and a valid-column
            // count per chunk suffice (chunk table); narrower slabs use a per-column table.
            const uint32_t cols = col_off + static_cast<uint32_t>(acc) * 256u * 8u;
            const bool wide_slabs = p.b.slab_w >= 32;
            if (wide_slabs) {
                if (et < (p.BN >> 5)) {
                    bool ch_ok;
                    int d0 = 0;
                    const int j = et * 32;
                    const int b_slab = j / p.b.slab_w, b_in = j % p.b.slab_w;
                    const long long off = slab_c_offset(p.b, tn * SB + b_slab, &d0, &ch_ok);
                    int nvalid = p.b.slab_mode_ext - (d0 * p.b.slab_w + b_in);
                    nvalid = !ch_ok ? 0 : nvalid > 32 ? 32 : nvalid < 0 ? 0 : nvalid;
                    st_shared_s64(cols + static_cast<uint32_t>(et) * 16u, off + b_in * p.b.row_elem_cstride);
                    st_shared_u32(cols + static_cast<uint32_t>(et) * 16u + 8u, static_cast<uint32_t>(nvalid));
                }
            } else {
                for (int j = et; j < p.BN; j += 128) {
                    bool col_ok;
                    int d0 = 0;
                    const int b_slab = j / p.b.slab_w, b_in = j % p.b.slab_w;
                    long long off = slab_c_offset(p.b, tn * SB + b_slab, &d0, &col_ok);
                    col_ok = col_ok && (d0 * p.b.slab_w + b_in < p.b.slab_mode_ext);
                    st_shared_s64(cols + static_cast<uint32_t>(j) * 8u, col_ok ? off + b_in * p.b.row_elem_cstride : -1);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            // accumulator-empty barrier lives in the MMA-issuing CTA; in a pair both CTAs' epilogues arrive on it
            const uint32_t tempty_addr = PAIR ? map_to_cta(smem_u32(bar_tempty + acc), 0u) : smem_u32(bar_tempty + acc);
            auto release_acc = [&]() {
                if (PAIR) mbar_arrive_cluster(tempty_addr);
                else mbar_arrive(tempty_addr);
            };
            bool ok = true;
            const long long t0 = p.prof ? clock64() : 0;
            if (lane == 0) ok = mbar_wait(smem_u32(bar_tfull + acc), acc_parity, abort_flag, 0, p.wait_limit_ns);
            if (p.prof) t_tfull += clock64() - t0;
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            tcgen05_fence_after();
            if (ok) {
                // (with a contracted-mode split over several GPUs the tile's column range belongs to one owner, whose
                // memory, local or a peer's over NVLink, takes the plain stores below)
                float* cbase = p.owners > 1 ? p.owner_base[tn / static_cast<uint32_t>(p.tn_per_owner)] : p.C;
                float* crow = cbase + static_cast<long long>(w.split) * p.split_stride + row_off;
                const long long col_stride = p.b.row_elem_cstride;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * p.BN);
                const int nchunks = p.BN >> 5;
                // TMEM loads run one chunk ahead of the stores.
                auto store_chunk = [&](const uint32_t (&v)[32], int c) {
                    if (wide_slabs) {
                        const long long base = ld_shared_s64(cols + static_cast<uint32_t>(c) * 16u);
                        const int nvalid = row_ok ? static_cast<int>(ld_shared_u32(cols + static_cast<uint32_t>(c) * 16u + 8u)) : 0;
                        float* ptr = crow + base;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (j < nvalid) __stcs(ptr, __uint_as_float(v[j]));
                            ptr += col_stride;
                        }
                    } else {
                        // lane j keeps the offset of column 32*c + j; fetch all 32 by shuffle, then store
                        const long long mine = ld_shared_s64(cols + static_cast<uint32_t>(c * 32 + lane) * 8u);
                        const int lo = static_cast<int>(mine), hi = static_cast<int>(mine >> 32);
                        long long co[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const unsigned ulo = static_cast<unsigned>(__shfl_sync(0xffffffffu, lo, j));
                            const int shi = __shfl_sync(0xffffffffu, hi, j);
                            co[j] = (static_cast<long long>(shi) << 32) | ulo;
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (row_ok && co[j] >= 0) __stcs(crow + co[j], __uint_as_float(v[j]));
                    }
                };
                uint32_t v0[32], v1[32];
                tmem_ld_32x32(taddr, v0);
                for (int c = 0; c < nchunks; c += 2) {
                    tmem_ld_wait();
                    if (c + 1 < nchunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 1) * 32), v1);
                    else {
                        // all of the accumulator is in registers: hand it back to the MMA warp early
                        tcgen05_fence_before();
                        release_acc();
                    }
                    store_chunk(v0, c);
                    if (c + 1 < nchunks) {
                        tmem_ld_wait();
                        if (c + 2 < nchunks) tmem_ld_32x32(taddr + static_cast<uint32_t>((c + 2) * 32), v0);
                        else {
                            tcgen05_fence_before();
                            release_acc();
                        }
                        store_chunk(v1, c + 1);
                    }
                }
            } else {
                tcgen05_fence_before();
                release_acc();
            }
        }
        if (p.prof && et == 0) {
            p.prof[blockIdx.x * 8 + 4] = clock64() - t_epi;
            p.prof[blockIdx.x * 8 + 5] = t_tfull;
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // neither CTA leaves while its partner may still read or signal its memory
    tcgen05_fence_after();
    if (warp == 1) {
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
    if (threadIdx.x == 0 && ld_shared_u32(abort_flag)) atomicMax(p.status, 1);
}

}  // namespace

// The dynamic shared-memory cap is a property of the function on a device, not of a run: every run sets
// the same opt-in maximum, so runs with different stage counts can live side by side.
cudaError_t umma_tf32_configure()
{
    cudaError_t e = cudaFuncSetAttribute(umma_tf32_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(umma_tf32_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(umma_tf32_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmemBytes);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(umma_tf32_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmemBytes);
}

cudaError_t launch_umma_tf32(const UmmaParams& p, const void* tmapA, const void* tmapB, int smem_bytes, int num_sms,
                             cudaStream_t stream)
{
    const CUtensorMap& ta = *static_cast<const CUtensorMap*>(tmapA);
    const CUtensorMap& tb = *static_cast<const CUtensorMap*>(tmapB);
    // (tuning switch TCONT_UMMA_IDLE_WARP=1: launch the seventh warp although nothing uses it)
    static const bool idle_warp = std::getenv("TCONT_UMMA_IDLE_WARP") != nullptr;
    const unsigned threads = p.producers == 2 || idle_warp ? kThreads : kThreads - 32;
    if (p.pair) {
        const long long units = ((p.tiles_m + 1) / 2) * p.tiles_n * p.k_splits;
        if (units <= 0) return cudaErrorInvalidValue;
        const long long clusters = units < num_sms / 2 ? units : num_sms / 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (p.producers == 2) return cudaLaunchKernelEx(&cfg, umma_tf32_kernel<true, 2>, ta, tb, p);
        return cudaLaunchKernelEx(&cfg, umma_tf32_kernel<true, 1>, ta, tb, p);
    }
    const long long total = p.tiles_m * p.tiles_n * p.k_splits;
    if (total <= 0) return cudaErrorInvalidValue;
    const unsigned grid = static_cast<unsigned>(total < num_sms ? total : num_sms);
    if (p.producers == 2) umma_tf32_kernel<false, 2><<<grid, threads, smem_bytes, stream>>>(ta, tb, p);
    else umma_tf32_kernel<false, 1><<<grid, threads, smem_bytes, stream>>>(ta, tb, p);
    return cudaGetLastError();
}

}  // namespace tcontb
