// tile_common.cuh -- device helpers shared by the TMA-fed kernels (tcgen05 TF32 and FP64 tensor
// path): mbarrier and bulk-tensor-copy wrappers, bounded waits, tile rasterisation and the
// mixed-radix slab arithmetic that maps a tile row or column to its place in C.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "kernels.hpp"

namespace tcontb {
namespace {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long global_timer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// One look at the barrier without waiting (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait.  Returns false (and raises the CTA's abort flag) when the limit passes, or
// immediately when another thread of the CTA already gave up.
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v)
{
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_shared_s64(uint32_t addr, long long v)
{
    asm volatile("st.shared.b64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ long long ld_shared_s64(uint32_t addr)
{
    long long v;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
    return v;
}

// Bounded wait.  The fast path is a bare try_wait; every 256 failed polls it looks at the CTA's
// abort flag (shared-memory word at `abort_addr`) and at the clock.  Returns false, and raises the
// flag, when the limit passes; returns false at once when another thread already gave up.
// `sleep_ns` > 0: the thread sleeps that long after a failed poll, for warps whose polling would
// otherwise take issue slots from the warps doing the arithmetic on the same scheduler.
// `limit_ns` = 0 means the default limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t abort_addr, uint32_t sleep_ns = 0,
                                          unsigned long long limit_ns = 0)
{
    const unsigned long long limit = limit_ns ? limit_ns : kWaitLimitNs;
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((spin & 255u) == 255u || spin == 0) {
            if (ld_shared_u32(abort_addr)) return false;
            if (spin == 0) continue;
            const unsigned long long now = global_timer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit) {
                st_shared_u32(abort_addr, 1u);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// Raster order: groups of `g` tile rows are swept column by column, so the CTAs that run
// together share A and B panels in L2.  Tile and slab counts fit 32 bits (the planner checks).
__device__ __forceinline__ void decode_tile(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t g, uint32_t* tm, uint32_t* tn)
{
    const uint32_t per_group = g * tiles_n;
    const uint32_t group = tile / per_group;
    const uint32_t first_m = group * g;
    const uint32_t rows = (tiles_m - first_m) < g ? (tiles_m - first_m) : g;
    const uint32_t local = tile - group * per_group;
    *tm = first_m + local % rows;
    *tn = local / rows;
}

// A unit of work: one tile, or with split-K one range of a tile's k iterations.  Units are numbered
// tile * k_splits + split.
struct WorkUnit {
    uint32_t tm, tn, split;
    int it0, n_it;
};
__device__ __forceinline__ WorkUnit decode_unit(uint32_t unit, const UmmaParams& p, uint32_t tiles_m, uint32_t tiles_n)
{
    WorkUnit w;
    const uint32_t splits = static_cast<uint32_t>(p.k_splits);
    const uint32_t tile = splits > 1 ? unit / splits : unit;
    w.split = splits > 1 ? unit - tile * splits : 0u;
    decode_tile(tile, tiles_m, tiles_n, static_cast<uint32_t>(p.raster_group), &w.tm, &w.tn);
    if (p.tn_rotate) w.tn = (w.tn + static_cast<uint32_t>(p.tn_rotate)) % tiles_n;
    w.it0 = static_cast<int>(w.split) * p.k_iters_per_split;
    w.n_it = p.k_iters - w.it0 < p.k_iters_per_split ? p.k_iters - w.it0 : p.k_iters_per_split;
    return w;
}

// Splits a slab index into its mixed-radix digits and returns the C offset of the slab start.
// valid = false when the slab lies beyond the tensor.
__device__ __forceinline__ long long slab_c_offset(const UmmaOperandDev& o, uint32_t slab, int* digit0, bool* valid)
{
    *valid = slab < static_cast<uint32_t>(o.total_slabs);
    uint32_t rem = slab;
    long long off = 0;
#pragma unroll
    for (int d = 0; d < kMaxTmaRank; ++d) {
        if (d < o.n_row_digits) {
            const uint32_t e = static_cast<uint32_t>(o.row_digit_ext[d]);
            const uint32_t idx = rem % e;
            rem /= e;
            off += static_cast<long long>(idx) * o.row_digit_cstride[d];
            if (d == o.chunk_digit) *digit0 = static_cast<int>(idx);
        }
    }
    return off;
}

// C offset of position `in` of a slab whose digit-0 index is `digit0`, relative to what slab_c_offset returned.
// With operand-level row fusion (split_inner > 0) the slab mode is two C modes, and digit 0 carries no C
// stride of its own: the position inside the fused mode is split here.
__device__ __forceinline__ long long slab_elem_offset(const UmmaOperandDev& o, int digit0, int in)
{
    if (o.split_inner > 0) {
        const int pos = digit0 * o.slab_w + in;
        return static_cast<long long>(pos % o.split_inner) * o.row_elem_cstride +
               static_cast<long long>(pos / o.split_inner) * o.split_outer_cstride;
    }
    return static_cast<long long>(in) * o.row_elem_cstride;
}

}  // namespace
}  // namespace tcontb
