// transpose.cu -- tensor permutation through a padded shared-memory tile, 16-byte vectors on
// both the read and the write side.
//
// Replaces the cuTT kernels the reference's TTGT route calls (external/cutt/src/cuttkernel.cu:
// transposeTiled :38-118, transposePacked :123-222, transposeTiledCopy :356-426).  It keeps
// cuTT's two ideas -- merge ranks that stay adjacent (external/cutt/src/cuttplan.cpp:63-126) and
// stage the (input-contiguous x output-contiguous) plane through shared memory -- but moves
// 16-byte vectors, uses 64-bit offsets, and is selected by the planner rather than by timing
// every candidate in prepare().
#include <algorithm>
#include <cstdint>

#include "kernels.hpp"

namespace tcontb {

bool make_transpose_params(int rank, const int64_t* src_extent, const int* perm, TransposeParams* out, const int64_t* src_stride)
{
    if (rank < 1 || rank > kMaxModes) return false;
    bool seen[kMaxModes] = {false};
    for (int i = 0; i < rank; ++i) {
        if (perm[i] < 0 || perm[i] >= rank || seen[perm[i]] || src_extent[i] <= 0) return false;
        seen[perm[i]] = true;
    }
    int64_t dst_stride_of_src[kMaxModes];
    int64_t s = 1;
    for (int i = 0; i < rank; ++i) {
        dst_stride_of_src[perm[i]] = s;
        s *= src_extent[perm[i]];
    }
    // Merge source modes j, j+1 that are also neighbours (same order) in the destination.
    int pos_in_dst[kMaxModes];
    for (int i = 0; i < rank; ++i) pos_in_dst[perm[i]] = i;
    // (the source may be a view into a larger tensor: its strides are then given, and two modes merge only
    // when the second also follows the first in the source's memory)
    int n = 0;
    int64_t st = 1, dense = 1;
    for (int j = 0; j < rank; ++j) {
        const int64_t sj = src_stride ? src_stride[j] : dense;
        if (n > 0 && pos_in_dst[j] == pos_in_dst[j - 1] + 1 && sj == out->src_stride[n - 1] * out->ext[n - 1]) {
            out->ext[n - 1] *= src_extent[j];
        } else {
            out->ext[n] = src_extent[j];
            out->src_stride[n] = sj;
            out->dst_stride[n] = dst_stride_of_src[j];
            ++n;
        }
        st *= src_extent[j];
        dense *= src_extent[j];
    }
    if (n > 0 && out->src_stride[0] != 1) return false;   // the kernels copy along a contiguous first mode
    out->rank = n;
    out->elements = st;
    return true;
}

namespace {

template <typename V>
struct VecOf;

constexpr int TILE = 64;

struct TileGeom {
    int d0;  // merged source mode that is fastest in the destination
    int64_t tiles0, tiles1;
    int t0, t1;  // tile extents along source mode 0 and along mode d0
};

template <>
struct VecOf<float> {
    using type = float4;
};
template <>
struct VecOf<double> {
    using type = double2;
};

// Leading mode preserved: plain row copies.  Every thread moves four vectors per round, the four loads issued
// before the first store so that four 16-byte requests per thread are in flight, and the index arithmetic is
// done in 32 bits when the tensor has fewer than 2^31 elements (64-bit division is emulated and was what the
// threads spent their time on: 0.67 of the copy bandwidth with one vector per round and 64-bit indices).
template <typename T, int VEC, typename I>
__global__ void __launch_bounds__(256) permute_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, TransposeParams p)
{
    constexpr int UNROLL = 4;
    const I vec_per_row = static_cast<I>(p.ext[0] / VEC);
    const I total = static_cast<I>(p.elements / VEC);
    const I step = static_cast<I>(gridDim.x) * blockDim.x;
    const int rank = p.rank;
    for (I v0 = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x; v0 < total; v0 += step * UNROLL) {
        using V = typename VecOf<T>::type;
        V val[UNROLL];
        T one[UNROLL];
        I dof[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const I v = v0 + static_cast<I>(u) * step;
            ok[u] = v < total;
            if (ok[u]) {
                I rem = v / vec_per_row;
                const I c = (v - rem * vec_per_row) * VEC;
                I so = c;
                dof[u] = c;
                for (int i = 1; i < rank; ++i) {
                    const I e = static_cast<I>(p.ext[i]);
                    const I q = rem / e;
                    const I idx = rem - q * e;
                    rem = q;
                    so += idx * static_cast<I>(p.src_stride[i]);
                    dof[u] += idx * static_cast<I>(p.dst_stride[i]);
                }
                if constexpr (VEC == 1) one[u] = __ldg(src + so);
                else val[u] = __ldg(reinterpret_cast<const V*>(src + so));
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (ok[u]) {
                if constexpr (VEC == 1) dst[dof[u]] = one[u];
                else *reinterpret_cast<V*>(dst + dof[u]) = val[u];
            }
        }
    }
}

// General case: a t0 x t1 plane over (source-fastest mode 0, destination-fastest mode d0)
// goes through shared memory; the remaining modes are spread over the grid.  The tile extents are
// chosen per launch so that whole tiles cover the two modes evenly (extent 72: one tile of 72, not
// 64 + 8), up to 96 elements of 4 bytes or 64 of 8 a side.
// FIXED: 64 x 64 tiles known at compile time (the loops unroll; 4 to 7 % faster where such tiles fit the extents well).
template <typename T, int VEC, bool FIXED>
__global__ void __launch_bounds__(256, sizeof(T) == 4 ? 8 : 6) permute_tiled_kernel(const T* __restrict__ src, T* __restrict__ dst, TransposeParams p,
                                                            TileGeom g)
{
    extern __shared__ __align__(16) unsigned char tile_raw[];
    T* tile = reinterpret_cast<T*>(tile_raw);   // [t1][t0 + 1]
    const int t0 = FIXED ? TILE : g.t0, t1 = FIXED ? TILE : g.t1;
    const int pitch = t0 + 1;
    int64_t t = blockIdx.x;
    const int64_t c0 = (t % g.tiles0) * t0;  // offset along source mode 0
    t /= g.tiles0;
    const int64_t r0 = (t % g.tiles1) * t1;  // offset along source mode d0
    t /= g.tiles1;
    int64_t sbase = 0, dbase = 0;
    for (int i = 1; i < p.rank; ++i) {
        if (i == g.d0) continue;
        const int64_t idx = t % p.ext[i];
        t /= p.ext[i];
        sbase += idx * p.src_stride[i];
        dbase += idx * p.dst_stride[i];
    }
    const int64_t e0 = p.ext[0], e1 = p.ext[g.d0];
    const int64_t s1 = p.src_stride[g.d0];  // source stride of mode d0
    const int64_t d0s = p.dst_stride[0];    // destination stride of source mode 0
    const int vpr0 = t0 / VEC, vpr1 = t1 / VEC;   // vectors per tile row, read side and write side

    // Slots (one vector each) are handled two at a time per thread, both global loads issued before either is used;
    // the kernel is held to 32 registers so that eight blocks share an SM (with 48 it lost a fifth of its rate).
    // slot / vpr by multiplication: exact for slot < 2^20 / vpr (at most 96 x 96 slots, vpr at most 96).
    const unsigned inv0 = (1u << 20) / static_cast<unsigned>(vpr0) + 1u, inv1 = (1u << 20) / static_cast<unsigned>(vpr1) + 1u;
    const int slots0 = t1 * vpr0, slots1 = t0 * vpr1;
    using V = typename VecOf<T>::type;
    for (int base = threadIdx.x; base < slots0; base += 2 * 256) {
        int at[2];
        bool ok[2];
        V val[2];
        T one[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int idx = base + u * 256;
            const int r = static_cast<int>((static_cast<unsigned>(idx) * inv0) >> 20), cv = (idx - r * vpr0) * VEC;
            ok[u] = idx < slots0 && r0 + r < e1 && c0 + cv < e0;
            at[u] = r * pitch + cv;
            if (ok[u]) {
                const T* ptr = src + sbase + (r0 + r) * s1 + (c0 + cv);
                if constexpr (VEC == 1) one[u] = __ldg(ptr);
                else val[u] = __ldg(reinterpret_cast<const V*>(ptr));
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (ok[u]) {
                if constexpr (VEC == 1) {
                    tile[at[u]] = one[u];
                } else {
                    const T* e = reinterpret_cast<const T*>(&val[u]);
#pragma unroll
                    for (int q = 0; q < VEC; ++q) tile[at[u] + q] = e[q];
                }
            }
        }
    }
    __syncthreads();
    for (int base = threadIdx.x; base < slots1; base += 2 * 256) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int idx = base + u * 256;
            const int c = static_cast<int>((static_cast<unsigned>(idx) * inv1) >> 20), rv = (idx - c * vpr1) * VEC;
            if (idx < slots1 && c0 + c < e0 && r0 + rv < e1) {
                T* ptr = dst + dbase + (c0 + c) * d0s + (r0 + rv);
                if constexpr (VEC == 1) {
                    *ptr = tile[rv * pitch + c];
                } else {
                    V out;
                    T* e = reinterpret_cast<T*>(&out);
#pragma unroll
                    for (int q = 0; q < VEC; ++q) e[q] = tile[(rv + q) * pitch + c];
                    *reinterpret_cast<V*>(ptr) = out;
                }
            }
        }
    }
}

template <typename T>
cudaError_t launch_typed(const T* src, T* dst, const TransposeParams& p, cudaStream_t stream)
{
    constexpr int VMAX = 16 / sizeof(T);
    if (p.elements == 0) return cudaSuccess;
    const bool aligned = (reinterpret_cast<uintptr_t>(src) % 16 == 0) && (reinterpret_cast<uintptr_t>(dst) % 16 == 0);
    // Find the merged source mode that is fastest in the destination.
    int d0 = 0;
    for (int i = 0; i < p.rank; ++i)
        if (p.dst_stride[i] == 1) d0 = i;
    if (d0 == 0) {
        bool strides_ok = true;   // (a view's rows must start on 16-byte boundaries for the vector loads)
        for (int i = 1; i < p.rank; ++i) strides_ok = strides_ok && p.src_stride[i] % VMAX == 0;
        const bool vec = aligned && strides_ok && p.ext[0] % VMAX == 0;
        const int64_t total = p.elements / (vec ? VMAX : 1);
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 4 * 256 - 1) / (4 * 256), int64_t(sms) * 16));
        const bool small = p.elements < (int64_t(1) << 31);
        if (vec && small) permute_rows_kernel<T, VMAX, uint32_t><<<blocks, 256, 0, stream>>>(src, dst, p);
        else if (vec) permute_rows_kernel<T, VMAX, int64_t><<<blocks, 256, 0, stream>>>(src, dst, p);
        else if (small) permute_rows_kernel<T, 1, uint32_t><<<blocks, 256, 0, stream>>>(src, dst, p);
        else permute_rows_kernel<T, 1, int64_t><<<blocks, 256, 0, stream>>>(src, dst, p);
        return cudaGetLastError();
    }
    bool strides_ok = true;
    for (int i = 1; i < p.rank; ++i) strides_ok = strides_ok && p.src_stride[i] % VMAX == 0;
    const bool vec = aligned && strides_ok && p.ext[0] % VMAX == 0 && p.ext[d0] % VMAX == 0;
    // whole tiles of (nearly) equal size along both modes, a multiple of the vector width
    constexpr int kTileMax = sizeof(T) == 4 ? 96 : TILE;
    const int64_t unit = vec ? VMAX : 1;
    // (an extent of up to kTileMax is one tile; longer ones are cut evenly into tiles of up to 64, which keep more
    // blocks on an SM: 8192 x 8192 floats move at 5.5 TB/s with 64-wide tiles against 4.7 with 96-wide ones)
    auto even_tile = [&](int64_t extent, int64_t* tiles) {
        *tiles = extent <= kTileMax ? 1 : (extent + TILE - 1) / TILE;
        const int64_t per = (extent + *tiles - 1) / *tiles;
        return static_cast<int>((per + unit - 1) / unit * unit);
    };
    TileGeom g;
    g.d0 = d0;
    g.t0 = even_tile(p.ext[0], &g.tiles0);
    g.t1 = even_tile(p.ext[d0], &g.tiles1);
    // fixed 64 x 64 tiles where they waste less than 45 % of their slots on these extents
    auto eff64 = [](int64_t e) { return double(e) / double((e + TILE - 1) / TILE * TILE); };
    const bool fixed = eff64(p.ext[0]) * eff64(p.ext[d0]) >= 0.55;
    if (fixed) {
        g.t0 = g.t1 = TILE;
        g.tiles0 = (p.ext[0] + TILE - 1) / TILE;
        g.tiles1 = (p.ext[d0] + TILE - 1) / TILE;
    }
    int64_t blocks = g.tiles0 * g.tiles1;
    for (int i = 1; i < p.rank; ++i)
        if (i != d0) blocks *= p.ext[i];
    if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
    const size_t smem = static_cast<size_t>(g.t1) * static_cast<size_t>(g.t0 + 1) * sizeof(T);   // at most 37 KB
    if (vec && fixed) permute_tiled_kernel<T, VMAX, true><<<static_cast<unsigned>(blocks), 256, smem, stream>>>(src, dst, p, g);
    else if (vec) permute_tiled_kernel<T, VMAX, false><<<static_cast<unsigned>(blocks), 256, smem, stream>>>(src, dst, p, g);
    else if (fixed) permute_tiled_kernel<T, 1, true><<<static_cast<unsigned>(blocks), 256, smem, stream>>>(src, dst, p, g);
    else permute_tiled_kernel<T, 1, false><<<static_cast<unsigned>(blocks), 256, smem, stream>>>(src, dst, p, g);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_transpose(const void* src, void* dst, const TransposeParams& p, int elem_bytes, cudaStream_t stream)
{
    if (elem_bytes == 4) return launch_typed(static_cast<const float*>(src), static_cast<float*>(dst), p, stream);
    if (elem_bytes == 8) return launch_typed(static_cast<const double*>(src), static_cast<double*>(dst), p, stream);
    return cudaErrorInvalidValue;
}

}  // namespace tcontb
