// planner.cpp -- see planner.hpp.
#include "planner.hpp"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

namespace tcontb {
namespace {

int find_char(const std::string& s, char c)
{
    const size_t p = s.find(c);
    return p == std::string::npos ? -1 : static_cast<int>(p);
}

bool has_duplicates(const std::string& s)
{
    for (size_t i = 0; i < s.size(); ++i)
        for (size_t j = i + 1; j < s.size(); ++j)
            if (s[i] == s[j]) return true;
    return false;
}

int index_of(const std::vector<int>& v, int x)
{
    for (size_t i = 0; i < v.size(); ++i)
        if (v[i] == x) return static_cast<int>(i);
    return -1;
}

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Builds the kernel-facing problem from mode strings of C, left and right.
// Returns 0 / 1 (invalid) / 3 (unsupported).
// `parC` / `parL` / `parR`: for a sub-tensor view, the extents of the tensor's modes in the parent it is a view of
// (by position; empty = the tensor is dense).
int build_problem(const std::string& mC, const std::string& mL, const std::string& mR, const std::string& ext_mode,
                  const std::vector<int64_t>& ext_val, int scalar_type, Problem* out, std::string* err,
                  const std::vector<int64_t>& parC = {}, const std::vector<int64_t>& parL = {}, const std::vector<int64_t>& parR = {})
{
    Problem p;
    p.scalar_type = scalar_type;
    auto extent_of = [&](char c) -> int64_t {
        const int i = find_char(ext_mode, c);
        return i < 0 ? -1 : ext_val[static_cast<size_t>(i)];
    };
    for (const std::string* s : {&mC, &mL, &mR}) {
        for (char c : *s) {
            const int64_t e = extent_of(c);
            if (e < 0) {
                *err = std::string("Missing extent for mode: ") + c;
                return 1;
            }
            if (e == 0) {
                *err = std::string("Extent of mode '") + c + "' must be positive";
                return 1;
            }
        }
        if (has_duplicates(*s)) {
            *err = "A mode appears twice in one tensor (traces/diagonals are not expressible)";
            return 3;
        }
        // Element counts are products of caller-supplied 64-bit extents: multiply with an overflow check
        // before anything derives strides, table sizes or allocations from them.
        int64_t n = 1;
        for (char c : *s) {
            const int64_t e = extent_of(c);
            if (e >= (int64_t(1) << 31) || __builtin_mul_overflow(n, e, &n) || n >= (int64_t(1) << 40)) {
                *err = "Tensor too large: extents must stay below 2^31 and a tensor below 2^40 elements";
                return 3;
            }
        }
    }
    // C's stride-1 mode decides which caller operand plays role A.
    p.swapped = !mC.empty() && find_char(mL, mC[0]) < 0 && find_char(mR, mC[0]) >= 0;
    const std::string& mA = p.swapped ? mR : mL;
    const std::string& mB = p.swapped ? mL : mR;

    std::string all;
    for (char c : mC + mA + mB)
        if (find_char(all, c) < 0) all.push_back(c);
    for (char c : all) {
        const bool inC = find_char(mC, c) >= 0, inA = find_char(mA, c) >= 0, inB = find_char(mB, c) >= 0;
        Mode m;
        m.names = std::string(1, c);
        m.extent = extent_of(c);
        if (inC && inA && inB) {
            *err = std::string("Mode '") + c + "' is in C, A and B: batch modes are not supported (the reference rejects them too)";
            return 3;
        }
        if (inC && !inA && !inB) {
            *err = std::string("Mode '") + c + "' of C is in neither input";
            return 3;
        }
        if (!inC && inA != inB) {
            *err = std::string("Mode '") + c + "' is in one input only and not in C (free reductions are not supported)";
            return 3;
        }
        m.group = inC ? (inA ? GROUP_M : GROUP_N) : GROUP_K;
        p.modes.push_back(m);
    }
    auto ids = [&](const std::string& s) {
        std::vector<int> v;
        for (char c : s) v.push_back(find_char(all, c));
        return v;
    };
    p.A = ids(mA);
    p.B = ids(mB);
    p.C = ids(mC);
    // Element strides, mode by mode, before anything is fused: the product of the extents in front of the mode, taken
    // from the parent where the tensor is a view of a larger one.
    const std::vector<int64_t>& parA = p.swapped ? parR : parL;
    const std::vector<int64_t>& parB = p.swapped ? parL : parR;
    auto set_strides = [&](const std::vector<int>& t, const std::vector<int64_t>& parent, int which, int64_t* span) -> bool {
        if (!parent.empty() && parent.size() != t.size()) return false;
        int64_t st = 1;
        for (size_t i = 0; i < t.size(); ++i) {
            Mode& m = p.modes[static_cast<size_t>(t[i])];
            (which == 0 ? m.sA : which == 1 ? m.sB : m.sC) = st;
            const int64_t e = parent.empty() ? m.extent : parent[i];
            if (e < m.extent || e >= (int64_t(1) << 31) || __builtin_mul_overflow(st, e, &st) || st >= (int64_t(1) << 40)) return false;
        }
        *span = st;
        return true;
    };
    int64_t spanA = 1, spanB = 1, spanC = 1;
    if (!set_strides(p.A, parA, 0, &spanA) || !set_strides(p.B, parB, 1, &spanB) || !set_strides(p.C, parC, 2, &spanC)) {
        *err = "Parent extents of a sub-tensor view must be given for every mode, be at least the view's extents and stay below 2^40 elements";
        return 1;
    }
    p.strided = !parC.empty() || !parL.empty() || !parR.empty();
    p.c_strided = !parC.empty();

    // Fuse y into x when y follows x immediately in every tensor that holds them.
    bool fused = true;
    while (fused) {
        fused = false;
        for (size_t x = 0; x < p.modes.size() && !fused; ++x) {
            for (size_t y = 0; y < p.modes.size() && !fused; ++y) {
                if (x == y || p.modes[x].group != p.modes[y].group) continue;
                if (p.modes[x].extent == 0 || p.modes[y].extent == 0) continue;
                bool ok = true;
                int which = 0;
                for (std::vector<int>* t : {&p.A, &p.B, &p.C}) {
                    const int ix = index_of(*t, static_cast<int>(x)), iy = index_of(*t, static_cast<int>(y));
                    if ((ix < 0) != (iy < 0)) ok = false;
                    else if (ix >= 0 && iy != ix + 1) ok = false;
                    else if (ix >= 0) {   // and y must follow x in memory too (a view may have gaps between them)
                        const Mode &mx = p.modes[x], &my = p.modes[y];
                        const int64_t sx = which == 0 ? mx.sA : which == 1 ? mx.sB : mx.sC, sy = which == 0 ? my.sA : which == 1 ? my.sB : my.sC;
                        if (sy != sx * mx.extent) ok = false;
                    }
                    ++which;
                }
                if (!ok) continue;
                p.modes[x].names += p.modes[y].names;
                p.modes[x].extent *= p.modes[y].extent;
                p.modes[y].extent = 0;  // tombstone
                for (std::vector<int>* t : {&p.A, &p.B, &p.C}) {
                    const int iy = index_of(*t, static_cast<int>(y));
                    if (iy >= 0) t->erase(t->begin() + iy);
                }
                fused = true;
            }
        }
    }
    // element counts of the views (what is read, written and computed); spans are what the strides cover
    auto count_of = [&](const std::vector<int>& t) {
        int64_t n = 1;
        for (int id : t) n *= p.modes[static_cast<size_t>(id)].extent;
        return n;
    };
    p.sizeA = count_of(p.A);
    p.sizeB = count_of(p.B);
    p.sizeC = count_of(p.C);
    p.spanA = spanA;
    p.spanB = spanB;
    p.spanC = spanC;

    for (int id : p.C) {
        if (p.modes[static_cast<size_t>(id)].group == GROUP_M) p.M.push_back(id);
        else p.N.push_back(id);
    }
    // K order: follow the operand whose stride-1 mode is contracted, so that operand's loads
    // run along memory; A decides when both or neither are.
    const bool a_kfirst = !p.A.empty() && p.modes[static_cast<size_t>(p.A[0])].group == GROUP_K;
    const bool b_kfirst = !p.B.empty() && p.modes[static_cast<size_t>(p.B[0])].group == GROUP_K;
    const std::vector<int>& korder = (!a_kfirst && b_kfirst) ? p.B : p.A;
    for (int id : korder)
        if (p.modes[static_cast<size_t>(id)].group == GROUP_K) p.K.push_back(id);
    for (int id : p.M) p.Mtot *= p.modes[static_cast<size_t>(id)].extent;
    for (int id : p.N) p.Ntot *= p.modes[static_cast<size_t>(id)].extent;
    for (int id : p.K) p.Ktot *= p.modes[static_cast<size_t>(id)].extent;
    *out = p;
    return 0;
}

// Fills one operand's staging description. `t` = tensor mode list, `rows` = its row modes in C
// order, `tile_rows` = 128 for A, BN for B.
bool stage_operand(const Problem& p, const std::vector<int>& t, const std::vector<int>& rows, bool is_a, int kc_mode,
                   int BK, UmmaOperand* o, std::string* why)
{
    const int elt = p.scalar_type == 1 ? 8 : 4, W = 128 / elt;  // W = elements per 128-byte swizzle row
    o->rank = static_cast<int>(t.size());
    for (int d = 0; d < kMaxTmaRank; ++d) {
        o->ext[d] = 1;
        o->box[d] = 1;
        o->stride[d] = 0;
    }
    const int64_t s = is_a ? p.spanA : p.spanB;  // elements the strides cover (the parent's, for a view)
    for (int d = 0; d < o->rank; ++d) {
        const Mode& m = p.modes[static_cast<size_t>(t[static_cast<size_t>(d)])];
        o->ext[d] = m.extent;
        o->stride[d] = is_a ? m.sA : m.sB;
        if (m.extent >= (int64_t(1) << 31)) {
            *why = "a mode extent does not fit a TMA dimension";
            return false;
        }
        if (d > 0 && (o->stride[d] * elt) % 16 != 0) {
            *why = "a stride is not a multiple of 16 bytes (TMA global strides)";
            return false;
        }
    }
    if (o->rank > 0 && o->stride[0] != 1) {
        *why = "the first mode is not contiguous";
        return false;
    }
    const int64_t pad = (s + 3) / 4 * 4;  // (any multiple of 16 bytes will do)
    for (int d = o->rank; d < kMaxTmaRank; ++d) o->stride[d] = pad;  // padded unit dims
    if (s * elt >= (int64_t(1) << 40)) {
        *why = "tensor too large for TMA strides";
        return false;
    }
    const int first = t[0];
    o->major = p.modes[static_cast<size_t>(first)].group == GROUP_K ? 0 : 1;
    o->kc_dim = index_of(t, kc_mode);
    int slab_mode;
    if (o->major == 1) {
        slab_mode = first;
        o->slab_w = W;
        // FP64: slabs of 8 doubles (64-byte rows, 64-byte swizzle) where 16 would pad the mode by over 8 %
        // (extent 72: 5 x 16 = 80 against 9 x 8)
        const int64_t e = p.modes[static_cast<size_t>(first)].extent;
        if (elt == 8 && double(ceil_div(e, 16) * 16) > 1.08 * double(ceil_div(e, 8) * 8)) o->slab_w = 8;
    } else {
        if (first != kc_mode) {
            *why = "K-major operand whose stride-1 mode is not the chunked K mode";
            return false;
        }
        slab_mode = rows[0];
        o->slab_w = 8;  // refined by the caller once the tile height is known
    }
    o->slab_dim = index_of(t, slab_mode);
    const Mode& sm = p.modes[static_cast<size_t>(slab_mode)];
    o->slab_mode_ext = sm.extent;
    o->row_elem_cstride = sm.sC;
    (void)is_a;
    (void)BK;
    return true;
}

// `lead_mode` >= 0: that row mode becomes digit 0 of the slab index, in front of the chunk digit, so that the
// slabs of a tile are consecutive indices of it (see rows_across_slabs).
void finish_operand(const Problem& p, const std::vector<int>& t, const std::vector<int>& rows, int tile_rows, int BK,
                    const std::vector<int>& kdigits, UmmaOperand* o, int max_slab_rows = 256, int lead_mode = -1)
{
    const int elt = p.scalar_type == 1 ? 8 : 4, W = 128 / elt;
    if (o->major == 0) {
        // K-major: rows per slab = the largest power of two (8..tile height) that pads the slab
        // mode by at most 15 % (TF32, where fewer and larger TMA boxes matter more) or 3 % (FP64,
        // where padded rows cost FP64 tensor time); failing that, the one that pads least.
        const double limit = p.scalar_type == 1 ? 1.03 : 1.15;
        int best = 8;
        double best_waste = 1e30;
        for (int w = 8; w <= tile_rows && w <= max_slab_rows; w *= 2) {
            const double waste = double(ceil_div(o->slab_mode_ext, w) * w) / double(o->slab_mode_ext);
            const bool ok = waste <= limit, best_ok = best_waste <= limit;
            if ((ok && (!best_ok || w > best)) || (!ok && !best_ok && waste < best_waste - 1e-12)) {
                best = w;
                best_waste = waste;
            }
        }
        if (tile_rows / best > 16) best = tile_rows / 16;  // at most 16 slabs per operand tile
        o->slab_w = best;
    }
    o->slabs_per_tile = tile_rows / o->slab_w;
    const int slab_mode = t[static_cast<size_t>(o->slab_dim)];
    o->n_row_digits = 0;
    o->chunk_digit = 0;
    o->total_slabs = 1;
    if (lead_mode >= 0) {
        const Mode& m = p.modes[static_cast<size_t>(lead_mode)];
        o->row_digit_dim[0] = index_of(t, lead_mode);
        o->row_digit_ext[0] = m.extent;
        o->row_digit_cstride[0] = m.sC;
        o->n_row_digits = 1;
        o->chunk_digit = 1;
        o->total_slabs = m.extent;
    }
    {
        const int n = o->n_row_digits++;
        o->row_digit_dim[n] = o->slab_dim;
        o->row_digit_ext[n] = ceil_div(o->slab_mode_ext, o->slab_w);
        o->row_digit_cstride[n] = o->row_elem_cstride * o->slab_w;
        o->total_slabs *= o->row_digit_ext[n];
    }
    for (int id : rows) {
        if (id == slab_mode || id == lead_mode) continue;
        const Mode& m = p.modes[static_cast<size_t>(id)];
        const int n = o->n_row_digits++;
        o->row_digit_dim[n] = index_of(t, id);
        o->row_digit_ext[n] = m.extent;
        o->row_digit_cstride[n] = m.sC;
        o->total_slabs *= m.extent;
    }
    for (int i = 0; i < 3; ++i)
        o->k_digit_dim[i] = i < static_cast<int>(kdigits.size()) ? index_of(t, kdigits[static_cast<size_t>(i)]) : -1;
    if (o->major == 1) {
        o->box[o->slab_dim] = o->slab_w;
        o->box[o->kc_dim] = BK;
        o->slab_bytes = BK * o->slab_w * elt;
    } else {
        o->box[o->kc_dim] = BK;  // = W except for FP64 with a k chunk of 8: 64-byte rows
        o->box[o->slab_dim] = o->slab_w;
        o->slab_bytes = o->slab_w * BK * elt;
    }
    o->slabs_per_op = 1;
    o->k0_scale = BK;
    o->digit0_scale = o->slab_w;
    o->oob_coord = static_cast<int>(ceil_div(o->slab_mode_ext, W) * W);  // (any coordinate past the mode's end)
}

// Merged boxes for an MN-major operand: the slab mode (stride-1, extent a multiple of 32) is
// presented to TMA as two dimensions (32 contiguous elements, extent/32 chunks), ordered
// (lo, chunked K mode, hi, rest...), so that one copy with box {32, BK, g} lands g whole slabs one
// after the other.  Fewer, larger copies: the 4 KB single-slab boxes kept the copy engine busy
// with per-copy overhead (GEMM 8192x8192x4096 on B200: 377 TFLOP/s with 12 copies per stage
// against 615 with 2).  `cta_slabs` = slabs of this operand one CTA stages per K step.
void merge_slabs(UmmaOperand* o, int BK, int cta_slabs)
{
    const int W = o->slab_w;  // 32 floats or 16 doubles
    if (o->major != 1 || o->rank > kMaxTmaRank - 1 || o->slab_dim != 0 || o->slab_mode_ext % W || o->slabs_per_op > 1) return;
    const int64_t chunks = o->slab_mode_ext / W;
    int g = 1;
    while (g * 2 <= cta_slabs && chunks % (g * 2) == 0 && cta_slabs % (g * 2) == 0) g *= 2;
    if (g <= 1) return;
    UmmaOperand n = *o;
    int map[kMaxTmaRank];
    for (int d = 0; d < kMaxTmaRank; ++d) map[d] = -1;
    n.ext[0] = W; n.stride[0] = 1;
    n.ext[1] = o->ext[o->kc_dim]; n.stride[1] = o->stride[o->kc_dim];
    n.ext[2] = chunks; n.stride[2] = W;
    map[0] = 2;
    map[o->kc_dim] = 1;
    int next = 3;
    for (int d = 1; d < o->rank; ++d) {
        if (d == o->kc_dim) continue;
        n.ext[next] = o->ext[d];
        n.stride[next] = o->stride[d];
        map[d] = next++;
    }
    const int64_t total = o->stride[kMaxTmaRank - 1];  // padded dims carry the tensor's element count
    for (int d = next; d < kMaxTmaRank; ++d) { n.ext[d] = 1; n.stride[d] = total; }
    n.rank = o->rank + 1;
    for (int d = 0; d < kMaxTmaRank; ++d) n.box[d] = 1;
    n.box[0] = W; n.box[1] = BK; n.box[2] = g;
    n.slab_dim = 2;
    n.kc_dim = 1;
    for (int i = 0; i < o->n_row_digits; ++i) n.row_digit_dim[i] = map[o->row_digit_dim[i]];
    for (int i = 0; i < 3; ++i) n.k_digit_dim[i] = o->k_digit_dim[i] >= 0 ? map[o->k_digit_dim[i]] : -1;
    n.slabs_per_op = g;
    n.digit0_scale = 1;
    n.oob_coord = static_cast<int>(chunks);
    *o = n;
}

// How much slabs of 16 or 8 doubles pad a stride-1 mode of extent e.
double slab_padding_f64(int64_t e)
{
    return double(std::min(ceil_div(e, 16) * 16, ceil_div(e, 8) * 8)) / double(e);
}

// K-major operand with a k chunk of 64 (two 128-byte rows of k per tile row): the chunked mode is shown to TMA
// as two dimensions (32 contiguous elements, extent / 32 chunks), the chunk dimension last, so that ONE copy
// with box {32, rows, ..., 2} lands the two 32-wide K chunks of the slab one after the other, each a canonical
// K-major tile of `rows` x 128 bytes.  Needs a free tensor-map dimension, an extent that is a multiple of 32
// (a ragged last chunk would read the next row's elements instead of zeros) and one slab per CTA (the rows of
// a chunk must be contiguous in shared memory for the MMA descriptor).
bool chunk_kmajor(UmmaOperand* o, int BK, int cta_slabs)
{
    if (o->major != 0 || BK <= 32) return true;
    if (o->rank >= kMaxTmaRank || o->kc_dim != 0 || o->ext[0] % 32 || cta_slabs != 1) return false;
    const int r = o->rank;
    o->ext[r] = o->ext[0] / 32;
    o->stride[r] = 32;
    o->box[r] = BK / 32;
    o->ext[0] = 32;
    o->box[0] = 32;
    o->rank = r + 1;
    o->k_digit_dim[0] = r;
    o->k0_scale = BK / 32;
    return true;
}

void plan_umma_impl(const Problem& p_in, const CostTable& cost, UmmaSpec* u, int bk_request)
{
    u->eligible = false;
    const bool f64 = p_in.scalar_type == 1;
    // Operand-level row fusion (FP64 kernel, whose epilogue takes every row's C offset from a table): when the
    // stride-1 mode of an MN-major operand is so short that whole slabs would pad it by over 8 % (extent 6:
    // a quarter of every 8-row slab empty) and the next row mode in C's order follows it directly in the
    // operand, the two are staged as ONE mode: TMA sees a single dimension of the fused extent, tiles have no
    // empty rows, and the table builder splits a row's position back into the two C modes.
    Problem p = p_in;
    int64_t split_inner[2] = {0, 0}, split_outer_cstride[2] = {0, 0};
    if (f64 && !std::getenv("TCONT_NO_ROW_FUSION")) {
        for (int which = 0; which < 2; ++which) {
            std::vector<int>& t = which == 0 ? p.A : p.B;
            std::vector<int>& rows = which == 0 ? p.M : p.N;
            if (t.size() < 3 || rows.size() < 2 || t[0] != rows[0] || t[1] != rows[1]) continue;
            const Mode m0 = p.modes[static_cast<size_t>(t[0])], m1 = p.modes[static_cast<size_t>(t[1])];
            if (slab_padding_f64(m0.extent) <= 1.08) continue;
            if ((which == 0 ? m1.sA : m1.sB) != (which == 0 ? m0.sA : m0.sB) * m0.extent) continue;  // (a view with a gap between them)
            Mode f;
            f.names = m0.names + m1.names;
            f.extent = m0.extent * m1.extent;
            f.group = m0.group;
            f.sA = m0.sA;
            f.sB = m0.sB;
            f.sC = m0.sC;
            const int id = static_cast<int>(p.modes.size());
            p.modes.push_back(f);
            split_inner[which] = m0.extent;
            split_outer_cstride[which] = m1.sC;
            t[0] = id;
            t.erase(t.begin() + 1);
            rows[0] = id;
            rows.erase(rows.begin() + 1);
        }
    }
    const int elt = f64 ? 8 : 4, W = 128 / elt;
    u->elt = elt;
    if (const char* k = std::getenv("TCONT_KERNEL")) {
        // Debug switch: TCONT_KERNEL=gather keeps FP64 on the cp.async gather kernel.
        if (f64 && std::strcmp(k, "gather") == 0) { u->why_not = "disabled by TCONT_KERNEL=gather"; return; }
        // Debug switch: TCONT_KERNEL=simt keeps Float32 contractions on the CUDA-core kernel.
        if (std::strcmp(k, "simt") == 0) { u->why_not = "disabled by TCONT_KERNEL=simt"; return; }
    }
    if (p.A.size() < 2 || p.B.size() < 2 || p.A.size() > kMaxTmaRank || p.B.size() > kMaxTmaRank) {
        u->why_not = "operand rank outside 2..5 after fusion";
        return;
    }
    if (p.M.empty() || p.N.empty() || p.K.empty() || p.K.size() > 3) {
        u->why_not = "needs M, N and 1..3 K modes";
        return;
    }
    const bool a_kmajor = p.modes[static_cast<size_t>(p.A[0])].group == GROUP_K;
    const bool b_kmajor = p.modes[static_cast<size_t>(p.B[0])].group == GROUP_K;
    int kc;
    if (a_kmajor && b_kmajor) {
        if (p.A[0] != p.B[0]) { u->why_not = "both operands K-major on different modes"; return; }
        kc = p.A[0];
    } else if (a_kmajor) kc = p.A[0];
    else if (b_kmajor) kc = p.B[0];
    else {
        // Both operands MN-major: any contracted mode may be the one cut into BK-row chunks.  The
        // rows of a TMA box are one stride of that mode apart; far-apart rows (a slow mode) cost
        // DRAM-page and TLB locality, and the B tile is up to twice as tall as the A tile, so weigh
        // log2(stride) by the tile height.  (cfg5 on B200: 446 TFLOP/s with B's fast K mode chunked,
        // 274 with A's.)
        kc = p.K[0];
        double best = 1e300;
        for (int id : p.K) {
            const Mode& m = p.modes[static_cast<size_t>(id)];
            const double cost = 128.0 * std::log2(double(m.sA)) + 256.0 * std::log2(double(m.sB));
            if (cost < best) {
                best = cost;
                kc = id;
            }
        }
        // Tuning switch: TCONT_UMMA_KC=<mode letter> picks the contracted mode that is cut into
        // BK-sized chunks when both operands are MN-major (any K mode is legal then).
        if (const char* want = std::getenv("TCONT_UMMA_KC"))
            for (int id : p.K)
                if (p.modes[static_cast<size_t>(id)].names.find(want[0]) != std::string::npos) kc = id;
    }
    const int64_t kc_ext = p.modes[static_cast<size_t>(kc)].extent;
    u->kc_names = p.modes[static_cast<size_t>(kc)].names;
    int BK = W;  // a K-major operand brings 128 bytes of K per row
    // Both operands MN-major: the k chunk may be narrower than a 128-byte row.  FP64 takes 8 instead of
    // 16 where that spares more than 15 % of zero-filled k (24 = 3 x 8 against 2 x 16).
    // (A K-major FP64 operand then has 64-byte rows under the 64-byte swizzle; the tcgen05 kernel keeps
    // 128-byte rows for K-major operands.)
    if (f64) BK = kc_ext <= 8 || double(ceil_div(kc_ext, 16) * 16) > 1.15 * double(ceil_div(kc_ext, 8) * 8) ? 8 : 16;
    else if (!a_kmajor && !b_kmajor) {
        BK = kc_ext <= 8 ? 8 : kc_ext <= 16 ? 16 : 32;
        // chunks of 24 (three MMAs per stage) where 32 would pad the mode by over 15 % and 24 by nothing: extents 24, 72, 120
        if (kc_ext % 24 == 0 && double(ceil_div(kc_ext, 32) * 32) > 1.15 * double(kc_ext) && !std::getenv("TCONT_UMMA_NO_BK24")) BK = 24;
    }
    // A k chunk of 64 (eight MMAs per stage, stages of 64 KB per CTA of a pair): half the barrier round trips and
    // half the copy instructions per flop.  The producer warp needs 700 to 900 cycles per stage for its
    // wait / announce / copy sequence whatever the stage holds, which is more than the 512 cycles four MMAs take
    // and less than the 1 024 of eight.  Only where it pads the chunked mode by at most a tenth more.
    if (!f64 && bk_request == 64 && BK == 32 && kc_ext >= 64 &&
        double(ceil_div(kc_ext, 64) * 64) <= 1.1 * double(ceil_div(kc_ext, 32) * 32))
        BK = 64;
    u->BK = BK;
    std::vector<int> kdigits{kc};
    for (int id : p.K)
        if (id != kc) kdigits.push_back(id);
    u->n_k_digits = static_cast<int>(kdigits.size());
    u->k_iters = 1;
    for (int i = 0; i < 3; ++i) u->k_digit_ext[i] = 1;
    for (size_t i = 0; i < kdigits.size(); ++i) {
        const int64_t e = p.modes[static_cast<size_t>(kdigits[i])].extent;
        u->k_digit_ext[i] = i == 0 ? ceil_div(e, BK) : e;
        u->k_iters *= u->k_digit_ext[i];
    }
    if (!stage_operand(p, p.A, p.M, true, kc, BK, &u->a, &u->why_not)) return;
    if (!stage_operand(p, p.B, p.N, false, kc, BK, &u->b, &u->why_not)) return;

    u->BM = 128;
    finish_operand(p, p.A, p.M, u->BM, BK, kdigits, &u->a);
    // Rows across slabs (FP64 kernel): A is MN-major on a mode that is not C's stride-1 mode (reference cases 3,
    // 4, 6-8: C[a,...] from A[d,...,a]).  Rows that run along A's stride-1 mode alone would be stored element by
    // element, and moving a 200-300 MB A through a transpose first costs more than the contraction.  Instead a
    // tile is 8 slabs of 16 rows: 16 consecutive elements of A's stride-1 mode (one 128-byte TMA row) times 8
    // consecutive indices of C's stride-1 mode, fetched by ONE box that spans both modes, and a thread stores
    // the same row of four neighbouring slabs as one 32-byte piece of C.  Needs C's stride-1 mode behind the
    // chunked contracted mode in A's memory order (the box then lands slab by slab) and an extent that is a
    // multiple of 8 (a tile never wraps to the next chunk).
    int lead_a = -1;
    if (f64 && u->a.major == 1 && u->a.row_elem_cstride != 1 && split_inner[0] == 0 && !p.M.empty() && !std::getenv("TCONT_NO_ROWS_ACROSS_SLABS")) {
        const int c1 = p.M[0];
        const Mode& m1 = p.modes[static_cast<size_t>(c1)];
        const int dim1 = index_of(p.A, c1);
        if (m1.sC == 1 && dim1 > u->a.kc_dim && dim1 != u->a.slab_dim && m1.extent % 8 == 0) {
            lead_a = c1;
            u->a.slab_w = 16;
            finish_operand(p, p.A, p.M, u->BM, BK, kdigits, &u->a, 256, lead_a);
            u->a.box[dim1] = u->a.slabs_per_tile;   // one copy per stage: 8 slabs = 8 indices of C's stride-1 mode
            u->a.slabs_per_op = u->a.slabs_per_tile;
            u->store_across_slabs = true;
        }
    }
    u->tiles_m = ceil_div(u->a.total_slabs, u->a.slabs_per_tile);
    // N tile: the widest of 256/128/64/32 that is not wider than the (padded) N extent needs and
    // still yields at least one tile per SM; otherwise the narrowest admissible one.
    int bn = 32;
    if (f64) {
        // the FP64 kernel has 128 x 64 and 128 x 32 tiles: the narrow one where it pads N by over 15 % less
        UmmaOperand probe = u->b;
        finish_operand(p, p.B, p.N, 32, BK, kdigits, &probe);
        const int64_t padded = probe.total_slabs * probe.slab_w;
        bn = double(ceil_div(padded, 32) * 32) * 1.15 < double(ceil_div(padded, 64) * 64) ? 32 : 64;
    } else {
        UmmaOperand probe = u->b;
        finish_operand(p, p.B, p.N, 32, BK, kdigits, &probe);
        const int64_t padded = probe.total_slabs * probe.slab_w;
        int widest = 32;
        while (widest < 256 && widest < padded) widest *= 2;
        bn = widest;
        for (int cand = widest; cand >= 32; cand /= 2) {
            UmmaOperand tmp = u->b;
            finish_operand(p, p.B, p.N, cand, BK, kdigits, &tmp);
            if (tmp.slabs_per_tile < 1) break;
            bn = cand;
            if (u->tiles_m * ceil_div(tmp.total_slabs, tmp.slabs_per_tile) >= cost.num_sms) break;
        }
    }
    u->BN = bn;
    finish_operand(p, p.B, p.N, u->BN, BK, kdigits, &u->b);
    if (u->b.slabs_per_tile < 1 || u->a.slabs_per_tile + u->b.slabs_per_tile > 32) {
        u->why_not = "too many slabs per stage";
        return;
    }
    u->tiles_n = ceil_div(u->b.total_slabs, u->b.slabs_per_tile);
    if (u->tiles_m * u->tiles_n >= (int64_t(1) << 31) || (u->tiles_m + 1) * u->a.slabs_per_tile >= (int64_t(1) << 31) ||
        (u->tiles_n + 1) * u->b.slabs_per_tile >= (int64_t(1) << 31)) {
        u->why_not = "tile or slab count does not fit 32 bits";
        return;
    }
    // Two-CTA pairs (256-row tiles): each CTA stages its own 128 rows of A and half of the B tile,
    // so B must split into an even number of slabs.  TCONT_UMMA_PAIR=1 selects it.
    {
        UmmaOperand b2 = u->b;
        if (b2.major == 0 && b2.slabs_per_tile % 2) finish_operand(p, p.B, p.N, u->BN, BK, kdigits, &b2, u->BN / 2);
        const int64_t tn2 = ceil_div(b2.total_slabs, b2.slabs_per_tile);
        // (a short K loop is output-bound: pairing buys nothing there and costs the cluster handshakes)
        // Measured on B200 the pair kernel does not beat one CTA per tile (GEMM 8192x8192x4096: 580 vs
        // 605 TFLOP/s; cfg5: 455 vs 526): the MMA of a pair reads half of B from the partner SM and issues
        // more slowly, which eats the saving in copies.  It therefore stays opt-in.
        // With a k chunk of 64 the pair is the point: 64 KB per CTA per stage is what the 64 B/clk an SM takes in
        // from L2 delivers in the 1 024 cycles the stage's eight MMAs need, where one CTA per 128 x 256 tile would
        // need 96 KB.  Taken when there are at least two waves of pairs and four stages of k.
        bool pair = false;
        if (f64) b2 = u->b;
        const bool can_pair = !f64 && u->tiles_m >= 2 && b2.slabs_per_tile % 2 == 0;
        if (BK == 64) pair = can_pair && u->BN == 256 && ceil_div(u->tiles_m, 2) * tn2 >= cost.num_sms && u->k_iters >= 4;
        if (const char* e = std::getenv("TCONT_UMMA_PAIR")) {
            if (e[0] == '0') pair = false;
            else if (e[0] == '1') pair = can_pair;
        }
        if (BK == 64 && !pair) {
            u->why_not = "a k chunk of 64 is only used by CTA pairs";
            return;
        }
        if (pair) {
            u->pair = true;
            u->b = b2;
            u->tiles_n = tn2;
        }
    }
    {
        const double a_bytes = double(u->a.slabs_per_tile) * u->a.slab_bytes;
        const double b_bytes = double(u->b.slabs_per_tile) * u->b.slab_bytes;
        // rows of a box that lie in different 2 MB pages
        const bool a_far = u->a.major == 1 && u->a.stride[u->a.kc_dim] * elt >= (int64_t(2) << 20);
        const bool b_far = u->b.major == 1 && u->b.stride[u->b.kc_dim] * elt >= (int64_t(2) << 20);
        u->far_fraction = ((a_far ? a_bytes : 0.0) + (b_far ? b_bytes : 0.0)) / (a_bytes + b_bytes);
    }
    if (!chunk_kmajor(&u->a, BK, u->a.slabs_per_tile) ||
        !chunk_kmajor(&u->b, BK, u->pair ? u->b.slabs_per_tile / 2 : u->b.slabs_per_tile)) {
        u->why_not = "a K-major operand cannot be staged with a k chunk of 64";
        return;
    }
    if (!std::getenv("TCONT_UMMA_NO_MERGE")) {
        merge_slabs(&u->a, BK, u->a.slabs_per_tile);
        merge_slabs(&u->b, BK, u->pair ? u->b.slabs_per_tile / 2 : u->b.slabs_per_tile);
    }
    const int stage_bytes = u->a.slabs_per_tile * u->a.slab_bytes +
                            (u->pair ? u->b.slabs_per_tile / 2 : u->b.slabs_per_tile) * u->b.slab_bytes;
    // both kernels own an SM; the FP64 one stops at eight 24 KB stages
    const int budget = f64 ? 200 * 1024 : 227 * 1024 - 8 * 1024;
    u->stages = std::max(2, std::min(8, budget / stage_bytes));
    if (f64) u->stages &= ~1;  // one ring of stages per consumer group
    // One CTA per tile (k chunks of up to 32: a stage is at most four MMAs, 512 cycles): two producer warps take
    // turns stage by stage, because one warp's wait-announce-copy round trip takes 700 to 900 cycles whatever the
    // stage holds (reference cases 13, 15, 21, 24 in TF32: 1.24 to 1.67 times faster; nothing to gain with one k
    // iteration per tile).  CTA pairs keep one producer and stages of 64 k (two producers on half-size stages were
    // measured slower there: 0.297 against 0.248 ms on the 3-D configuration).  TCONT_UMMA_PRODUCERS=1|2 overrides.
    if (!f64 && !u->pair && u->stages >= 4 && u->k_iters >= 2) u->producers = 2;
    if (const char* e = std::getenv("TCONT_UMMA_PRODUCERS"))
        if (!f64) u->producers = std::atoi(e) == 2 && u->stages >= 4 ? 2 : 1;
    if (u->producers == 2) u->stages &= ~1;
    u->smem_bytes = u->stages * stage_bytes + 8 * 1024 + 1024;
    // Split-K: with few waves of tiles and a long contracted extent, cut the k iterations into ranges
    // computed as separate work units (partials summed by a second kernel).  Of the admissible counts
    // (ranges of at least 4 iterations, workspace of at most 512 MB) the one with the smallest estimate
    // wins: arithmetic over the share of the last wave's SMs that have a unit, plus the partials written
    // and read back.  A wave is one unit per SM for the tcgen05 kernel (per SM pair for CTA pairs) and two for the FP64 kernel, which
    // wants a unit for each of its two consumer groups.
    {
        const int64_t tiles = (u->pair ? ceil_div(u->tiles_m, 2) : u->tiles_m) * u->tiles_n;
        const int64_t wave = f64 ? 2 * cost.num_sms : u->pair ? cost.num_sms / 2 : cost.num_sms;
        const double flops = 2.0 * double(u->tiles_m * u->BM) * double(u->tiles_n * u->BN) * double(u->k_iters * u->BK);
        const double rate = (f64 ? cost.dmma_f64_tflops : cost.umma_tf32_tflops) * 1e6;  // flops per microsecond
        // The tcgen05 kernel's ring advances by one stage per `umma_stage_us` at best, whatever the stage holds (the
        // producer's wait-announce-copy round trip): a work unit takes at least its stages times that, which is what
        // a long k loop on narrow tiles costs, not its flops.
        auto estimate = [&](int64_t s) {
            const int64_t units = tiles * s;
            const int64_t rounds = ceil_div(units, wave);
            const double eff = double(units) / double(rounds * wave);
            double t = flops / (rate * eff);
            if (!f64) t = std::max(t, double(rounds) * double(ceil_div(u->k_iters, s)) * cost.umma_stage_us / u->producers);
            return t + (s > 1 ? cost.launch_us + 2.0 * double(s) * double(p.sizeC) * elt / (cost.hbm_gbs * 1e3) : 0.0);
        };
        int64_t splits = 1;
        // (a C that is a view into a larger tensor has no workspace "laid out like C" to add partial tiles up in)
        if (tiles < 4 * wave && u->k_iters >= 8 && !p.c_strided) {
            double best = estimate(1);
            for (int64_t s = 2; s <= std::min<int64_t>(64, u->k_iters / 4); ++s) {
                if (double(s) * double(p.sizeC) * elt > 512.0 * 1024 * 1024) break;  // workspace
                const double e = estimate(s);
                if (e < 0.97 * best) best = e, splits = s;  // (a split has to pay for its second kernel)
            }
        }
        if (const char* e = std::getenv("TCONT_SPLITK")) {
            splits = p.c_strided ? 1 : std::max<int64_t>(1, std::min<int64_t>(std::atoll(e), u->k_iters));
            while (splits > 1 && double(splits) * double(p.sizeC) * elt > 512.0 * 1024 * 1024) --splits;
        }
        u->k_iters_per_split = ceil_div(u->k_iters, splits);
        u->k_splits = static_cast<int>(ceil_div(u->k_iters, u->k_iters_per_split));
    }
    u->raster_group = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(u->tiles_m,
                      std::llround(std::sqrt(double(cost.num_sms) * u->BN / u->BM)))));
    // Tuning switch: TCONT_UMMA_RASTER=<g> sets the number of tile rows (pair rows for CTA pairs) swept together.
    if (const char* e = std::getenv("TCONT_UMMA_RASTER"))
        u->raster_group = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(u->tiles_m, std::atoll(e))));
    // fused row modes: digit 0 carries no C stride of its own, the kernel splits the position (slab_elem_offset)
    for (int which = 0; which < 2; ++which) {
        UmmaOperand& o = which == 0 ? u->a : u->b;
        if (split_inner[which] > 0) {
            o.split_inner = split_inner[which];
            o.split_outer_cstride = split_outer_cstride[which];
            o.row_digit_cstride[0] = 0;
        }
    }
    u->eligible = true;
}

// The tcgen05 kernel is planned twice where that can pay: with a k chunk of 64 on CTA pairs, and, where that
// form does not apply (short or ragged contracted mode, too few tiles, a B tile that does not split), with the
// 32-wide chunk on one CTA per tile.  TCONT_UMMA_BK=32 and TCONT_UMMA_PAIR=0 keep the second form.
void plan_umma(const Problem& p, const CostTable& cost, UmmaSpec* u)
{
    const char* bk = std::getenv("TCONT_UMMA_BK");
    const char* pr = std::getenv("TCONT_UMMA_PAIR");
    if (p.scalar_type != 1 && !(bk && std::atoi(bk) == 32) && !(pr && pr[0] == '0')) {
        UmmaSpec v;
        plan_umma_impl(p, cost, &v, 64);
        if (v.eligible && v.BK == 64) {
            *u = v;
            return;
        }
    }
    *u = UmmaSpec();
    plan_umma_impl(p, cost, u, 32);
}

std::string perm_modes(const Problem& p, const std::vector<int>& ids)
{
    std::string s;
    for (int id : ids) s += p.modes[static_cast<size_t>(id)].names;
    return s;
}

void fill_transpose(const std::string& src, const std::string& dst, const std::string& ext_mode,
                    const std::vector<int64_t>& ext_val, TransposeSpec* t, const std::vector<int64_t>& src_parent = {})
{
    t->needed = src != dst;
    t->rank = static_cast<int>(src.size());
    t->elements = 1;
    t->strided_src = !src_parent.empty();
    int64_t st = 1;
    for (size_t i = 0; i < src.size(); ++i) {
        t->src_extent[i] = ext_val[static_cast<size_t>(find_char(ext_mode, src[i]))];
        t->elements *= t->src_extent[i];
        t->perm[i] = find_char(src, dst[i]);
        t->src_stride[i] = st;   // the source may be a view: strides from its parent's extents
        st *= src_parent.empty() ? t->src_extent[i] : src_parent[i];
    }
}

// Share of the last wave's SMs that have a tile: t tiles on n SMs take ceil(t / n) rounds.
double wave_efficiency(int64_t tiles, int sms)
{
    const int64_t t = std::max<int64_t>(tiles, 1);
    return double(t) / double(ceil_div(t, sms) * sms);
}

// The gather kernel fetches 16 bytes per load when the stride-1 mode of an operand is the first row
// mode of its tile (C's order) or the first contracted mode, and has an even extent; else 8 bytes.
bool gathers_16_bytes(const Problem& p)
{
    auto ok = [&](const std::vector<int>& t, const std::vector<int>& rows) {
        if (t.empty()) return false;
        const Mode& m = p.modes[static_cast<size_t>(t[0])];
        const bool lead = (!rows.empty() && t[0] == rows[0]) || (!p.K.empty() && t[0] == p.K[0]);
        return lead && m.extent % 2 == 0;
    };
    return ok(p.A, p.M) && ok(p.B, p.N);
}

double contraction_us(const Problem& p, int kernel, const UmmaSpec& u, const CostTable& c)
{
    const double elt = p.scalar_type == 1 ? 8.0 : 4.0;
    const double flops = 2.0 * double(p.Mtot) * double(p.Ntot) * double(p.Ktot);
    double c_bytes = double(p.sizeC) * elt;
    double rate = p.scalar_type == 1 ? c.simt_f64_tflops : c.simt_f32_tflops;
    double extra_us = 0, scatter_us = 0, extra_floor_us = 0;
    // tiles are computed whole: the work of an FP64 kernel is that of the extents rounded up to its tile
    auto padded = [&](int64_t bm, int64_t bn) {
        return double(ceil_div(p.Mtot, bm) * bm) / double(p.Mtot) * double(ceil_div(p.Ntot, bn) * bn) / double(p.Ntot);
    };
    if (kernel == KERNEL_SIMT && p.scalar_type == 1)
        rate *= wave_efficiency(ceil_div(p.Mtot, 64) * ceil_div(p.Ntot, 64), c.num_sms) / padded(64, 64);
    // TMA-fed kernels: slabs and k chunks are whole, ragged extents are zero-filled and multiplied anyway
    // (extents of 72 in 32-wide slabs and chunks: abcd-aefb-fdce ran at 138 TFLOP/s direct, 415 after a
    // transpose that fuses the ragged modes away)
    const double tma_padding = double(u.tiles_m * u.BM) / double(p.Mtot) * double(u.tiles_n * u.BN) / double(p.Ntot) *
                               double(u.k_iters * u.BK) / double(p.Ktot);
    if ((kernel == KERNEL_DMMA_F64_TMA || kernel == KERNEL_UMMA_TF32) && u.k_splits > 1) {
        // partial tensors written, read back and summed by a second kernel
        extra_us += c.launch_us + 2.0 * double(u.k_splits) * double(p.sizeC) * elt / (c.hbm_gbs * 1e3);
    }
    if (kernel == KERNEL_DMMA_F64_TMA) {
        rate = c.dmma_f64_tflops * wave_efficiency(u.tiles_m * u.tiles_n * u.k_splits, c.num_sms) / tma_padding;
        // Rows of a slab that are not contiguous in C are stored element by element
        // (abcdef-dega-gfbc: 37.7 M elements of C, 1.08 ms against 0.10 ms for its coalesced siblings).
        // (runs shorter than 64 bytes count as scattered too: cfg3 cut to a = 6 ran at 17.6 TFLOP/s here
        // against 20.2 on the gather kernel, which sees those rows as one flat index)
        if ((u.a.row_elem_cstride != 1 && !u.store_across_slabs) || u.a.slab_mode_ext < 8)
            scatter_us = double(p.sizeC) * double(u.k_splits) * c.scatter_store_ps * 1e-6;
    }
    if (kernel == KERNEL_DMMA_F64) {
        const int64_t bn = p.Ntot <= 48 ? 32 : 64, bm = p.Ntot <= 48 ? 256 : 128;
        // Measured: 19 to 20 TFLOP/s with 16-byte gathers on both operands (abc-ad-bdc), 13 to 15 with
        // one operand on 8-byte gathers (abcd-eafb-fdec), 3.5 to 4.4 on the 256 x 32 tiles for narrow N.
        const double r = p.Ntot <= 48 ? c.dmma_f64_gather_narrow_tflops
                                      : (gathers_16_bytes(p) ? c.dmma_f64_gather_tflops : c.dmma_f64_gather8_tflops);
        rate = r *
               wave_efficiency(ceil_div(p.Mtot, bm) * ceil_div(p.Ntot, bn), c.num_sms) / padded(bm, bn);
    }
    if (kernel == KERNEL_UMMA_TF32) {
        rate = c.umma_tf32_tflops * (1.0 - c.far_row_penalty * u.far_fraction) *
               wave_efficiency((u.pair ? ceil_div(u.tiles_m, 2) : u.tiles_m) * u.tiles_n * u.k_splits, u.pair ? c.num_sms / 2 : c.num_sms) / tma_padding;
        // Rows of a slab that are not contiguous in C are stored element by element, a 32-byte sector each
        // (abcd-dbea-ec, 9.0 M elements of C: 0.125 ms against a 0.022 ms traffic floor).
        if (u.a.row_elem_cstride != 1) scatter_us = double(p.sizeC) * double(u.k_splits) * c.scatter_store_f32_ps * 1e-6;
        // (one stage per umma_stage_us at best: see plan_umma_impl)
        const int64_t units = (u.pair ? ceil_div(u.tiles_m, 2) : u.tiles_m) * u.tiles_n * u.k_splits;
        const int64_t wave = u.pair ? c.num_sms / 2 : c.num_sms;
        // ... and a tile leaves an SM no faster than the epilogue stores it (cfg4: 7 776 tiles of 128 x 256 in 0.196 ms)
        const double tile_store_us = double(u.BM) * double(u.BN) * 4.0 / (c.umma_store_gbs_per_sm * 1e3);
        extra_floor_us = double(ceil_div(units, wave)) * std::max(double(u.k_iters_per_split) * c.umma_stage_us / u.producers, tile_store_us);
    }
    const double bytes = (double(p.sizeA) + double(p.sizeB)) * elt + c_bytes;
    // scattered stores are a third ceiling rather than an addition: one consumer group stores while the
    // other computes (abc-bda-dc, K = 312: 0.086 ms scattered against 0.072 ms for its coalesced sibling)
    return c.launch_us + std::max({flops / (rate * 1e6), bytes / (c.hbm_gbs * 1e3), scatter_us, extra_floor_us}) + extra_us;
}

// TF32 goes to the tcgen05 kernel whenever its tiles can be described to TMA.  FP64 takes the
// cheapest of the TMA-fed tensor-path kernel, the gather tensor-path kernel (needs a tile per SM)
// and the 64 x 64 CUDA-core tiles, by the cost table.
int pick_kernel(const Problem& p, const UmmaSpec& u, const CostTable& c)
{
    if (u.eligible && u.elt == 4) return KERNEL_UMMA_TF32;
    if (p.scalar_type != 1) return KERNEL_SIMT;
    const char* k = std::getenv("TCONT_KERNEL");
    if (k && std::strcmp(k, "simt") == 0) return KERNEL_SIMT;
    if (k && std::strcmp(k, "tma") == 0 && u.eligible && u.elt == 8) return KERNEL_DMMA_F64_TMA;
    int best = KERNEL_SIMT;
    double best_us = contraction_us(p, KERNEL_SIMT, u, c);
    const int64_t bn = p.Ntot <= 48 ? 32 : 64, bm = p.Ntot <= 48 ? 256 : 128;  // the gather kernel's smallest fitting tile
    if (k && std::strcmp(k, "gather") == 0 && ceil_div(p.Mtot, bm) * ceil_div(p.Ntot, bn) >= c.num_sms) return KERNEL_DMMA_F64;
    if (ceil_div(p.Mtot, bm) * ceil_div(p.Ntot, bn) >= c.num_sms) {
        const double us = contraction_us(p, KERNEL_DMMA_F64, u, c);
        if (us < best_us) best = KERNEL_DMMA_F64, best_us = us;
    }
    if (u.eligible && u.elt == 8) {
        // The gather kernel's rates come from long contracted extents; on short ones it falls well below
        // them (8 TFLOP/s at K = 24), so it has to look 30 % better than the TMA-fed kernel to be taken.
        const double us = contraction_us(p, KERNEL_DMMA_F64_TMA, u, c);
        if (us < (best == KERNEL_DMMA_F64 ? 1.3 : 1.0) * best_us) best = KERNEL_DMMA_F64_TMA, best_us = us;
    }
    return best;
}

}  // namespace

bool read_cost_table_file(const std::string& path, CostTable* table)
{
    CostTable& c = *table;
    std::ifstream f(path);
    if (!f) return false;
    std::string key;
    double v;
    // "key value" pairs, one per line; unknown keys are ignored.
    while (f >> key >> v) {
        if (key == "hbm_gbs") c.hbm_gbs = v;
        else if (key == "umma_tf32_tflops") c.umma_tf32_tflops = v;
        else if (key == "simt_f32_tflops") c.simt_f32_tflops = v;
        else if (key == "simt_f64_tflops") c.simt_f64_tflops = v;
        else if (key == "launch_us") c.launch_us = v;
        else if (key == "dmma_f64_tflops") c.dmma_f64_tflops = v;
        else if (key == "dmma_f64_gather_tflops") c.dmma_f64_gather_tflops = v;
        else if (key == "dmma_f64_gather8_tflops") c.dmma_f64_gather8_tflops = v;
        else if (key == "dmma_f64_gather_narrow_tflops") c.dmma_f64_gather_narrow_tflops = v;
        else if (key == "scatter_store_ps") c.scatter_store_ps = v;
        else if (key == "scatter_store_f32_ps") c.scatter_store_f32_ps = v;
        else if (key == "far_row_penalty") c.far_row_penalty = v;
        else if (key == "umma_stage_us") c.umma_stage_us = v;
        else if (key == "umma_store_gbs_per_sm") c.umma_store_gbs_per_sm = v;
        else if (key == "num_sms" && v >= 1) c.num_sms = static_cast<int>(v);
    }
    return true;
}

CostTable load_cost_table()
{
    CostTable c;
    if (const char* path = std::getenv("TCONT_COST_TABLE")) read_cost_table_file(path, &c);
    return c;
}

int make_plan(const char* modeC, int nC, const char* modeA, int nA, const char* modeB, int nB, char op, int scalar_type,
              const char* ext_mode, const int64_t* ext_val, int n_ext, int backend_selection, const CostTable& cost,
              Plan* plan, std::string* err, const int64_t* parentC, const int64_t* parentA, const int64_t* parentB)
{
    if (!plan || !err) return 1;
    if (nC < 0 || nA < 0 || nB < 0 || n_ext < 0 || nC > kMaxModes || nA > kMaxModes || nB > kMaxModes || n_ext > 64) {
        *err = "Mode counts out of range";
        return 1;
    }
    if ((nC && !modeC) || (nA && !modeA) || (nB && !modeB) || (n_ext && (!ext_mode || !ext_val))) {
        *err = "Null mode or extent array";
        return 1;
    }
    if (scalar_type != 0 && scalar_type != 1) {
        *err = "Unsupported scalar type";
        return 1;
    }
    if (backend_selection < 0 || backend_selection > 2) {
        *err = "Unknown backend selection";
        return 1;
    }
    if (nA == 0 || nB == 0 || nC == 0) {
        *err = "Each tensor needs at least one mode";
        return 1;
    }
    Plan pl;
    pl.modeC.assign(modeC, static_cast<size_t>(nC));
    pl.modeA.assign(modeA, static_cast<size_t>(nA));
    pl.modeB.assign(modeB, static_cast<size_t>(nB));
    pl.ext_mode.assign(ext_mode, static_cast<size_t>(n_ext));
    pl.ext_val.assign(ext_val, ext_val + n_ext);
    pl.op = op;
    pl.scalar_type = scalar_type;
    pl.backend_selection = backend_selection;
    if (parentC) pl.parentC.assign(parentC, parentC + nC);
    if (parentA) pl.parentA.assign(parentA, parentA + nA);
    if (parentB) pl.parentB.assign(parentB, parentB + nB);

    Problem direct;
    int rc = build_problem(pl.modeC, pl.modeA, pl.modeB, pl.ext_mode, pl.ext_val, scalar_type, &direct, err, pl.parentC, pl.parentA, pl.parentB);
    if (rc) return rc;
    if (direct.sizeA >= (int64_t(1) << 32) || direct.sizeB >= (int64_t(1) << 32)) {
        *err = "Input tensors with 2^32 or more elements are not supported";
        return 3;
    }
    auto count = [&](const std::string& s) {
        int64_t n = 1;
        for (char c : s) n *= pl.ext_val[static_cast<size_t>(find_char(pl.ext_mode, c))];
        return n;
    };
    pl.sizeL = count(pl.modeA);
    pl.sizeR = count(pl.modeB);
    pl.sizeC = count(pl.modeC);
    pl.flops = 2.0 * std::sqrt(double(pl.sizeL) * double(pl.sizeR) * double(pl.sizeC));

    UmmaSpec direct_umma;
    plan_umma(direct, cost, &direct_umma);
    const int direct_kernel = pick_kernel(direct, direct_umma, cost);
    pl.est_direct_us = contraction_us(direct, direct_kernel, direct_umma, cost);

    // Transpose-assisted candidate.  A role's transposed layout is
    //     [lead | K modes | remaining row modes in C order]
    // where `lead` is the shortest run of the role's first row modes (consecutive in C) whose fused
    // extent is a multiple of 32: the slab mode stays stride-1 and the K rows of a tile follow it
    // directly, so a TMA box is one contiguous piece of memory.  An operand that already starts
    // with [lead, first K mode] (or is K-major on that K mode) is used where it lies.  Three K
    // orders are tried (by A's strides, by B's strides, the direct plan's); the one that moves
    // the fewest bytes wins.  C is written in its final order by the contraction kernel, so
    // there is never a third transpose (the reference's TTGT always pays C' -> C,
    // backends/ttgt_cutt/src/ttgt_cutt.cpp:811-816).
    const std::string& roleA_src = direct.swapped ? pl.modeB : pl.modeA;
    const std::string& roleB_src = direct.swapped ? pl.modeA : pl.modeB;
    auto ext_of = [&](char c) { return pl.ext_val[static_cast<size_t>(find_char(pl.ext_mode, c))]; };
    auto lead_of = [&](const std::string& src) {  // row modes of `src` in C order, split into (lead, rest)
        std::string rows;
        for (char c : pl.modeC)
            if (find_char(src, c) >= 0) rows.push_back(c);
        size_t n = 0;
        int64_t prod = 1;
        bool found = false;
        while (n < rows.size()) {
            if (n > 0 && find_char(pl.modeC, rows[n]) != find_char(pl.modeC, rows[n - 1]) + 1) break;
            prod *= ext_of(rows[n]);
            ++n;
            if (prod % 32 == 0) { found = true; break; }
        }
        if (!found) {  // no multiple of 32: keep the whole leading run together
            n = 1;
            while (n < rows.size() && find_char(pl.modeC, rows[n]) == find_char(pl.modeC, rows[n - 1]) + 1) ++n;
        }
        // FP64: a leading run too short for whole slabs (extent 6 or 12: a quarter of the rows empty) takes the
        // next run of row modes along, so that the kernel's planner can stage both as one fused mode
        // (operand-level row fusion in plan_umma)
        if (scalar_type == 1 && n < rows.size()) {
            int64_t lead_ext = 1;
            for (size_t i = 0; i < n; ++i) lead_ext *= ext_of(rows[i]);
            if (slab_padding_f64(lead_ext) > 1.08) {
                size_t m = n + 1;
                while (m < rows.size() && find_char(pl.modeC, rows[m]) == find_char(pl.modeC, rows[m - 1]) + 1) ++m;
                n = m;
            }
        }
        return std::make_pair(rows.substr(0, n), rows.substr(n));
    };
    const auto leadA = lead_of(roleA_src), leadB = lead_of(roleB_src);
    std::string kall;
    for (char c : roleA_src)
        if (find_char(pl.modeC, c) < 0) kall.push_back(c);
    auto sorted_by = [&](const std::string& src) {
        std::string k = kall;
        std::sort(k.begin(), k.end(), [&](char x, char y) { return find_char(src, x) < find_char(src, y); });
        return k;
    };
    auto starts_with = [](const std::string& s, const std::string& pre) { return s.compare(0, pre.size(), pre) == 0; };
    std::string roleA_dst = roleA_src, roleB_dst = roleB_src;
    {
        double best = 1e300;
        for (const std::string& korder : {sorted_by(roleB_src), sorted_by(roleA_src), perm_modes(direct, direct.K)}) {
            if (korder.empty()) continue;
            auto keep = [&](const std::string& src, const std::string& lead) {
                return src[0] == korder[0] || starts_with(src, lead + korder[0]);
            };
            const bool keepA = keep(roleA_src, leadA.first), keepB = keep(roleB_src, leadB.first);
            const double moved = (keepA ? 0.0 : double(direct.sizeA)) + (keepB ? 0.0 : double(direct.sizeB));
            if (moved < best) {
                best = moved;
                roleA_dst = keepA ? roleA_src : leadA.first + korder + leadA.second;
                roleB_dst = keepB ? roleB_src : leadB.first + korder + leadB.second;
            }
        }
    }
    // (a transposed operand is a dense scratch tensor; one that is used where it lies keeps its parent's strides)
    const std::vector<int64_t>& roleA_parent = direct.swapped ? pl.parentB : pl.parentA;
    const std::vector<int64_t>& roleB_parent = direct.swapped ? pl.parentA : pl.parentB;
    const std::vector<int64_t> dense;
    Problem ttgt;
    rc = build_problem(pl.modeC, roleA_dst, roleB_dst, pl.ext_mode, pl.ext_val, scalar_type, &ttgt, err, pl.parentC,
                       roleA_dst == roleA_src ? roleA_parent : dense, roleB_dst == roleB_src ? roleB_parent : dense);
    if (rc) return rc;
    UmmaSpec ttgt_umma;
    plan_umma(ttgt, cost, &ttgt_umma);
    const int ttgt_kernel = pick_kernel(ttgt, ttgt_umma, cost);
    TransposeSpec tA, tB;
    fill_transpose(roleA_src, roleA_dst, pl.ext_mode, pl.ext_val, &tA, roleA_parent);
    fill_transpose(roleB_src, roleB_dst, pl.ext_mode, pl.ext_val, &tB, roleB_parent);
    const double elt = scalar_type == 1 ? 8.0 : 4.0;
    double t_us = 0;
    if (tA.needed) t_us += cost.launch_us + 2.0 * double(tA.elements) * elt / (cost.hbm_gbs * 0.7 * 1e3);
    if (tB.needed) t_us += cost.launch_us + 2.0 * double(tB.elements) * elt / (cost.hbm_gbs * 0.7 * 1e3);
    pl.est_ttgt_us = t_us + contraction_us(ttgt, ttgt_kernel, ttgt_umma, cost);

    bool use_ttgt;
    if (backend_selection == 1) use_ttgt = false;
    else if (backend_selection == 2) use_ttgt = true;
    else use_ttgt = (tA.needed || tB.needed) && pl.est_ttgt_us < pl.est_direct_us;

    if (use_ttgt) {
        pl.backend = 1;
        pl.prob = ttgt;
        pl.prob.swapped = direct.swapped;  // roles still map to the caller's operands as in `direct`
        pl.tA = tA;
        pl.tB = tB;
        pl.kernel = ttgt_kernel;
        pl.umma = ttgt_umma;
    } else {
        pl.backend = 0;
        pl.prob = direct;
        pl.kernel = direct_kernel;
        pl.umma = direct_umma;
    }
    const Problem& p = pl.prob;
    auto first_is = [&](const std::vector<int>& t, const std::vector<int>& grp) {
        return !t.empty() && !grp.empty() && t[0] == grp[0];
    };
    // SIMT loads run along m (or n) when the operand's stride-1 mode is the fastest mode of the
    // flat m (n) index, along k when it is the fastest contracted mode.
    pl.simt.a_load_along_k = first_is(p.A, p.M) ? 0 : (first_is(p.A, p.K) ? 1 : 0);
    pl.simt.b_load_along_k = first_is(p.B, p.N) ? 0 : (first_is(p.B, p.K) ? 1 : 0);
    *plan = pl;
    return 0;
}

void build_offset_tables(const Problem& p, OffsetTables* t)
{
    auto fill = [&](const std::vector<int>& grp, int64_t total, int which, std::vector<int64_t>* out) {
        out->assign(static_cast<size_t>(total), 0);
        for (int64_t i = 0; i < total; ++i) {
            int64_t rem = i, off = 0;
            for (int id : grp) {
                const Mode& m = p.modes[static_cast<size_t>(id)];
                const int64_t idx = rem % m.extent;
                rem /= m.extent;
                off += idx * (which == 0 ? m.sA : which == 1 ? m.sB : m.sC);
            }
            (*out)[static_cast<size_t>(i)] = off;
        }
    };
    fill(p.M, p.Mtot, 0, &t->offAm);
    fill(p.K, p.Ktot, 0, &t->offAk);
    fill(p.N, p.Ntot, 1, &t->offBn);
    fill(p.K, p.Ktot, 1, &t->offBk);
    fill(p.M, p.Mtot, 2, &t->offCm);
    fill(p.N, p.Ntot, 2, &t->offCn);
}

std::string describe_plan(const Plan& pl)
{
    std::ostringstream o;
    const Problem& p = pl.prob;
    auto list = [&](const std::vector<int>& ids) {
        std::string s = "[";
        for (size_t i = 0; i < ids.size(); ++i) {
            const Mode& m = p.modes[static_cast<size_t>(ids[i])];
            s += (i ? "," : "") + std::string("\"") + m.names + ":" + std::to_string(m.extent) + "\"";
        }
        return s + "]";
    };
    auto perm = [&](const TransposeSpec& t) {
        std::string s = "[";
        for (int i = 0; i < t.rank; ++i) s += (i ? "," : "") + std::to_string(t.perm[i]);
        return s + "]";
    };
    o << "{\"backend\":\"" << (pl.backend == 0 ? "direct" : "ttgt") << "\",\"kernel\":\""
      << (pl.kernel == KERNEL_UMMA_TF32 ? "umma_tf32" : pl.kernel == KERNEL_DMMA_F64 ? "dmma_f64"
          : pl.kernel == KERNEL_DMMA_F64_TMA ? "dmma_f64_tma" : "simt") << "\""
      << ",\"scalar\":\"" << (pl.scalar_type == 1 ? "f64" : "f32") << "\",\"swapped\":" << (p.swapped ? "true" : "false")
      << ",\"views\":" << (p.strided ? "true" : "false")
      << ",\"A\":" << list(p.A) << ",\"B\":" << list(p.B) << ",\"C\":" << list(p.C) << ",\"M\":" << list(p.M)
      << ",\"N\":" << list(p.N) << ",\"K\":" << list(p.K) << ",\"Mtot\":" << p.Mtot << ",\"Ntot\":" << p.Ntot
      << ",\"Ktot\":" << p.Ktot << ",\"transpose_a\":" << (pl.tA.needed ? perm(pl.tA) : "null")
      << ",\"transpose_b\":" << (pl.tB.needed ? perm(pl.tB) : "null") << ",\"est_direct_us\":" << pl.est_direct_us
      << ",\"est_ttgt_us\":" << pl.est_ttgt_us << ",\"simt\":{\"a_along_k\":" << pl.simt.a_load_along_k
      << ",\"b_along_k\":" << pl.simt.b_load_along_k << "}";
    const UmmaSpec& u = pl.umma;
    o << ",\"umma\":{\"eligible\":" << (u.eligible ? "true" : "false");
    if (!u.eligible) o << ",\"why_not\":\"" << u.why_not << "\"";
    else {
        o << ",\"BM\":" << u.BM << ",\"BN\":" << u.BN << ",\"BK\":" << u.BK << ",\"stages\":" << u.stages
          << ",\"pair\":" << (u.pair ? "true" : "false") << ",\"kc\":\"" << u.kc_names << "\",\"k_iters\":" << u.k_iters << ",\"k_splits\":" << u.k_splits << ",\"tiles_m\":" << u.tiles_m << ",\"tiles_n\":" << u.tiles_n
          << ",\"a_major\":\"" << (u.a.major ? "MN" : "K") << "\",\"b_major\":\"" << (u.b.major ? "MN" : "K") << "\""
          << ",\"a_slab_w\":" << u.a.slab_w << ",\"b_slab_w\":" << u.b.slab_w << ",\"a_slabs_per_copy\":" << u.a.slabs_per_op << ",\"b_slabs_per_copy\":" << u.b.slabs_per_op << ",\"a_slabs\":" << u.a.slabs_per_tile
          << ",\"b_slabs\":" << u.b.slabs_per_tile << ",\"smem_bytes\":" << u.smem_bytes
          << ",\"coalesced_store\":" << (u.a.row_elem_cstride == 1 ? "true" : "false")
          << ",\"store_across_slabs\":" << (u.store_across_slabs ? "true" : "false") << ",\"producers\":" << u.producers;
    }
    o << "}}";
    return o.str();
}

}  // namespace tcontb
