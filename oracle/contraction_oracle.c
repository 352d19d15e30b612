/*
 * contraction_oracle.c -- CPU restatement of the reference's verification path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing the library ships may call into this file; it exists so
 * the tests, the smoke check and the benchmark's CPU-baseline leg have an independent answer
 * to compare the CUDA path with.
 *
 * What is restated (paths are inside the TconT reference tree):
 *   - the contraction loop nests of benchmarks/tccg/tccg_verify.cpp:18-1616.  Every one of the
 *     49 hand-written cases there has the same shape: an OpenMP "parallel for collapse" over
 *     the output modes, innermost loops over the contracted modes, column-major address
 *     polynomials (first mode fastest), and "output[...] += left[...] * right[...]" into a
 *     zero-filled double array (e.g. case 21 at :660-689, case 18 at :567-592).  oracle_contract
 *     is that loop nest for an arbitrary mode pattern.
 *   - the Float32 widening of tccg_verify.cpp:1779-1802 (inputs and device output are converted
 *     to double before the loops run): oracle_contract_f32.
 *   - the comparator of tccg_verify.cpp:1620-1687 and the tolerance table of :1690-1701:
 *     oracle_compare / oracle_tolerance.
 *
 * Parity pin: the reference ships no golden vectors (its inputs are time-seeded), so the pin is
 * the reference verifier itself compiled from its own sources (oracle/ref_bridge.cpp, built
 * into oracle/_ref by oracle/Makefile): tests/golden/make_golden.py feeds this file's output
 * through all 49 reference loop nests and records the fixtures only when every case reports
 * zero differences.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_MAX_MODES 16

typedef struct {
    int nC, nA, nB;
    const char* modeC;
    const char* modeA;
    const char* modeB;
    int n_ext;
    const char* ext_mode;
    const int64_t* ext_val;
} oracle_desc;

typedef struct {
    int64_t differences;
    int64_t total;
    int64_t same;
    int64_t non_finite;
    int passed;
} oracle_compare_result;

static int64_t extent_of(const oracle_desc* d, char m)
{
    for (int i = 0; i < d->n_ext; ++i)
        if (d->ext_mode[i] == m) return d->ext_val[i];
    return -1;
}

static int find_mode(const char* modes, int n, char m)
{
    for (int i = 0; i < n; ++i)
        if (modes[i] == m) return i;
    return -1;
}

/* Column-major stride of position p (first mode has stride 1), as in every address
 * polynomial of the reference loops, e.g. idx_a + (idx_b + idx_c * size_b) * size_a. */
static int64_t stride_at(const oracle_desc* d, const char* modes, int p)
{
    int64_t s = 1;
    for (int i = 0; i < p; ++i) s *= extent_of(d, modes[i]);
    return s;
}

typedef struct {
    int nK;
    int64_t Ktot;
    int64_t* offA_k; /* A offset contributed by each flattened contracted index */
    int64_t* offB_k;
    int64_t c_ext[ORACLE_MAX_MODES];
    int64_t c_strideA[ORACLE_MAX_MODES]; /* stride in A of C's mode p (0 if the mode is in B) */
    int64_t c_strideB[ORACLE_MAX_MODES];
    int64_t Ctot;
} oracle_layout;

/* Returns 0 on success, non-zero for a descriptor the reference could not express either:
 * missing extent, repeated mode, a mode of C that is in neither or both inputs, a mode of an
 * input that is neither an output nor a contracted mode. */
static int build_layout(const oracle_desc* d, oracle_layout* L)
{
    if (d->nC > ORACLE_MAX_MODES || d->nA > ORACLE_MAX_MODES || d->nB > ORACLE_MAX_MODES) return 1;
    for (int i = 0; i < d->nC; ++i) if (extent_of(d, d->modeC[i]) <= 0) return 2;
    for (int i = 0; i < d->nA; ++i) if (extent_of(d, d->modeA[i]) <= 0) return 2;
    for (int i = 0; i < d->nB; ++i) if (extent_of(d, d->modeB[i]) <= 0) return 2;

    L->Ctot = 1;
    for (int p = 0; p < d->nC; ++p) {
        const char m = d->modeC[p];
        const int ia = find_mode(d->modeA, d->nA, m);
        const int ib = find_mode(d->modeB, d->nB, m);
        if ((ia < 0) == (ib < 0)) return 3;
        L->c_ext[p] = extent_of(d, m);
        L->c_strideA[p] = ia >= 0 ? stride_at(d, d->modeA, ia) : 0;
        L->c_strideB[p] = ib >= 0 ? stride_at(d, d->modeB, ib) : 0;
        L->Ctot *= L->c_ext[p];
    }

    /* Contracted modes: in A and B but not in C, outermost first in A's order, so the last
     * contracted mode of A is the innermost loop (the reference's case 21 loops e outside f
     * for A[a,e,b,f]). */
    char kmodes[ORACLE_MAX_MODES];
    L->nK = 0;
    for (int i = 0; i < d->nA; ++i) {
        const char m = d->modeA[i];
        const int ic = find_mode(d->modeC, d->nC, m);
        const int ib = find_mode(d->modeB, d->nB, m);
        if (ic < 0 && ib < 0) return 4;
        if (ic < 0) kmodes[L->nK++] = m;
    }
    for (int i = 0; i < d->nB; ++i) {
        const char m = d->modeB[i];
        if (find_mode(d->modeC, d->nC, m) < 0 && find_mode(d->modeA, d->nA, m) < 0) return 4;
    }

    L->Ktot = 1;
    for (int i = 0; i < L->nK; ++i) L->Ktot *= extent_of(d, kmodes[i]);
    L->offA_k = (int64_t*)malloc(sizeof(int64_t) * (size_t)L->Ktot);
    L->offB_k = (int64_t*)malloc(sizeof(int64_t) * (size_t)L->Ktot);
    if (!L->offA_k || !L->offB_k) return 5;
    for (int64_t k = 0; k < L->Ktot; ++k) {
        int64_t rem = k, oa = 0, ob = 0;
        for (int i = L->nK - 1; i >= 0; --i) { /* last contracted mode varies fastest */
            const int64_t e = extent_of(d, kmodes[i]);
            const int64_t idx = rem % e;
            rem /= e;
            oa += idx * stride_at(d, d->modeA, find_mode(d->modeA, d->nA, kmodes[i]));
            ob += idx * stride_at(d, d->modeB, find_mode(d->modeB, d->nB, kmodes[i]));
        }
        L->offA_k[k] = oa;
        L->offB_k[k] = ob;
    }
    return 0;
}

static void free_layout(oracle_layout* L)
{
    free(L->offA_k);
    free(L->offB_k);
}

static inline void split_output_index(const oracle_layout* L, int nC, int64_t c, int64_t* baseA, int64_t* baseB)
{
    int64_t rem = c, a = 0, b = 0;
    for (int p = 0; p < nC; ++p) {
        const int64_t idx = rem % L->c_ext[p];
        rem /= L->c_ext[p];
        a += idx * L->c_strideA[p];
        b += idx * L->c_strideB[p];
    }
    *baseA = a;
    *baseB = b;
}

/* C = sum_K A * B, double in, double out; C is overwritten (the reference zero-fills its
 * reference_output and accumulates into it, tccg_verify.cpp:1819-1828). */
int oracle_contract(const oracle_desc* d, const double* A, const double* B, double* C)
{
    oracle_layout L;
    const int rc = build_layout(d, &L);
    if (rc) return rc;
    const int nC = d->nC;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < L.Ctot; ++c) {
        int64_t baseA, baseB;
        split_output_index(&L, nC, c, &baseA, &baseB);
        double acc = 0.0;
        for (int64_t k = 0; k < L.Ktot; ++k)
            acc += A[baseA + L.offA_k[k]] * B[baseB + L.offB_k[k]];
        C[c] = acc;
    }
    free_layout(&L);
    return 0;
}

/* How an fp32 operand is narrowed before the product:
 *   0  not at all (the reference's CPU path: exact fp32 values widened to double)
 *   1  TF32 by truncation (13 low mantissa bits dropped)
 *   2  TF32 by round-to-nearest, ties away from zero (what cvt.rna.tf32.f32 does) */
static inline double narrow_operand(float x, int mode)
{
    if (mode == 0) return (double)x;
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7f800000u) != 0x7f800000u) {
        if (mode == 2) u += 0x00001000u;
        u &= 0xffffe000u;
    }
    memcpy(&x, &u, 4);
    return (double)x;
}

/* Float32 flavour: operands widened to double (tccg_verify.cpp:1790-1793), double accumulate,
 * double output.  `rounding` selects the TF32-operand oracle used to separate format error
 * from kernel bugs. */
int oracle_contract_f32(const oracle_desc* d, const float* A, const float* B, double* C, int rounding)
{
    oracle_layout L;
    const int rc = build_layout(d, &L);
    if (rc) return rc;
    const int nC = d->nC;
#pragma omp parallel for schedule(static)
    for (int64_t c = 0; c < L.Ctot; ++c) {
        int64_t baseA, baseB;
        split_output_index(&L, nC, c, &baseA, &baseB);
        double acc = 0.0;
        for (int64_t k = 0; k < L.Ktot; ++k)
            acc += narrow_operand(A[baseA + L.offA_k[k]], rounding) * narrow_operand(B[baseB + L.offB_k[k]], rounding);
        C[c] = acc;
    }
    free_layout(&L);
    return 0;
}

/* Same sums, but only for the listed linear output indices: lets the full-size configurations
 * be checked on a random sample without hours of CPU time. */
int oracle_contract_sampled(const oracle_desc* d, int scalar_type, const void* A, const void* B,
                            int64_t n_samples, const int64_t* c_index, double* out, int rounding)
{
    oracle_layout L;
    const int rc = build_layout(d, &L);
    if (rc) return rc;
    const int nC = d->nC;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t s = 0; s < n_samples; ++s) {
        int64_t baseA, baseB;
        split_output_index(&L, nC, c_index[s], &baseA, &baseB);
        double acc = 0.0;
        if (scalar_type == 1) {
            const double* a = (const double*)A;
            const double* b = (const double*)B;
            for (int64_t k = 0; k < L.Ktot; ++k) acc += a[baseA + L.offA_k[k]] * b[baseB + L.offB_k[k]];
        } else {
            const float* a = (const float*)A;
            const float* b = (const float*)B;
            for (int64_t k = 0; k < L.Ktot; ++k)
                acc += narrow_operand(a[baseA + L.offA_k[k]], rounding) * narrow_operand(b[baseB + L.offB_k[k]], rounding);
        }
        out[s] = acc;
    }
    free_layout(&L);
    return 0;
}

/* tccg_verify.cpp:1690-1701: Float32 (TF32) abs 2e-3 / rel 5e-2, Float64 abs 1e-11 / rel 1e-9.
 * scalar_type: 0 = Float32, 1 = Float64 (the enum order of include/tcont.hpp:12-15). */
void oracle_tolerance(int scalar_type, double* abs_tol, double* rel_tol)
{
    if (scalar_type == 0) {
        *abs_tol = 2e-3;
        *rel_tol = 5e-2;
    } else {
        *abs_tol = 1e-11;
        *rel_tol = 1e-9;
    }
}

/* tccg_verify.cpp:1620-1687: an element differs when it is not finite on either side or when
 * |h-d| > max(abs_tol, rel_tol * max(|h|,|d|)); the run passes only with zero differences. */
void oracle_compare(int64_t total, const double* host, const double* device, double abs_tol, double rel_tol,
                    oracle_compare_result* r)
{
    int64_t diff = 0, same = 0, nonfinite = 0;
#pragma omp parallel for reduction(+ : diff, same, nonfinite) schedule(static)
    for (int64_t i = 0; i < total; ++i) {
        const double h = host[i], dv = device[i];
        if (!isfinite(h) || !isfinite(dv)) {
            nonfinite++;
            diff++;
            continue;
        }
        const double err = fabs(h - dv);
        const double scale = fmax(fabs(h), fabs(dv));
        const double tol = fmax(abs_tol, rel_tol * scale);
        if (err > tol) diff++;
        else same++;
    }
    r->differences = diff;
    r->total = total;
    r->same = same;
    r->non_finite = nonfinite;
    r->passed = diff == 0;
}

/* Counter-based uniform generator shared (by specification, not by code) with the library's
 * tcontb_fill_uniform: element i of a stream is lo + (hi-lo) * u, u = top 53 bits of
 * splitmix64(seed * 0x9E3779B97F4A7C15 + offset + i) scaled by 2^-53; fp32 tensors round the
 * double to float.  A is the stream at offset 0, B the stream at offset |A|. */
static inline uint64_t splitmix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

void oracle_fill_uniform(void* dst, int scalar_type, int64_t n, uint64_t seed, uint64_t offset, double lo, double hi)
{
    const uint64_t base = seed * 0x9E3779B97F4A7C15ull + offset;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const double u = (double)(splitmix64(base + (uint64_t)i) >> 11) * (1.0 / 9007199254740992.0);
        const double v = lo + (hi - lo) * u;
        if (scalar_type == 1) ((double*)dst)[i] = v;
        else ((float*)dst)[i] = (float)v;
    }
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the OpenMP team size of later calls made from the calling thread.  A launcher may have
 * exported OMP_NUM_THREADS=1 (torch.distributed.run does for several ranks); the timed CPU baseline
 * asks for all the cores the process may run on instead. */
void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
