// ref_bridge.cpp -- C entry points around the reference's own CPU verifier and case table.
//
// TEST INFRASTRUCTURE ONLY.  This file is compiled together with the reference's unmodified
// sources (benchmarks/tccg/tccg_verify.cpp and benchmarks/tccg/tccg_cases.cpp, taken from where
// the reference tree lies) into oracle/_ref/libtccg_ref.so by oracle/Makefile.  It adds no
// arithmetic of its own: it builds a TconT::TCEquation from plain C arguments and forwards to
// verify_tccg_case (tccg_verify.cpp:1805-1840), and it reads list_tccg_bench /
// list_tccg_bench_fp32 (tccg_cases.cpp:3-509) so the fixture generator can enumerate the 49 case
// descriptors without parsing C++.
#include <cstdint>
#include <cstring>
#include <exception>

#include "tccg_cases.hpp"
#include "tccg_verify.hpp"
#include "tcont.hpp"

extern "C" {

struct ref_verify_result {
    int passed;
    int differences;
    int total_size;
    int same;
    int non_finite;
};

int ref_case_count(void) { return static_cast<int>(list_tccg_bench.size()); }

// Copies case `index` into caller buffers (each at least 16 chars / 16 extents).
// Returns the scalar type (0 Float32, 1 Float64) or -1 for a bad index.
int ref_case_get(int index, int fp32, char* modeC, int* nC, char* modeA, int* nA, char* modeB, int* nB,
                 char* ext_mode, int64_t* ext_val, int* n_ext, char* op)
{
    const auto& table = fp32 ? list_tccg_bench_fp32 : list_tccg_bench;
    if (index < 0 || index >= static_cast<int>(table.size())) return -1;
    const TconT::TCEquation& eq = table[static_cast<size_t>(index)];
    *nC = static_cast<int>(eq.modeC.size());
    *nA = static_cast<int>(eq.modeA.size());
    *nB = static_cast<int>(eq.modeB.size());
    std::memcpy(modeC, eq.modeC.data(), eq.modeC.size());
    std::memcpy(modeA, eq.modeA.data(), eq.modeA.size());
    std::memcpy(modeB, eq.modeB.data(), eq.modeB.size());
    int n = 0;
    for (const auto& kv : eq.extent) {
        ext_mode[n] = kv.first;
        ext_val[n] = kv.second;
        ++n;
    }
    *n_ext = n;
    *op = eq.op;
    return eq.scalar_type == TconT::ScalarType::Float64 ? 1 : 0;
}

// Runs the reference loop nest of `case_index` on (left, right) and compares it with `output`
// using the reference comparator.  scalar_type: 0 Float32, 1 Float64.  Returns 0, or -1 when
// the reference threw.
int ref_verify_case(int case_index, int scalar_type, const char* modeC, int nC, const char* modeA, int nA,
                    const char* modeB, int nB, const char* ext_mode, const int64_t* ext_val, int n_ext,
                    const void* output, const void* left, const void* right, ref_verify_result* out)
{
    try {
        TconT::TCEquation eq;
        eq.modeC.assign(modeC, modeC + nC);
        eq.modeA.assign(modeA, modeA + nA);
        eq.modeB.assign(modeB, modeB + nB);
        eq.op = '-';
        eq.scalar_type = scalar_type == 1 ? TconT::ScalarType::Float64 : TconT::ScalarType::Float32;
        for (int i = 0; i < n_ext; ++i) eq.extent[ext_mode[i]] = ext_val[i];
        const VerificationResult r = verify_tccg_case(static_cast<size_t>(case_index), eq, output, left, right);
        out->passed = r.passed ? 1 : 0;
        out->differences = r.differences;
        out->total_size = r.total_size;
        out->same = r.same;
        out->non_finite = r.non_finite;
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

}  // extern "C"
