// The recorded program of a fused pass: plain data shared by the host (which fills it in), the kernels compiled into
// the library and the kernels compiled at run time for chains that have no compiled-in specialisation (fused_rtc.cu).
// Nothing but built-in types, so that the run-time compiler needs no host headers.
#pragma once

#ifdef __CUDACC_RTC__
typedef int int32_t;
typedef unsigned int uint32_t;
typedef long long int64_t;
typedef unsigned long long uint64_t;
#ifndef INFINITY
#define INFINITY __int_as_float(0x7f800000)
#endif
#ifndef NAN
#define NAN __int_as_float(0x7fffffff)
#endif
#else
#include <cmath>
#include <cstdint>
#endif

namespace db2 {

constexpr int FUSED_MAX_STEPS = 10;
constexpr int FUSED_MAX_AGGS = 4;

enum FusedOperandKind : int32_t {
    FK_MATRIX = 0, // same shape as the base operand
    FK_ROWVEC = 1, // 1 x cols
    FK_COLVEC = 2, // rows x 1
    FK_SCALAR = 3, // immediate
    FK_UNARY = 4,  // no operand
};

// internal opcode of a fused step (a subset of the binary/unary op codes: the cheap, exactly rounded ones)
enum FusedOp : int32_t {
    FO_ADD = 0, FO_SUB, FO_MUL, FO_DIV, FO_SQUARE, FO_EQ, FO_NEQ, FO_LT, FO_LE, FO_GT, FO_GE, FO_MIN, FO_MAX, FO_AND,
    FO_OR, FO_NEG, FO_ABS, FO_SIGN, FO_FLOOR, FO_CEIL, FO_ROUND, FO_ISNAN, FO_COUNT
};

struct FusedStep {
    int32_t kind;     // FusedOperandKind
    int32_t op;       // FusedOp
    int32_t reversed; // operand (op) value instead of value (op) operand
    int32_t smem_off; // ROWVEC operands staged in shared memory: element offset of this step's copy, else -1
    const void *ptr;  // operand (device) for MATRIX / ROWVEC / COLVEC
    int64_t ld;       // leading dimension of a MATRIX / COLVEC operand
    double imm;       // SCALAR operand
};

// kinds of row trackers; MIN/MAX trackers can deliver the extremum (out) and its position (out_idx) together
enum FusedTapKind : int32_t { FT_SUM = 0, FT_PROD = 1, FT_MIN = 2, FT_MAX = 3, FT_MEAN = 4 };

struct FusedTap {
    int32_t after_step; // the aggregation sees the value after this many steps (0 = the base operand itself)
    int32_t kind;       // FusedTapKind
    void *out;          // rows x 1 values (may be null for MIN/MAX when only the position is wanted)
    void *out_idx;      // rows x 1 uint64 positions of the extremum (MIN/MAX only, may be null)
};

struct FusedProgram {
    const void *base;
    int64_t base_ld;
    int64_t rows, cols;
    int32_t nsteps, ntaps;
    int32_t smem_elems; // total elements of staged row-vector operands (2 per column and step: value, reciprocal)
    int32_t pad;
    void *ew_out; // if set: the value after all steps is stored here (materialisation)
    int64_t ew_out_ld;
    // column passes only: if set, the pass runs only when this device word is non-zero at the time the kernel starts
    // (a fallback that is queued behind a kernel which decides on the device whether it is needed)
    const int32_t *run_if;
    FusedStep steps[FUSED_MAX_STEPS];
    FusedTap taps[FUSED_MAX_AGGS];
};

} // namespace db2
