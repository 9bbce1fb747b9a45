// Fused evaluation of deferred elementwise chains.
//
// DAPHNE's compiled pipelines call one kernel per operator, so a chain such as  Z = (X - mu) / sd;  r = sum(Z^2, 0);
// m = aggMax(Z, 0);  i = idxMax(Z, 0)  would move the 4 GiB operand through HBM once per call.  The runtime therefore
// records cheap elementwise operators as a CHAIN on their (materialised) base operand instead of running them, and
// the consumers -- row aggregations, column aggregations, or a plain materialisation -- evaluate the chain inside
// their own load loop: value = base[r][c]; for each step: value = op(value, operand) with the operand a same-shape
// matrix, a row vector, a column vector or an immediate.  Several row aggregations whose chains are prefixes of one
// another are served by ONE pass ("taps" after the step where their chain ends).
//
// The step list is a tiny interpreted program (uniform control flow: every thread executes the same step), passed to
// the kernel as a __grid_constant__ parameter; there is no run-time code generation.
#pragma once

#include "common.cuh"

struct db2_context;

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

// host side launchers (fused.cu)
int fused_row_pass_f64(const FusedProgram &prog, cudaStream_t st);
// Specialised (compile-time) versions of frequent chains (fused_ct.cu).  `signature` spells the chain and its taps,
// e.g. "SUB.R|DIV.R|SQ.S#MAX@2,SUM@3"; returns true when a specialised kernel was launched.
bool fused_row_pass_ct(const FusedProgram &prog, const char *signature, cudaStream_t st, int *rc);
bool fused_col_pass_ct(const FusedProgram &prog, const char *signature, int agg_op, void *res, void *scratch,
                       size_t scratch_bytes, cudaStream_t st, int *rc);
// column aggregation of a chain: kind = K_SUM / K_MIN / K_MAX / K_PROD of agg.cu, epilogue like db2k_agg_col
int fused_col_pass_f64(const FusedProgram &prog, int agg_op, void *res, void *scratch, size_t scratch_bytes,
                       cudaStream_t st);
size_t fused_col_scratch_bytes(int64_t cols);
// flat pass (fused.cu): chains on column vectors or contiguous same-shape operands; optional prefix output after
// `mid_after` steps (contiguous, mid_out) and optional sum of the final values (*sum_out on the device)
bool fused_flat_eligible(const FusedProgram &prog);
size_t fused_flat_scratch_bytes();
int fused_flat_pass_f64(const FusedProgram &prog, void *mid_out, int mid_after, double *sum_out, void *scratch,
                        size_t scratch_bytes, cudaStream_t st);

// row aggregation of a CSR matrix with a fused epilogue on the rows x 1 result (csr.cu): prog.steps are applied to every
// row's aggregate (operands: column vectors / same-shape rows x 1 matrices, 1 x 1 matrices, immediates), prog.ew_out
// receives the final values, mid_out the values after mid_after steps, *sum_out (device) the sum of the final values
// (folded in block order by the last block to finish); prog.base is not used.  scratch: at least
// csr_agg_scratch_bytes() bytes; ticket: a device word that is zero before and after every launch.
struct CsrSrc;
size_t csr_agg_scratch_bytes();
int csr_agg_pass(struct ::db2_context *ctx, const CsrSrc &src, const FusedProgram &prog, double *mid_out, int mid_after,
                 double *sum_out, void *scratch, size_t scratch_bytes);

// tall-skinny product with fused row epilogue (skinny.cu): D = A @ op(B), then prog.steps on D, prog.taps (row MIN /
// MAX with positions, at the end of the chain) and prog.ew_out (the values after all steps); prog.base is not used
struct SkinnyArgs {
    const double *A;
    int64_t lda, n;
    const double *B;
    int64_t ldb;
    int K, N, tb; // tb: B is stored N x K
    FusedProgram prog;
};
bool skinny_shape_ok(int64_t n, int64_t K, int64_t N, const void *A, int64_t lda);
bool skinny_op_supported(int fused_op);
int skinny_vec_slots(); // row-vector / column-vector operands (each kind) a fused chain may have
int skinny_gemm(const SkinnyArgs &a, cudaStream_t st);

} // namespace db2
