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
#include "fused_types.cuh"

struct db2_context;

namespace db2 {

// host side launchers (fused.cu)
int fused_row_pass_f64(const FusedProgram &prog, cudaStream_t st);
// Specialised (compile-time) versions of frequent chains (fused_ct.cu).  `signature` spells the chain and its taps,
// e.g. "SUB.R|DIV.R|SQ.S#MAX@2,SUM@3"; returns true when a specialised kernel was launched.
bool fused_row_pass_ct(const FusedProgram &prog, const char *signature, cudaStream_t st, int *rc);
// the specialisation of prog's chain compiled at run time (fused_rtc.cu): true if it was launched
// aligned: base (and stored result) rows start on 16-byte boundaries and the number of columns is even
bool fused_row_pass_rtc(const FusedProgram &prog, bool aligned, cudaStream_t st, int *rc);
bool fused_col_pass_rtc(const FusedProgram &prog, int mean, void *res, void *scratch, cudaStream_t st, int *rc);
// geometry and last step of the compile-time column pass (fused_ct.cu), shared with the kernels compiled at run time
void fused_col_geometry(const FusedProgram &prog, unsigned (&grid)[2], unsigned (&block)[2]);
int fused_col_finish(const FusedProgram &prog, unsigned parts, int mean, void *res, void *scratch, cudaStream_t st);
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
