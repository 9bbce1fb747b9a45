// Backend-"CPP" name of the elementwise binary kernel (src/runtime/local/kernels/EwBinaryMat.h:44-52), registered here
// only for the sparse-times-dense product EwBinaryMat<CSRMatrix, CSRMatrix, DenseMatrix> (EwBinaryMat.h:254-317: MUL,
// rhs of the same shape or a row / column vector, entries meeting a zero are dropped).  Dense operands keep going
// through the CUDA-backend names.
#pragma once
#include <B200Csr.h>
#include <runtime/local/kernels/BinaryOpCode.h>
template <class DTRes, class DTLhs, class DTRhs>
void ewBinaryMat(BinaryOpCode opCode, DTRes *&res, const DTLhs *lhs, const DTRhs *rhs, DCTX(ctx)) {
    static_assert(b200::is_csr<DTRes>::value && b200::is_csr<DTLhs>::value && !b200::is_csr<DTRhs>::value,
                  "registered for CSRMatrix = CSRMatrix (op) DenseMatrix only");
    b200::csr_ew_mul(opCode, res, lhs, rhs, ctx);
}
