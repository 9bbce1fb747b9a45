// Backend-"CPP" name of matMul (src/runtime/local/kernels/MatMul.h:44-47), registered here only for a CSRMatrix lhs and
// a dense rhs (MatMul.h:60-215); dense products keep going through the CUDA-backend name.
#pragma once
#include <B200Csr.h>
template <class DTRes, class DTLhs, class DTRhs>
void matMul(DTRes *&res, const DTLhs *lhs, const DTRhs *rhs, bool transa, bool transb, DCTX(ctx)) {
    static_assert(b200::is_csr<DTLhs>::value && !b200::is_csr<DTRhs>::value && !b200::is_csr<DTRes>::value,
                  "registered for DenseMatrix = CSRMatrix @ DenseMatrix only");
    b200::csr_mat_mul(res, lhs, rhs, transa, transb, ctx);
}
