// Backend-"CPP" name of gemv (src/runtime/local/kernels/Gemv.h:40-43), registered here only for a CSRMatrix operand
// (Gemv.h:79-117 computes mat @ vec for it, without the transposition of the dense form).
#pragma once
#include <B200Csr.h>
template <class DTRes, class DTMat, class DTVec> void gemv(DTRes *&res, const DTMat *mat, const DTVec *vec, DCTX(ctx)) {
    static_assert(b200::is_csr<DTMat>::value, "registered for a CSRMatrix operand only");
    b200::csr_mat_mul(res, mat, vec, false, false, ctx);
}
