// Backend-"CPP" name of matMul (src/runtime/local/kernels/MatMul.h:44-47), registered here for the forms the CUDA
// catalog does not name: a CSRMatrix lhs with a dense rhs (MatMul.h:60-215) and dense int64_t / int32_t operands (the
// reference's Eigen path, MatMul.cpp:40-134).  Dense double / float products keep going through the CUDA-backend name.
#pragma once
#include <B200Csr.h>
template <class DTRes, class DTLhs, class DTRhs>
void matMul(DTRes *&res, const DTLhs *lhs, const DTRhs *rhs, bool transa, bool transb, DCTX(ctx)) {
    if constexpr (b200::is_csr<DTLhs>::value) {
        static_assert(!b200::is_csr<DTRhs>::value && !b200::is_csr<DTRes>::value,
                      "registered for DenseMatrix = CSRMatrix @ DenseMatrix");
        b200::csr_mat_mul(res, lhs, rhs, transa, transb, ctx);
    } else {
        static_assert(std::is_integral_v<typename DTRes::VT>, "dense products of double / float are CUDA-backend names");
        b200::Call call(ctx);
        db2_matrix *r = res ? call.out(res) : nullptr;
        b200::check(db2_matMul(call.c, &r, call.in(lhs), call.in(rhs), transa, transb));
        if (!res)
            res = call.template wrap<typename DTRes::VT>(r);
    }
}
