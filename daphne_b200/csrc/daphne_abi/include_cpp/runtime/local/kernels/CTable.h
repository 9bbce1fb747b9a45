// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/CTable.h:44-48): res[lhs[i], rhs[i]] += weight with int64 coordinate vectors.
#pragma once
#include <B200Adapter.h>
template <class DTRes, class DTLhs, class DTRhs, typename VTWeight>
void ctable(DTRes *&res, const DTLhs *lhs, const DTRhs *rhs, VTWeight weight, int64_t resNumRows, int64_t resNumCols,
            DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_ctable(call.c, &r, call.in(lhs), call.in(rhs), static_cast<double>(weight), resNumRows, resNumCols));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
