// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/CondMatMatMat.h:41-46): res = cond ? thenVal : elseVal, element by element.
#pragma once
#include <B200Adapter.h>
template <class DTRes, class DTCond, class DTThen, class DTElse>
void condMatMatMat(DTRes *&res, const DTCond *cond, const DTThen *thenVal, const DTElse *elseVal, DCTX(ctx)) {
    using VT = typename DTRes::VT;
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_cond(call.c, &r, b200::dtype_of<VT>(), call.in(cond), call.in(thenVal), nullptr, call.in(elseVal),
                         nullptr));
    if (!res)
        res = call.template wrap<VT>(r);
}
