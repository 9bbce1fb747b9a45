// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/CondMatMatSca.h): res = cond ? thenVal : elseVal with a scalar elseVal.
#pragma once
#include <B200Adapter.h>
template <class DTRes, class DTCond, class DTThen, class VTElse>
void condMatMatSca(DTRes *&res, const DTCond *cond, const DTThen *thenVal, VTElse elseVal, DCTX(ctx)) {
    using VT = typename DTRes::VT;
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    const VT e = static_cast<VT>(elseVal);
    b200::check(db2_cond(call.c, &r, b200::dtype_of<VT>(), call.in(cond), call.in(thenVal), nullptr, nullptr, &e));
    if (!res)
        res = call.template wrap<VT>(r);
}
