// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/CondMatScaMat.h): res = cond ? thenVal : elseVal with a scalar thenVal.
#pragma once
#include <B200Adapter.h>
template <class DTRes, class DTCond, class VTThen, class DTElse>
void condMatScaMat(DTRes *&res, const DTCond *cond, VTThen thenVal, const DTElse *elseVal, DCTX(ctx)) {
    using VT = typename DTRes::VT;
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    const VT t = static_cast<VT>(thenVal);
    b200::check(db2_cond(call.c, &r, b200::dtype_of<VT>(), call.in(cond), nullptr, &t, call.in(elseVal), nullptr));
    if (!res)
        res = call.template wrap<VT>(r);
}
