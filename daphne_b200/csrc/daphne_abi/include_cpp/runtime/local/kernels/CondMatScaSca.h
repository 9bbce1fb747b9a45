// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/CondMatScaSca.h): res = cond ? thenVal : elseVal with two scalars.
#pragma once
#include <B200Adapter.h>
template <class DTRes, class DTCond, class VTThen, class VTElse>
void condMatScaSca(DTRes *&res, const DTCond *cond, VTThen thenVal, VTElse elseVal, DCTX(ctx)) {
    using VT = typename DTRes::VT;
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    const VT t = static_cast<VT>(thenVal), e = static_cast<VT>(elseVal);
    b200::check(db2_cond(call.c, &r, b200::dtype_of<VT>(), call.in(cond), nullptr, &t, nullptr, &e));
    if (!res)
        res = call.template wrap<VT>(r);
}
