// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/OuterBinary.h:41-44): res[r][c] = lhs[r] (op) rhs[c].
#pragma once
#include <B200Adapter.h>
#include <runtime/local/kernels/BinaryOpCode.h>
template <class DTRes, class DTLhs, class DTRhs>
void outerBinary(BinaryOpCode opCode, DTRes *&res, const DTLhs *lhs, const DTRhs *rhs, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_outerBinary(call.c, static_cast<int>(opCode), &r, call.in(lhs), call.in(rhs)));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
