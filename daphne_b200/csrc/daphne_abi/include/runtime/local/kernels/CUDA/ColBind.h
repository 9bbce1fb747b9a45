// B200 implementation behind the name and signature of the reference header of the same path
// (src/runtime/local/kernels/CUDA/ColBind.h): the generated extern "C" wrappers include it unchanged.
#pragma once
#include <B200Adapter.h>
namespace CUDA {
template <class DTRes, class DTLhs, class DTRhs>
void colBind(DTRes *&res, const DTLhs *lhs, const DTRhs *rhs, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_colBind(call.c, &r, call.in(lhs), call.in(rhs)));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
} // namespace CUDA
