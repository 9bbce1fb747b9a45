// B200 implementation behind the name and signature of the reference header of the same path
// (src/runtime/local/kernels/CUDA/ExtractCol.h): the generated extern "C" wrappers include it unchanged.
#pragma once
#include <B200Adapter.h>
namespace CUDA {
template <class DTRes, class DTArg, class DTSel>
void extractCol(DTRes *&res, const DTArg *arg, const DTSel *sel, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_extractCol(call.c, &r, call.in(arg), call.in(sel)));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
} // namespace CUDA
