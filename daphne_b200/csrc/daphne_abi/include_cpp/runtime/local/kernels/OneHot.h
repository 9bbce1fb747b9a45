// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/OneHot.h:43-46): per column keep / drop / expand into indicator columns.
#pragma once
#include <B200Adapter.h>
template <class DTRes, class DTArg>
void oneHot(DTRes *&res, const DTArg *arg, const DenseMatrix<int64_t> *info, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_oneHot(call.c, &r, call.in(arg), call.in(info)));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
