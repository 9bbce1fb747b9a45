// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/AggCum.h:39-42): cumulative aggregation down the rows of every column.
#pragma once
#include <B200Adapter.h>
#include <runtime/local/kernels/AggOpCode.h>
template <class DTRes, class DTArg> void aggCum(AggOpCode opCode, DTRes *&res, const DTArg *arg, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_aggCum(call.c, static_cast<int>(opCode), &r, call.in(arg)));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
