// B200 implementation behind the name and signature of the reference header of the same path
// (src/runtime/local/kernels/CUDA/AggCol.h): the generated extern "C" wrappers include it unchanged.
#pragma once
#include <B200Adapter.h>
#include <runtime/local/kernels/AggOpCode.h>
namespace CUDA {
template <class DTRes, class DTArg> void aggCol(AggOpCode opCode, DTRes *&res, const DTArg *arg, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_aggCol(call.c, static_cast<int>(opCode), &r, call.in(arg)));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
} // namespace CUDA
