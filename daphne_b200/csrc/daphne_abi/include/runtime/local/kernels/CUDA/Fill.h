// B200 implementation behind the name and signature of the reference header of the same path
// (src/runtime/local/kernels/CUDA/Fill.h): the generated extern "C" wrappers include it unchanged.
#pragma once
#include <B200Adapter.h>
namespace CUDA {
template <class DTRes, typename VTArg> void fill(DTRes *&res, VTArg arg, size_t numRows, size_t numCols, DCTX(ctx)) {
    using VT = typename DTRes::VT;
    b200::require_supported<VT>("fill");
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    const VT v = static_cast<VT>(arg);
    b200::check(db2_fill(call.c, &r, b200::dtype_of<VT>(), &v, (int64_t)numRows, (int64_t)numCols));
    if (!res)
        res = call.template wrap<VT>(r);
}
} // namespace CUDA
