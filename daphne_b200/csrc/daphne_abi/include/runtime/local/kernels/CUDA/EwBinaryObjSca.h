// B200 implementation behind the name and signature of the reference header of the same path
// (src/runtime/local/kernels/CUDA/EwBinaryObjSca.h): the generated extern "C" wrappers include it unchanged.
#pragma once
#include <B200Adapter.h>
#include <runtime/local/kernels/BinaryOpCode.h>
namespace CUDA {
template <class DTRes, class DTLhs, typename VTRhs>
void ewBinaryObjSca(BinaryOpCode opCode, DTRes *&res, const DTLhs *lhs, VTRhs rhs, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    const typename DTLhs::VT s = static_cast<typename DTLhs::VT>(rhs);
    b200::check(db2_ewBinaryObjSca(call.c, static_cast<int>(opCode), &r, call.in(lhs), &s));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
} // namespace CUDA
