// B200 implementation behind the name and signature of the reference's CPU kernel header of the same path
// (src/runtime/local/kernels/EwUnaryMat.h:41-46).  Elementwise unary operators have no CUDASupport trait in the
// reference's compiler, so they are always dispatched to backend "CPP"; registered from an extension catalog with
// priority >= 1 this wrapper keeps device-resident operands on the device.
#pragma once
#include <B200Adapter.h>
#include <runtime/local/kernels/UnaryOpCode.h>
template <class DTRes, class DTArg> void ewUnaryMat(UnaryOpCode opCode, DTRes *&res, const DTArg *arg, DCTX(ctx)) {
    b200::Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    b200::check(db2_ewUnaryMat(call.c, static_cast<int>(opCode), &r, call.in(arg)));
    if (!res)
        res = call.template wrap<typename DTRes::VT>(r);
}
