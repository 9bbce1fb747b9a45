// B200 implementation behind the name and signature of the reference header of the same path
// (src/runtime/local/kernels/CUDA/AggAll.h): the generated extern "C" wrappers include it unchanged.
#pragma once
#include <B200Adapter.h>
#include <runtime/local/kernels/AggOpCode.h>
namespace CUDA {
template <typename VTRes, class DTArg> VTRes aggAll(AggOpCode opCode, const DTArg *arg, DCTX(ctx)) {
    b200::Call call(ctx);
    typename DTArg::VT v{};
    b200::check(db2_aggAll(call.c, static_cast<int>(opCode), &v, call.in(arg)));
    return static_cast<VTRes>(v);
}
} // namespace CUDA
