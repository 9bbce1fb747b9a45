// Backend-"CPP" name of the full aggregation (src/runtime/local/kernels/AggAll.h:46-49): forwards to the device
// implementation.
#pragma once
#include <runtime/local/kernels/CUDA/AggAll.h>
template <typename VTRes, class DTArg> VTRes aggAll(AggOpCode opCode, const DTArg *arg, DCTX(ctx)) {
    return CUDA::aggAll<VTRes, DTArg>(opCode, arg, ctx);
}
