// Backend-"CPP" name of the column aggregation (src/runtime/local/kernels/AggCol.h:44-48): forwards to the device
// implementation (MEAN, VAR, STDDEV, IDXMIN and IDXMAX are never tagged for CUDA by the reference's compiler).
#pragma once
#include <runtime/local/kernels/CUDA/AggCol.h>
template <class DTRes, class DTArg> void aggCol(AggOpCode opCode, DTRes *&res, const DTArg *arg, DCTX(ctx)) {
    CUDA::aggCol<DTRes, DTArg>(opCode, res, arg, ctx);
}
