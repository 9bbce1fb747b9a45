// Backend-"CPP" name of the row aggregation (src/runtime/local/kernels/AggRow.h:44-48) for the opcodes the reference's
// compiler never tags for CUDA (IDXMIN, IDXMAX, MEAN, VAR, STDDEV, PROD): forwards to the device implementation.
#pragma once
#include <runtime/local/kernels/CUDA/AggRow.h>
template <class DTRes, class DTArg> void aggRow(AggOpCode opCode, DTRes *&res, const DTArg *arg, DCTX(ctx)) {
    CUDA::aggRow<DTRes, DTArg>(opCode, res, arg, ctx);
}
