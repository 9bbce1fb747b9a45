// Backend-"CPP" name of the row aggregation (src/runtime/local/kernels/AggRow.h:44-48): forwards to the device
// implementation.  Registered for the opcodes the reference's compiler never tags for CUDA (IDXMIN, IDXMAX, MEAN, VAR,
// STDDEV, PROD) on dense arguments, and for SUM / MIN / MAX on CSRMatrix arguments (AggRow.h:178-238), which have no
// CUDA instantiation in the reference at all.
#pragma once
#include <B200Csr.h>
#include <runtime/local/kernels/CUDA/AggRow.h>
template <class DTRes, class DTArg> void aggRow(AggOpCode opCode, DTRes *&res, const DTArg *arg, DCTX(ctx)) {
    if constexpr (b200::is_csr<DTArg>::value)
        b200::csr_agg_row(opCode, res, arg, ctx);
    else
        CUDA::aggRow<DTRes, DTArg>(opCode, res, arg, ctx);
}
