// Stand-in used ONLY when the adapter is built outside a DAPHNE build tree (this repository's own build and tests):
// the real header pulls in MLIR through DaphneUserConfig.h.  It carries the members the generated wrappers touch.
#pragma once
#include <util/KernelDispatchMapping.h>
struct DaphneContext {
    KernelDispatchMapping dispatchMapping;
};
#define DCTX(varname) DaphneContext *varname
