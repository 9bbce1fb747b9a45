// Shim used only when the reference's CPU kernels are compiled as the test oracle (oracle/_ref): the kernels take a
// DaphneContext* but the ones built here never dereference it, so a forward declaration is all they need.
#pragma once
struct DaphneContext;
#define DCTX(varname) DaphneContext *varname
