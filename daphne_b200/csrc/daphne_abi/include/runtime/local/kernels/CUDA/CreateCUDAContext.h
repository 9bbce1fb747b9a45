// B200 implementation behind the name and signature of the reference header of the same path
// (src/runtime/local/kernels/CUDA/CreateCUDAContext.h): the generated extern "C" wrappers include it unchanged.
#pragma once
#include <B200Adapter.h>
namespace CUDA {
// creates the device context(s) of this DaphneContext (the reference creates exactly one, for device 0:
// src/runtime/local/kernels/CUDA/CreateCUDAContext.cpp:4-9)
inline void createCUDAContext(DCTX(ctx)) { b200::create_context(ctx); }
} // namespace CUDA
