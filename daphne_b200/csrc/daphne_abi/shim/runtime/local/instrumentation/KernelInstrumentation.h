// Stand-in (outside a DAPHNE build tree): the hook points of the generated wrappers
// (src/runtime/local/instrumentation/KernelInstrumentation.cpp:19-27 start/stop the per-kernel timers).
#pragma once
struct DaphneContext;
inline void preKernelInstrumentation(int, DaphneContext *) {}
inline void postKernelInstrumentation(int, DaphneContext *) {}
