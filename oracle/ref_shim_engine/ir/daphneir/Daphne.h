// TEST INFRASTRUCTURE.  The two enums of the DaphneIR dialect that the vectorized engine uses
// (src/ir/daphneir/DaphneVectorizableOpInterface.td:23-36), without MLIR.
#pragma once
#include <cstdint>
#include <cstdlib>
namespace mlir::daphne {
enum class VectorSplit : int64_t { NONE = 0, ROWS = 1 };
enum class VectorCombine : int64_t { ROWS = 1, COLS = 2, ADD = 3, MIN = 4, MAX = 5 };
} // namespace mlir::daphne
#ifndef llvm_unreachable
#define llvm_unreachable(msg) abort()
#endif
#ifndef LLVM_FALLTHROUGH
#define LLVM_FALLTHROUGH [[fallthrough]]
#endif
