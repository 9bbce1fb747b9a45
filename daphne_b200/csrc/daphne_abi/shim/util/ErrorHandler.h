// Stand-in for util/ErrorHandler.h (outside a DAPHNE build tree): the real runtimeError() decorates the message with
// the kernel name and the script location (src/util/ErrorHandler.cpp:80-90).
#pragma once
#include <stdexcept>
#include <string>
#include <util/KernelDispatchMapping.h>
struct ErrorHandler {
    static std::runtime_error runtimeError(int kId, std::string msg, KernelDispatchMapping *) {
        return std::runtime_error("kernel " + std::to_string(kId) + ": " + msg);
    }
};
