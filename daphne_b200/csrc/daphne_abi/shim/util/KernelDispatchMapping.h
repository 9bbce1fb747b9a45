#pragma once
struct KernelDispatchMapping {};
