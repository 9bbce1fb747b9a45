#pragma once
#include <spdlog/fmt/bundled/core.h>
