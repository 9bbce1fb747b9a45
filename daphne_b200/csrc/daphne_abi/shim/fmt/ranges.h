#pragma once
#include <spdlog/fmt/bundled/ranges.h>
