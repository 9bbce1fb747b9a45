#pragma once
#include <spdlog/fmt/bundled/format.h>
