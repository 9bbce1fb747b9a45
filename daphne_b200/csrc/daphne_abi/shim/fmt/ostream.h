#pragma once
#include <spdlog/fmt/bundled/ostream.h>
