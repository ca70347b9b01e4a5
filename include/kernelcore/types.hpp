// Part of the consolidated host API header (kept so reference include paths resolve).
#pragma once
#include <kernelcore/api.hpp>
