// Resolves the reference tree's <common/logger_text.h> include path to the single
// header this host library keeps its whole backend contract in.
#pragma once
#include "../clpeak_api.hpp"
