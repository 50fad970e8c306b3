// Stand-in for gemma.c's src/gemma4_runtime.cuh:12-64 (Gemma4RuntimeState and its
// four functions); see gemma4_kv_cache.cuh beside this file. The reference's
// header also brings in the model constants of src/gemma4.h, so this one does
// too when that file is on the include path.
#pragma once
#if defined(__has_include)
#if __has_include("gemma4.h")
#include "gemma4.h"
#endif
#endif
#include "../gemma4_b200kv.hpp"
