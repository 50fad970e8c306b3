// Stand-in for gemma.c's src/gemma4_flash_attention.cuh:9-45 (the two prompt
// attention entry points); see gemma4_kv_cache.cuh beside this file.
#pragma once
#include "../gemma4_b200kv.hpp"
