// Stand-in for gemma.c's src/gemma4_kv_cache.cuh:9-66. Put this directory ahead
// of gemma.c's src/ on the include path (-I<b200kv>/include/compat -I<gemma.c>/src)
// and a translation unit that says #include "gemma4_kv_cache.cuh" gets the same
// types and functions, declared by the B200 library's header; it then links to
// libgemma4_b200kv.so instead of gemma4_kv_cache.cu. (Files inside gemma.c's
// src/ find their neighbours first and keep using the reference's own headers,
// which is fine: the layouts are identical, see gemma4_b200kv.hpp.)
#pragma once
#include "../gemma4_b200kv.hpp"
