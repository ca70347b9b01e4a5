// Stand-in for MSVC's <intrin.h> so the reference's generated AVX2 kernels compile with g++.
// TEST INFRASTRUCTURE ONLY (used by oracle/Makefile when building oracle/_ref).
#pragma once
#include <cpuid.h>
#include <x86intrin.h>

#include <cstdlib>
#include <cstring>

#ifndef __cpuidex
#define __cpuidex(r, leaf, sub) __cpuid_count((leaf), (sub), (r)[0], (r)[1], (r)[2], (r)[3])
#endif
static inline void __debugbreak() { __builtin_trap(); }
static inline int _dupenv_s(char** value, size_t* len, const char* name) {
    const char* e = std::getenv(name);
    *value = e ? strdup(e) : nullptr;
    *len = e ? std::strlen(e) + 1 : 0;
    return 0;
}
