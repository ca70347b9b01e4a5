/* Stand-in for the six Win32 file-mapping calls the reference's GGUF reader makes (llm/gguf.cpp:79-91, :141-145), over
 * POSIX open / fstat / mmap, so that its reader compiles here unchanged.  Test infrastructure (oracle/_ref) only. */
#pragma once

#include <fcntl.h>
#include <stdint.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

typedef void* HANDLE;
typedef union {
    long long QuadPart;
} LARGE_INTEGER;
#define INVALID_HANDLE_VALUE ((HANDLE)(intptr_t)-1)
#define GENERIC_READ 0x80000000u
#define FILE_SHARE_READ 1u
#define OPEN_EXISTING 3u
#define FILE_ATTRIBUTE_NORMAL 0x80u
#define FILE_FLAG_SEQUENTIAL_SCAN 0x08000000u
#define PAGE_READONLY 2u
#define FILE_MAP_READ 4u

/* A file HANDLE is (fd + 1) so that fd 0 is not NULL; a mapping HANDLE is the same number tagged in bit 40. */
static inline HANDLE CreateFileA(const char* path, unsigned, unsigned, void*, unsigned, unsigned, void*) {
    const int fd = open(path, O_RDONLY);
    return fd < 0 ? INVALID_HANDLE_VALUE : (HANDLE)(intptr_t)(fd + 1);
}
static inline int GetFileSizeEx(HANDLE f, LARGE_INTEGER* out) {
    struct stat st;
    if (fstat((int)(intptr_t)f - 1, &st) != 0) return 0;
    out->QuadPart = st.st_size;
    return 1;
}
static inline HANDLE CreateFileMappingA(HANDLE f, void*, unsigned, unsigned, unsigned, const char*) {
    return (HANDLE)((intptr_t)f | ((intptr_t)1 << 40));
}
static inline void* MapViewOfFile(HANDLE m, unsigned, unsigned, unsigned, size_t) {
    const int fd = (int)((intptr_t)m & 0xFFFFFFFF) - 1;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size == 0) return 0;
    void* p = mmap(0, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    return p == MAP_FAILED ? 0 : p;
}
static inline int UnmapViewOfFile(const void*) { return 1; } /* the view lives until the process ends: sizes are not kept */
static inline int CloseHandle(HANDLE h) {
    if (((intptr_t)h >> 40) & 1) return 1; /* a mapping handle owns nothing */
    return close((int)(intptr_t)h - 1) == 0;
}
