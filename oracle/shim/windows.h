// Test scaffolding only: a POSIX stand-in for the handful of Win32 file-mapping calls that the
// reference's GGUF reader uses, so that its unmodified sources compile on Linux for the oracle.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <string>

struct ElShimHandle {
    int fd = -1;
    uint64_t size = 0;
};
using HANDLE = ElShimHandle*;
#define INVALID_HANDLE_VALUE (reinterpret_cast<HANDLE>(intptr_t(-1)))
struct LARGE_INTEGER {
    long long QuadPart;
};
using DWORD = unsigned long;
using BOOL = int;
using LPCWSTR = const wchar_t*;

constexpr unsigned CP_UTF8 = 65001, MB_ERR_INVALID_CHARS = 8;
constexpr DWORD GENERIC_READ = 0x80000000ul, FILE_SHARE_READ = 1, OPEN_EXISTING = 3;
constexpr DWORD FILE_ATTRIBUTE_NORMAL = 0x80, FILE_FLAG_RANDOM_ACCESS = 0x10000000ul;
constexpr DWORD PAGE_READONLY = 2, FILE_MAP_READ = 4;

// The path stays UTF-8 on POSIX: each byte is widened to one wchar_t and narrowed back in CreateFileW.
inline int MultiByteToWideChar(unsigned, DWORD, const char* src, int, wchar_t* dst, int dst_len) {
    const int need = int(std::strlen(src)) + 1;
    if (!dst || dst_len == 0) return need;
    if (dst_len < need) return 0;
    for (int i = 0; i < need; ++i) dst[i] = wchar_t(static_cast<unsigned char>(src[i]));
    return need;
}
inline HANDLE CreateFileW(LPCWSTR wpath, DWORD, DWORD, void*, DWORD, DWORD, void*) {
    std::string p;
    for (const wchar_t* c = wpath; *c; ++c) p.push_back(char(*c));
    const int fd = ::open(p.c_str(), O_RDONLY);
    if (fd < 0) return INVALID_HANDLE_VALUE;
    struct stat st {};
    if (::fstat(fd, &st) != 0) {
        ::close(fd);
        return INVALID_HANDLE_VALUE;
    }
    auto* h = new ElShimHandle;
    h->fd = fd;
    h->size = uint64_t(st.st_size);
    return h;
}
inline BOOL GetFileSizeEx(HANDLE h, LARGE_INTEGER* out) {
    out->QuadPart = (long long)h->size;
    return 1;
}
inline HANDLE CreateFileMappingW(HANDLE file, void*, DWORD, DWORD, DWORD, void*) {
    auto* m = new ElShimHandle;
    m->fd = file->fd;
    m->size = file->size;
    return m;
}
inline void* MapViewOfFile(HANDLE map, DWORD, DWORD, DWORD, size_t) {
    void* p = ::mmap(nullptr, map->size, PROT_READ, MAP_PRIVATE, map->fd, 0);
    return p == MAP_FAILED ? nullptr : p;
}
// The oracle keeps its few mappings until the process exits; file descriptors likewise.
inline BOOL UnmapViewOfFile(const void*) { return 1; }
inline BOOL CloseHandle(HANDLE h) {
    if (h && h != INVALID_HANDLE_VALUE) {
        delete h;
    }
    return 1;
}
