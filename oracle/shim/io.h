// Test scaffolding only: POSIX stand-in for the MSVC <io.h> names the reference's CLI uses.
#pragma once
#include <cstdio>
#define _O_BINARY 0
inline int _setmode(int, int) { return 0; }
inline int _fileno(FILE* f) { return fileno(f); }
