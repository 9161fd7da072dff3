// Status block shared by every kernel family of the library (see status.cu).
#pragma once
#include <cstring>
#include "common.cuh"

enum : int { EXO_STATUS_TC = 0, EXO_STATUS_GEMV = 1, EXO_STATUS_COMM = 2 };

// Device-writable pointer to status word `which` of the current device (allocated on first use, which must not
// happen inside a stream capture); nullptr on failure.
int* exo_status_word(int which);
int* exo_status_block();
// Wait budget of the peer-memory collectives in nanoseconds (set by exo_set_collective_timeout_us).
unsigned long long exo_wait_budget_ns();
// Reads (clear != 0: and clears) status word `which` from host memory.
extern "C" int exo_status_take(int which, int clear);
