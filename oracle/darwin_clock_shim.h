/* Force-included when compiling the reference's portable sources on Linux:
 * runtime/AwakeClock.hpp reads Darwin's awake-time clock. */
#pragma once
#include <stdint.h>
#include <time.h>
#ifndef CLOCK_UPTIME_RAW
#define CLOCK_UPTIME_RAW CLOCK_MONOTONIC
static inline uint64_t clock_gettime_nsec_np(clockid_t id) {
  struct timespec t;
  clock_gettime(id, &t);
  return (uint64_t)t.tv_sec * 1000000000ull + (uint64_t)t.tv_nsec;
}
#endif
