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

/* runtime/model/SlotFile.cpp uses three Darwin fcntl commands: uncached IO (a hint: accepted and ignored here), a full
 * flush to the drive (fsync here) and hole punching (fallocate here). */
#ifndef F_NOCACHE
#include <fcntl.h>
#include <stdarg.h>
#include <unistd.h>
#define F_NOCACHE 0x7001
#define F_FULLFSYNC 0x7002
#define F_PUNCHHOLE 0x7003
typedef struct fpunchhole { unsigned int fp_flags; unsigned int reserved; off_t fp_offset; off_t fp_length; } fpunchhole_t;
static inline int rk_shim_fcntl(int descriptor, int command, ...) {
  va_list arguments;
  va_start(arguments, command);
  int result;
  if (command == F_NOCACHE) {
    result = 0;
  } else if (command == F_FULLFSYNC) {
    result = fsync(descriptor);
  } else if (command == F_PUNCHHOLE) {
    const fpunchhole_t *hole = va_arg(arguments, const fpunchhole_t *);
    result = fallocate(descriptor, FALLOC_FL_PUNCH_HOLE | FALLOC_FL_KEEP_SIZE, hole->fp_offset, hole->fp_length);
  } else {
    result = fcntl(descriptor, command, va_arg(arguments, long));
  }
  va_end(arguments);
  return result;
}
#define fcntl rk_shim_fcntl
#endif
