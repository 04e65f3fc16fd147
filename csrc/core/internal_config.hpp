// Compile-time constants of the runtime (counterpart of the reference's
// src/common/internal-config.hpp:34-56, with bounded waits instead of endless ones).
#pragma once
#include <stdint.h>

namespace geeps_b200 {

constexpr int kInitialClock = 0;
constexpr int kInitialDataAge = -10000000;   // "nothing received yet"
constexpr int kBigIter = 10000000;
constexpr int kOpBufferSlots = 2;            // per-op hand-off slots: double buffering by clock parity
constexpr int kWatchdogSeconds = 12;         // period of "still waiting on X" diagnostics
constexpr unsigned kStopCmd = 0;             // work-queue command that stops a background worker
constexpr unsigned kIterateCmd = 1;          // work-queue command: push the updates of (clock, table)
constexpr unsigned kSnapshotCmd = 2;
constexpr size_t kLocalTableId = 0xdeadbeef; // table id recorded for LocalAccess ops
constexpr int kRowFloats = 128;
constexpr size_t kRowBytes = 512;

}  // namespace geeps_b200
