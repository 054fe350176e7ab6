// Memory patterns and buffer-reuse planning.
//
// The first run of a session with a given set of input shapes records, per intermediate value, how many bytes its
// producer allocated, where it lives and between which two steps it is alive (its producer and the step whose
// release list frees it).  From those lifetimes the planner packs the values into one arena per device: a value
// takes the lowest offset that is free during its whole lifetime (largest values first), so two values whose
// lifetimes do not overlap share memory.  The result answers "how large an arena would serve this pattern without a
// single allocation" (peak) against "what the producers asked for in total" and against the lower bound (the most
// bytes alive at one step); InferenceSession.get_memory_plans() reports it.  The arena that serves the requests is
// the torch caching allocator: after the first run of a pattern it hands out the same blocks from its pool without
// calling the driver, and a captured CUDA graph replays with the addresses of its private pool.
//
// Counterparts in the reference: onnxruntime/core/framework/allocation_planner.cc (static reuse plan),
// mem_pattern_planner.h (OrtValuePatternPlanner::TraceAllocation, first run traced, later runs served from one
// block) and bfc_arena.cc (the arena the block comes from; here the arena is the torch caching allocator).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace ortb {

struct PlannedBuffer {
  std::string name;
  int64_t bytes = 0;     // rounded up to the allocation granularity
  int first_step = 0;    // producer
  int last_step = 0;     // last consumer (inclusive)
  bool on_gpu = false;
  int64_t offset = -1;   // assigned by PlanBuffers
};

struct MemoryPlan {
  std::string pattern;   // input shapes this plan belongs to
  std::vector<PlannedBuffer> buffers;
  // index 0: host, 1: device
  int64_t peak_bytes[2] = {0, 0};    // arena size that serves the pattern
  int64_t total_bytes[2] = {0, 0};   // sum of all requests (no reuse)
  int64_t live_peak_bytes[2] = {0, 0};  // largest sum of simultaneously live values: lower bound for any plan
  int num_reused[2] = {0, 0};        // values placed on memory another value used before
};

constexpr int64_t kPlanAlignment = 256;
inline int64_t AlignPlanBytes(int64_t n) { return (n + kPlanAlignment - 1) / kPlanAlignment * kPlanAlignment; }

// Assigns offsets.  Values with bytes == 0 (views of other values) keep offset -1.
MemoryPlan PlanBuffers(std::vector<PlannedBuffer> buffers, const std::string& pattern);

// Checks that no two values with overlapping lifetimes overlap in memory (used by tests and debug builds).
bool PlanIsValid(const MemoryPlan& plan, std::string* why);

}  // namespace ortb
