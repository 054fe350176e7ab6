#include "allocation_planner.h"

#include <algorithm>
#include <numeric>

namespace ortb {

namespace {

bool LifetimesOverlap(const PlannedBuffer& a, const PlannedBuffer& b) {
  return a.first_step <= b.last_step && b.first_step <= a.last_step;
}

}  // namespace

MemoryPlan PlanBuffers(std::vector<PlannedBuffer> buffers, const std::string& pattern) {
  MemoryPlan plan;
  plan.pattern = pattern;
  for (auto& b : buffers) {
    b.bytes = b.bytes > 0 ? AlignPlanBytes(b.bytes) : 0;
    b.offset = -1;
  }
  for (int dev = 0; dev < 2; ++dev) {
    std::vector<size_t> order;
    int max_step = 0;
    for (size_t i = 0; i < buffers.size(); ++i) {
      if (buffers[i].on_gpu != (dev == 1) || buffers[i].bytes == 0) continue;
      order.push_back(i);
      plan.total_bytes[dev] += buffers[i].bytes;
      max_step = std::max(max_step, buffers[i].last_step);
    }
    // lower bound: the largest amount alive at one step
    std::vector<int64_t> live(static_cast<size_t>(max_step) + 2, 0);
    for (size_t i : order) {
      live[static_cast<size_t>(buffers[i].first_step)] += buffers[i].bytes;
      live[static_cast<size_t>(buffers[i].last_step) + 1] -= buffers[i].bytes;
    }
    int64_t running = 0;
    for (int64_t d : live) {
      running += d;
      plan.live_peak_bytes[dev] = std::max(plan.live_peak_bytes[dev], running);
    }
    // largest first; ties by earlier producer, so the order is deterministic
    std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
      if (buffers[a].bytes != buffers[b].bytes) return buffers[a].bytes > buffers[b].bytes;
      return buffers[a].first_step < buffers[b].first_step;
    });
    std::vector<size_t> placed;
    for (size_t i : order) {
      // occupied intervals during this value's lifetime, by offset
      std::vector<std::pair<int64_t, int64_t>> busy;
      for (size_t j : placed)
        if (LifetimesOverlap(buffers[i], buffers[j])) busy.emplace_back(buffers[j].offset, buffers[j].offset + buffers[j].bytes);
      std::sort(busy.begin(), busy.end());
      int64_t offset = 0;
      for (auto& iv : busy) {
        if (iv.first - offset >= buffers[i].bytes) break;  // the gap in front of this interval fits
        offset = std::max(offset, iv.second);
      }
      buffers[i].offset = offset;
      if (offset + buffers[i].bytes <= plan.peak_bytes[dev]) {
        // inside the arena as it stands: some earlier value's memory (or a hole between values) is used again
        ++plan.num_reused[dev];
      }
      plan.peak_bytes[dev] = std::max(plan.peak_bytes[dev], offset + buffers[i].bytes);
      placed.push_back(i);
    }
  }
  plan.buffers = std::move(buffers);
  return plan;
}

bool PlanIsValid(const MemoryPlan& plan, std::string* why) {
  const auto& b = plan.buffers;
  for (size_t i = 0; i < b.size(); ++i) {
    if (b[i].bytes == 0) continue;
    if (b[i].offset < 0 || b[i].offset % kPlanAlignment != 0) {
      if (why) *why = "value '" + b[i].name + "' has no aligned offset";
      return false;
    }
    if (b[i].offset + b[i].bytes > plan.peak_bytes[b[i].on_gpu ? 1 : 0]) {
      if (why) *why = "value '" + b[i].name + "' ends beyond the arena";
      return false;
    }
    for (size_t j = i + 1; j < b.size(); ++j) {
      if (b[j].bytes == 0 || b[i].on_gpu != b[j].on_gpu || !LifetimesOverlap(b[i], b[j])) continue;
      if (b[i].offset < b[j].offset + b[j].bytes && b[j].offset < b[i].offset + b[i].bytes) {
        if (why) *why = "values '" + b[i].name + "' and '" + b[j].name + "' are alive together and overlap in memory";
        return false;
      }
    }
  }
  return true;
}

}  // namespace ortb
