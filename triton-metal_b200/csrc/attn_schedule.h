// Work lists of the persistent attention kernels (host side).
//
// A persistent kernel runs one CTA per SM; every CTA walks its own list of work items.  An
// item is one block of resident rows of one (batch, head): 256 query rows for the forward, 128
// query rows for dq, 128 key rows for dkdv.  Under a causal mask the items differ in cost (a
// late query block sees many key blocks, an early one few), and with few (batch, head) slices
// - a shard of a job spread over eight GPUs - there are about as many items as SMs, so how they
// are dealt out decides how many SMs idle at the end.
//
// The lists are built by list scheduling: items are taken in (batch, head)-major order, the
// long ones of a head first, and each goes to the CTA with the least work so far.  Because
// items are handed out in order, the CTAs that run at the same time work on the same few
// heads, whose streamed tensors they share in L2.  The last items - about three per CTA, whole
// heads - are dealt longest first regardless of their head (the classic longest-processing-time
// rule), which is what levels the finishing times; with few heads that is the whole list.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstdint>
#include <functional>
#include <list>
#include <mutex>
#include <queue>
#include <string>
#include <vector>

namespace tmc {

struct AttnWorkItem {
  int32_t bh;      // (batch, head) slice
  int32_t block;   // index of the block of resident rows inside the slice
};

struct AttnWorkList {
  std::vector<AttnWorkItem> items;   // CTA c owns items[begin[c] ... begin[c + 1])
  std::vector<int32_t> begin;        // ctas + 1 entries
  std::vector<int64_t> load;         // cost assigned to each CTA (for tests and tuning)
};

// `blocks` items per slice; cost(block) is the number of streamed blocks the item walks;
// `overhead` is what an item costs on top (pipeline fill and drain, the output pass), in the
// same unit.  Within a slice the items are issued in order of decreasing cost.
inline AttnWorkList schedule_attention(int bh, int blocks, int ctas, const std::function<int(int)>& cost,
                                       int overhead) {
  AttnWorkList out;
  ctas = (int)std::max<int64_t>(1, std::min<int64_t>(ctas, (int64_t)bh * blocks));
  if (const char* mode = std::getenv("TMCUDA_SCHED")) {
    if (std::string(mode) == "pairs") {
      // experimental: long block paired with a short one, units dealt round-robin
      std::vector<std::vector<AttnWorkItem>> per(ctas);
      const bool varying = cost(0) != cost(blocks - 1);
      const int units = varying ? (blocks + 1) / 2 : blocks;
      const bool long_last = cost(blocks - 1) > cost(0);
      int u = 0;
      for (int h = 0; h < bh; ++h)
        for (int k = 0; k < units; ++k, ++u) {
          auto& lst = per[u % ctas];
          if (!varying) { lst.push_back({h, k}); continue; }
          const int far = blocks - 1 - k;
          const int first = long_last ? far : k, second = long_last ? k : far;
          lst.push_back({h, first});
          if (second != first) lst.push_back({h, second});
        }
      out.load.assign(ctas, 0);
      out.begin.push_back(0);
      for (int c = 0; c < ctas; ++c) {
        for (auto& it : per[c]) out.load[c] += cost(it.block) + overhead;
        out.items.insert(out.items.end(), per[c].begin(), per[c].end());
        out.begin.push_back((int32_t)out.items.size());
      }
      return out;
    }
  }
  std::vector<int> order(blocks);
  for (int i = 0; i < blocks; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost(a) > cost(b); });
  int tail_tenths = 30, order_mode = 0;
  if (const char* e = std::getenv("TMCUDA_SCHED_TAIL")) tail_tenths = std::atoi(e);
  if (const char* e = std::getenv("TMCUDA_SCHED_ORDER")) order_mode = std::atoi(e);
  if (order_mode == 1) std::reverse(order.begin(), order.end());
  if (order_mode == 2) {   // heavy, light, second heaviest, second lightest, ...
    std::vector<int> mixed;
    for (int i = 0, j = blocks - 1; i <= j; ++i, --j) {
      mixed.push_back(order[i]);
      if (i != j) mixed.push_back(order[j]);
    }
    order = mixed;
  }
  std::vector<AttnWorkItem> sequence;
  sequence.reserve((size_t)bh * blocks);
  for (int h = 0; h < bh; ++h)
    for (int b : order) sequence.push_back({h, b});
  // the tail: the last whole heads that hold at most 3 items per CTA (at least one head)
  const int tail_heads = std::max(1, std::min(bh, (tail_tenths * ctas / 10) / std::max(1, blocks)));
  const size_t tail_start = (size_t)(bh - tail_heads) * blocks;
  std::stable_sort(sequence.begin() + tail_start, sequence.end(),
                   [&](const AttnWorkItem& a, const AttnWorkItem& b) { return cost(a.block) > cost(b.block); });
  std::vector<std::vector<AttnWorkItem>> per_cta(ctas);
  out.load.assign(ctas, 0);
  // least-loaded CTA first; ties go to the lower index
  using Entry = std::pair<int64_t, int>;
  std::priority_queue<Entry, std::vector<Entry>, std::greater<Entry>> heap;
  for (int c = 0; c < ctas; ++c) heap.push({0, c});
  for (const AttnWorkItem& item : sequence) {
    Entry e = heap.top();
    heap.pop();
    per_cta[e.second].push_back(item);
    e.first += cost(item.block) + overhead;
    out.load[e.second] = e.first;
    heap.push(e);
  }
  out.begin.reserve(ctas + 1);
  out.begin.push_back(0);
  for (int c = 0; c < ctas; ++c) {
    out.items.insert(out.items.end(), per_cta[c].begin(), per_cta[c].end());
    out.begin.push_back((int32_t)out.items.size());
  }
  return out;
}

// Forward: 256-row query blocks; a block starting at row m0 walks ceil(min(n_ctx, m0 + 256) / 128)
// key blocks under a causal mask, all of them otherwise.
inline AttnWorkList schedule_attn_fwd(int bh, int rows, int n_ctx, bool causal, int ctas) {
  const int blocks = (rows + 255) / 256;
  const int all = (n_ctx + 127) / 128;
  auto cost = [=](int b) { return causal ? std::min(all, (std::min(n_ctx, (b + 1) * 256) + 127) / 128) : all; };
  return schedule_attention(bh, blocks, ctas, cost, 3);
}

// Backward: 128-row tiles.  dq (long_last): query tile i walks i + 1 key blocks under a causal
// mask; dkdv: key tile i is walked by the query blocks from i on.
inline AttnWorkList schedule_attn_bwd(int bh, int rows, int n_ctx, bool causal, bool long_last, int ctas) {
  const int tiles = (rows + 127) / 128;
  const int all = (n_ctx + 127) / 128;
  auto cost = [=](int b) {
    if (!causal) return all;
    return long_last ? std::min(all, b + 1) : std::max(1, all - b);
  };
  return schedule_attention(bh, tiles, ctas, cost, 2);
}

// A work list in device memory.
struct DeviceWorkList {
  const AttnWorkItem* items = nullptr;
  const int32_t* begin = nullptr;
  int ctas = 0;
};

// Work lists already uploaded, by problem shape: a list depends only on (kind, slices, rows,
// n_ctx, mask, CTAs), so a training loop or a benchmark builds and uploads it once.  A few
// entries are kept per device context; the oldest is dropped (after the stream has drained)
// when a new shape arrives.
class WorkListCache {
 public:
  struct Key {
    int kind, bh, rows, n_ctx, causal, ctas;
    bool operator==(const Key& o) const {
      return kind == o.kind && bh == o.bh && rows == o.rows && n_ctx == o.n_ctx && causal == o.causal && ctas == o.ctas;
    }
  };
  // Returns the device list for `key`, building it with `build` on a miss.  Empty `error` on success.
  DeviceWorkList get(const Key& key, const std::function<AttnWorkList()>& build, cudaStream_t stream,
                     std::string& error) {
    std::lock_guard<std::mutex> guard(lock_);
    for (auto it = entries_.begin(); it != entries_.end(); ++it) {
      if (it->key == key) {
        entries_.splice(entries_.begin(), entries_, it);      // most recently used first
        return entries_.front().list;
      }
    }
    if (entries_.size() >= kEntries) {
      cudaStreamSynchronize(stream);                            // a launch may still be reading it
      cudaFree(entries_.back().memory);
      entries_.pop_back();
    }
    AttnWorkList host = build();
    const size_t item_bytes = host.items.size() * sizeof(AttnWorkItem);
    const size_t begin_bytes = host.begin.size() * sizeof(int32_t);
    Entry e;
    e.key = key;
    cudaError_t err = cudaMalloc(&e.memory, item_bytes + begin_bytes);
    if (err != cudaSuccess) {
      cudaGetLastError();
      error = std::string("could not allocate an attention work list: ") + cudaGetErrorString(err);
      return DeviceWorkList();
    }
    // pageable sources: both copies have left host memory when the calls return
    cudaMemcpyAsync(e.memory, host.items.data(), item_bytes, cudaMemcpyHostToDevice, stream);
    cudaMemcpyAsync((char*)e.memory + item_bytes, host.begin.data(), begin_bytes, cudaMemcpyHostToDevice, stream);
    e.list.items = (const AttnWorkItem*)e.memory;
    e.list.begin = (const int32_t*)((char*)e.memory + item_bytes);
    e.list.ctas = (int)host.begin.size() - 1;
    entries_.push_front(e);
    return e.list;
  }

 private:
  static constexpr size_t kEntries = 12;
  struct Entry {
    Key key;
    void* memory = nullptr;
    DeviceWorkList list;
  };
  std::mutex lock_;
  std::list<Entry> entries_;
};

}  // namespace tmc
