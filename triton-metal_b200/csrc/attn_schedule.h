// Work lists of the persistent attention kernels (host side).
//
// A persistent kernel runs one CTA per SM; every CTA walks its own list of work items.  An
// item is one block of resident rows of one (batch, head): 256 query rows for the forward, 128
// query rows for dq, 128 key rows for dkdv.  Under a causal mask the items differ in cost (a
// late query block sees many key blocks, an early one few), and with few (batch, head) slices
// - a shard of a job spread over eight GPUs - there are about as many items as SMs, so how they
// are dealt out decides how many SMs idle at the end.
//
// Two ways of dealing the items out are built for every shape and the one that finishes
// earlier by the cost model is used: equal-cost units in rounds (best use of L2, but whole
// rounds only) and list scheduling onto the least-loaded CTA (level finishing times for any
// number of heads).  See schedule_rounds / schedule_least_loaded below.
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
// Equal-cost units dealt round-robin: under a causal mask the long block k of a head is paired
// with the short block n-1-k, so that every unit costs the same; unit u goes to CTA u mod ctas.
// The CTAs then move through the heads in step - the units of a head run side by side and
// stream the same rows at the same time, which is the best use of L2 there is - but the number
// of units is rounded up to whole rounds: with few heads up to half a round of SMs idles.
inline AttnWorkList schedule_rounds(int bh, int blocks, int ctas, const std::function<int(int)>& cost,
                                    int overhead) {
  AttnWorkList out;
  const bool varying = cost(0) != cost(blocks - 1);
  const bool long_last = cost(blocks - 1) > cost(0);
  const int units = varying ? (blocks + 1) / 2 : blocks;
  std::vector<std::vector<AttnWorkItem>> per_cta(ctas);
  int u = 0;
  for (int h = 0; h < bh; ++h) {
    for (int k = 0; k < units; ++k, ++u) {
      auto& list = per_cta[u % ctas];
      if (!varying) {
        list.push_back({h, k});
        continue;
      }
      const int far = blocks - 1 - k;
      const int first = long_last ? far : k, second = long_last ? k : far;     // the long block first
      list.push_back({h, first});
      if (second != first) list.push_back({h, second});
    }
  }
  out.load.assign(ctas, 0);
  out.begin.push_back(0);
  for (int c = 0; c < ctas; ++c) {
    for (const AttnWorkItem& item : per_cta[c]) out.load[c] += cost(item.block) + overhead;
    out.items.insert(out.items.end(), per_cta[c].begin(), per_cta[c].end());
    out.begin.push_back((int32_t)out.items.size());
  }
  return out;
}

// List scheduling: items in (batch, head)-major order, the long ones of a head first, each to the
// CTA with the least work so far; the last whole heads holding at most three items per CTA are
// dealt longest first whatever their head.  Levels the finishing times for any number of heads.
inline AttnWorkList schedule_least_loaded(int bh, int blocks, int ctas, const std::function<int(int)>& cost,
                                          int overhead) {
  AttnWorkList out;
  std::vector<int> order(blocks);
  for (int i = 0; i < blocks; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return cost(a) > cost(b); });
  std::vector<AttnWorkItem> sequence;
  sequence.reserve((size_t)bh * blocks);
  for (int h = 0; h < bh; ++h)
    for (int b : order) sequence.push_back({h, b});
  const int tail_heads = std::max(1, std::min(bh, (3 * ctas) / std::max(1, blocks)));
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

// `blocks` items per slice; cost(block) is the number of streamed blocks the item walks;
// `overhead` is what an item costs on top (pipeline fill and drain, the output pass), in the
// same unit.  Both schedules are built and the one with the shorter modelled finishing time is
// taken; rounds win ties and near-ties (measured on a B200: with 128 heads of 4096 rows the
// kernels run 2 to 8 per cent faster on rounds than on an equally balanced list, for the
// lockstep use of L2; with 16 heads the list is 10 per cent ahead).
inline AttnWorkList schedule_attention(int bh, int blocks, int ctas, const std::function<int(int)>& cost,
                                       int overhead) {
  ctas = (int)std::max<int64_t>(1, std::min<int64_t>(ctas, (int64_t)bh * blocks));
  AttnWorkList rounds = schedule_rounds(bh, blocks, ctas, cost, overhead);
  AttnWorkList list = schedule_least_loaded(bh, blocks, ctas, cost, overhead);
  const int64_t t_rounds = *std::max_element(rounds.load.begin(), rounds.load.end());
  const int64_t t_list = *std::max_element(list.load.begin(), list.load.end());
  return t_rounds * 100 <= t_list * 105 ? rounds : list;
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

#ifdef __CUDACC__
// A CTA's walk over its list, with the next item fetched one item ahead: the fetch is a
// dependent global load of several hundred cycles, and every role of the kernel would otherwise
// wait for it at the top of each item - the loading warp before it can ask for the item's first
// tiles, the issuing warp before its first MMA.
struct WorkCursor {
  const int2* items;
  int it, end;
  int2 cur, nxt;      // (batch-head, block) of item `it` and of item `it + 1`
  __device__ __forceinline__ explicit WorkCursor(const DeviceWorkList& w)
      : items(reinterpret_cast<const int2*>(w.items)) {
    it = __ldg(w.begin + blockIdx.x);
    end = __ldg(w.begin + blockIdx.x + 1);
    cur = it < end ? __ldg(items + it) : make_int2(0, 0);
    nxt = it + 1 < end ? __ldg(items + it + 1) : cur;
  }
  __device__ __forceinline__ bool valid() const { return it < end; }
  __device__ __forceinline__ void advance() {
    ++it;
    cur = nxt;
    if (it + 1 < end) nxt = __ldg(items + it + 1);
  }
};
#endif

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
