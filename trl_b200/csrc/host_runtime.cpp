// Host runtime (C ABI, loaded through ctypes):
//
//  * BlockPool   - reference-counted allocator of paged-KV blocks (prefix sharing between the
//                  completions sampled from one prompt).
//  * Scheduler   - continuous-batching scheduler of the rollout engine: waiting queue, running
//                  slots, admission under a block budget, retirement, slot reuse.
//  * bfd_assign  - best-fit-decreasing sequence packing (segment-tree search), the same
//                  assignment as trl/data_utils.py:739-826 computes on Arrow tables.
//
// The reference delegates all three to external native code (vLLM's scheduler/block manager,
// pyarrow); there is no counterpart inside its own tree.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <numeric>
#include <unordered_map>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {

struct BlockPool {
  std::vector<int32_t> refcnt;
  std::vector<int32_t> free_list;
  explicit BlockPool(int n) : refcnt(n, 0) {
    free_list.reserve(n);
    for (int i = n - 1; i >= 0; --i) free_list.push_back(i);
  }
  int num_free() const { return (int)free_list.size(); }
  int alloc() {
    if (free_list.empty()) return -1;
    int b = free_list.back();
    free_list.pop_back();
    refcnt[b] = 1;
    return b;
  }
  void retain(int b) { ++refcnt[b]; }
  void release(int b) {
    if (b < 0) return;
    if (--refcnt[b] == 0) free_list.push_back(b);
  }
};

struct Request {
  int64_t id;
  int32_t prompt_len;
  int32_t max_new;
  int64_t group;  // requests of one group share their prompt (prefix) blocks
};

struct Running {
  int64_t id = -1;
  std::vector<int32_t> blocks;
};

struct Scheduler {
  int max_slots, block_size, max_blocks_per_seq;
  BlockPool pool;
  std::deque<Request> waiting;
  std::vector<Running> slots;
  // group -> shared full prompt blocks (kept alive while any member of the group is waiting/running)
  struct Shared { std::vector<int32_t> blocks; int users = 0; bool prefilled = false; int32_t tail_block = -1; };
  std::unordered_map<int64_t, Shared> shared;
  std::unordered_map<int64_t, int> group_pending;  // members not yet retired
  std::mutex mu;

  Scheduler(int slots_, int nblocks, int bs, int mbps)
      : max_slots(slots_), block_size(bs), max_blocks_per_seq(mbps), pool(nblocks), slots(slots_) {}

  int blocks_needed(const Request& r, bool have_shared) const {
    const int total = (r.prompt_len + r.max_new + block_size - 1) / block_size;
    const int shared_full = have_shared ? r.prompt_len / block_size : 0;
    return total - shared_full;
  }
};

}  // namespace

// ---------------------------------------------------------------------------------------------
// scheduler API
// ---------------------------------------------------------------------------------------------
API void* trlb_sched_create(int max_slots, int num_blocks, int block_size, int max_blocks_per_seq) {
  return new Scheduler(max_slots, num_blocks, block_size, max_blocks_per_seq);
}
API void trlb_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

API void trlb_sched_add(void* h, int64_t id, int prompt_len, int max_new, int64_t group) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  s->waiting.push_back({id, prompt_len, max_new, group});
  s->group_pending[group] += 1;
}

API int trlb_sched_num_waiting(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  return (int)s->waiting.size();
}
API int trlb_sched_num_running(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  int n = 0;
  for (auto& r : s->slots) n += r.id >= 0;
  return n;
}
API int trlb_sched_num_free_blocks(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  return s->pool.num_free();
}

// Admit as many waiting requests as slots and blocks allow (FIFO).  For each admitted request i:
//   out_ids[i], out_slots[i], out_prefill[i] (1 = this request must run the prompt prefill for
//   its group, 0 = the full prompt blocks are shared from an earlier member and only the partial
//   tail block must be copied from cache block out_copy_from_block[i] (-1: the prompt ends on a
//   block boundary) into this request's block number prompt_len / block_size).
// block_table (int32 [max_slots, max_blocks_per_seq], host memory) rows of admitted slots are filled.
API int trlb_sched_admit(void* h, int max_admit, int64_t* out_ids, int32_t* out_slots, int32_t* out_prefill,
                         int32_t* out_copy_from_block, int32_t* block_table) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  int n = 0;
  while (!s->waiting.empty() && n < max_admit) {
    int slot = -1;
    for (int i = 0; i < s->max_slots; ++i)
      if (s->slots[i].id < 0) { slot = i; break; }
    if (slot < 0) break;
    const Request r = s->waiting.front();
    auto it = s->shared.find(r.group);
    const bool have = it != s->shared.end() && it->second.prefilled;
    const int need = s->blocks_needed(r, have);
    if (need > s->pool.num_free()) break;
    const int total = (r.prompt_len + r.max_new + s->block_size - 1) / s->block_size;
    if (total > s->max_blocks_per_seq) { s->waiting.pop_front(); s->group_pending[r.group] -= 1; continue; }
    s->waiting.pop_front();
    Running& run = s->slots[slot];
    run.id = r.id;
    run.blocks.clear();
    const int shared_full = r.prompt_len / s->block_size;
    if (have) {
      for (int b = 0; b < shared_full; ++b) {
        s->pool.retain(it->second.blocks[b]);
        run.blocks.push_back(it->second.blocks[b]);
      }
      it->second.users += 1;
      out_prefill[n] = 0;
      out_copy_from_block[n] = it->second.tail_block;
    } else {
      out_prefill[n] = 1;
      out_copy_from_block[n] = -1;
    }
    while ((int)run.blocks.size() < total) run.blocks.push_back(s->pool.alloc());
    if (!have) {
      auto& sh = s->shared[r.group];
      sh.blocks.assign(run.blocks.begin(), run.blocks.begin() + shared_full);
      for (int b : sh.blocks) s->pool.retain(b);  // the group entry holds its own reference
      sh.users = 1;
      sh.prefilled = true;
      if (r.prompt_len % s->block_size != 0) {
        sh.tail_block = run.blocks[shared_full];
        s->pool.retain(sh.tail_block);
      }
    }
    int32_t* row = block_table + (size_t)slot * s->max_blocks_per_seq;
    for (int b = 0; b < s->max_blocks_per_seq; ++b) row[b] = b < (int)run.blocks.size() ? run.blocks[b] : 0;
    out_ids[n] = r.id;
    out_slots[n] = slot;
    ++n;
  }
  return n;
}

// Retire the request in `slot`; its blocks are released (shared prompt blocks survive while the
// group still has members).  Returns the request id or -1.
API int64_t trlb_sched_retire(void* h, int slot, int64_t group) {
  auto* s = static_cast<Scheduler*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  Running& run = s->slots[slot];
  const int64_t id = run.id;
  if (id < 0) return -1;
  for (int b : run.blocks) s->pool.release(b);
  run.blocks.clear();
  run.id = -1;
  auto pit = s->group_pending.find(group);
  if (pit != s->group_pending.end() && --pit->second <= 0) {
    s->group_pending.erase(pit);
    auto it = s->shared.find(group);
    if (it != s->shared.end()) {
      for (int b : it->second.blocks) s->pool.release(b);
      s->pool.release(it->second.tail_block);
      s->shared.erase(it);
    }
  }
  return id;
}

// ---------------------------------------------------------------------------------------------
// best-fit-decreasing packing
// ---------------------------------------------------------------------------------------------
namespace {
struct MaxTree {
  int size = 1;
  std::vector<int> t;
  explicit MaxTree(int maxval) {
    while (size < maxval) size <<= 1;
    t.assign(2 * size, 0);
  }
  void set(int val, bool present) {
    int i = size + val - 1;
    t[i] = present ? val : 0;
    for (i >>= 1; i >= 1; i >>= 1) t[i] = std::max(t[2 * i], t[2 * i + 1]);
  }
  int search(int val) const {  // smallest stored capacity >= val
    int i = 1;
    while (i < size) i = (t[2 * i] >= val) ? 2 * i : 2 * i + 1;
    return t[i];
  }
};
}  // namespace

// lengths[n] (each in 1..seq_length) -> bin_of[n]; returns the number of bins.  Items are visited
// in order of decreasing length (stable); a bin with exactly `space` left is reused first-in-first-out.
API int trlb_bfd_assign(const int32_t* lengths, int n, int seq_length, int32_t* bin_of) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lengths[a] > lengths[b]; });
  MaxTree tree(seq_length);
  tree.set(seq_length, true);
  std::vector<std::deque<int>> by_space(seq_length + 1);
  std::vector<int> space_left;
  for (int idx : order) {
    const int L = lengths[idx];
    const int space = tree.search(L);
    int bin;
    if (space < seq_length) {
      bin = by_space[space].front();
      by_space[space].pop_front();
      if (by_space[space].empty()) tree.set(space, false);
    } else {
      bin = (int)space_left.size();
      space_left.push_back(seq_length);
    }
    bin_of[idx] = bin;
    space_left[bin] -= L;
    const int rest = space_left[bin];
    if (rest > 0) {
      if (by_space[rest].empty()) tree.set(rest, true);
      by_space[rest].push_back(bin);
    }
  }
  return (int)space_left.size();
}
