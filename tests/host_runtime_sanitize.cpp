// Stress driver for the host runtime (scheduler, block pool, packer), built with -fsanitize=address,undefined by
// tests/test_runtime_cpu.py: random admit / retire cycles with shared prompt prefixes, then a packing run; any heap
// error, leak or undefined behaviour fails the run.
#include <cstdint>
#include <cstdio>
#include <random>
#include <vector>

extern "C" {
void* trlb_sched_create(int max_slots, int num_blocks, int block_size, int max_blocks_per_seq);
void trlb_sched_destroy(void* h);
void trlb_sched_add(void* h, int64_t id, int prompt_len, int max_new, int64_t group);
int trlb_sched_num_waiting(void* h);
int trlb_sched_num_running(void* h);
int trlb_sched_num_free_blocks(void* h);
int trlb_sched_admit(void* h, int max_admit, int64_t* out_ids, int32_t* out_slots, int32_t* out_prefill,
                     int32_t* out_copy_blk, int32_t* block_table);
int64_t trlb_sched_retire(void* h, int slot, int64_t group);
int trlb_bfd_assign(const int32_t* lengths, int n, int seq_length, int32_t* bin_of);
}

int main() {
  const int slots = 8, blocks = 64, bs = 16, max_blocks = 8;
  std::mt19937 rng(7);
  for (int round = 0; round < 50; ++round) {
    void* s = trlb_sched_create(slots, blocks, bs, max_blocks);
    int64_t next_id = 0;
    for (int g = 0; g < 6; ++g) {
      const int plen = 1 + (int)(rng() % 60);
      for (int j = 0; j < 4; ++j) trlb_sched_add(s, next_id++, plen, 1 + (int)(rng() % 40), g);
    }
    std::vector<int64_t> ids(slots), slot_group(slots, -1);
    std::vector<int32_t> sl(slots), pre(slots), cp(slots), table(slots * max_blocks, 0);
    int guard = 0;
    while ((trlb_sched_num_waiting(s) > 0 || trlb_sched_num_running(s) > 0) && ++guard < 10000) {
      const int n = trlb_sched_admit(s, slots, ids.data(), sl.data(), pre.data(), cp.data(), table.data());
      for (int i = 0; i < n; ++i) slot_group[sl[i]] = ids[i] / 4;
      for (int k = 0; k < slots; ++k)
        if (slot_group[k] >= 0 && rng() % 3 == 0) {
          trlb_sched_retire(s, k, slot_group[k]);
          slot_group[k] = -1;
        }
    }
    if (trlb_sched_num_free_blocks(s) != blocks) {
      std::printf("leaked blocks: %d free of %d\n", trlb_sched_num_free_blocks(s), blocks);
      return 2;
    }
    trlb_sched_destroy(s);
  }
  std::vector<int32_t> lens(500), bin(500);
  for (auto& l : lens) l = 1 + (int)(rng() % 128);
  const int nb = trlb_bfd_assign(lens.data(), (int)lens.size(), 128, bin.data());
  std::vector<int> fill(nb, 0);
  for (size_t i = 0; i < lens.size(); ++i) fill[bin[i]] += lens[i];
  for (int f : fill)
    if (f > 128) return 3;
  std::printf("SANITIZE_OK bins=%d\n", nb);
  return 0;
}
