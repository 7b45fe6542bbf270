// The page pool's data and the operations that the pool's C interface (page_pool.cpp) and the
// scheduler (scheduler.cpp) share.  Requests are known by their slot (the row id that the
// reference uses to index its tables, kv/KV_pool.h:31-37), which is also the index of a
// request's fixed-size state, and by the caller's key, a 64-bit number that the pool maps to the slot.
#pragma once

#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <unordered_map>
#include <vector>

#define LLMH_API extern "C" __attribute__((visibility("default")))

namespace llmh {

enum : int { KIND_FULL = 0, KIND_WINDOW = 1 };
enum : int { ERR_CONTRACT = -1, ERR_OUT_OF_PAGES = -2 };

struct Group {
  int kind, page_size, num_pages, window, width;     // width: table entries per request
  std::vector<int> free;                             // LIFO: back() is handed out next
  std::vector<int> table;                            // [max_requests][width], -1 = given back / not held
  std::vector<int> n_pages, first_live;              // per slot: logical pages in the table, first one still held

  int pages_for(int length) const { return (length + page_size - 1) / page_size; }
  // logical pages below this index can no longer be seen by a token at next_pos or later
  int dead_before(int next_pos) const {
    if (kind != KIND_WINDOW) return 0;
    const int lowest_key = next_pos - window + 1;
    return lowest_key <= 0 ? 0 : lowest_key / page_size;
  }
};

struct Pool {
  std::vector<Group> groups;
  int max_requests = 0, max_seq_len = 0;
  std::vector<int> free_slots;                       // LIFO
  std::vector<int> len;                              // per slot; -1 = not live
  std::vector<long long> key;                        // per slot: the caller's key
  std::unordered_map<long long, int> slot_of_key;    // the live requests
  std::vector<int> fresh;                            // admitted since the last take: state to be zeroed
  bool log_freed = false;                            // debug: remember which pages went back to the free lists
  std::vector<std::vector<int>> freed;               // per group, since the last take
  char error[512] = "";

  int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error, sizeof(error), fmt, ap);
    va_end(ap);
    return code;
  }
  bool live(int slot) const { return slot >= 0 && slot < max_requests && len[slot] >= 0; }
  int slot_of(long long k) const {
    auto it = slot_of_key.find(k);
    return it == slot_of_key.end() ? -1 : it->second;
  }

  // per group, the pages that growing by n_new takes from the free list, net of the window
  // pages that the same call gives back first
  void pages_needed(int slot, int cur, int n_new, int* out) const {
    for (size_t g = 0; g < groups.size(); ++g) {
      const Group& grp = groups[g];
      const int have_hi = grp.pages_for(cur), need_hi = grp.pages_for(cur + n_new);
      int give_back = 0;
      if (grp.kind == KIND_WINDOW) {
        const int first = slot >= 0 ? grp.first_live[slot] : 0;
        const int dead = std::min(grp.dead_before(cur), have_hi);
        give_back = std::max(0, dead - first);
      }
      out[g] = need_hi - have_hi - give_back;
    }
  }

  // A new request takes a state slot.
  int admit(long long k) {
    if (slot_of_key.count(k)) return fail(ERR_CONTRACT, "request %lld is already live", k);
    if (free_slots.empty()) return fail(ERR_CONTRACT, "no request slot free (%d live)", max_requests);
    const int slot = free_slots.back();
    free_slots.pop_back();
    len[slot] = 0;
    key[slot] = k;
    slot_of_key[k] = slot;
    for (Group& grp : groups) {
      grp.n_pages[slot] = 0;
      grp.first_live[slot] = 0;
    }
    fresh.push_back(slot);
    return slot;
  }

  void give(size_t g, int page) {
    groups[g].free.push_back(page);
    if (log_freed) freed[g].push_back(page);
  }

  // Window pages of the slot that no token at position cur or later can see go back.
  void give_back_window(int slot, int cur) {
    for (size_t g = 0; g < groups.size(); ++g) {
      Group& grp = groups[g];
      if (grp.kind != KIND_WINDOW) continue;
      int* row = grp.table.data() + (size_t)slot * grp.width;
      const int dead = std::min(grp.dead_before(cur), grp.n_pages[slot]);
      for (int i = grp.first_live[slot]; i < dead; ++i) {
        give(g, row[i]);
        row[i] = -1;
      }
      grp.first_live[slot] = std::max(grp.first_live[slot], dead);
    }
  }

  // The request ended: all its pages and its slot go back.
  int release(int slot) {
    if (!live(slot)) return fail(ERR_CONTRACT, "slot %d is not live (released twice?)", slot);
    for (size_t g = 0; g < groups.size(); ++g) {
      Group& grp = groups[g];
      int* row = grp.table.data() + (size_t)slot * grp.width;
      for (int i = grp.first_live[slot]; i < grp.n_pages[slot]; ++i) give(g, row[i]);
      std::fill(row, row + grp.n_pages[slot], -1);
      grp.n_pages[slot] = 0;
      grp.first_live[slot] = 0;
    }
    free_slots.push_back(slot);
    len[slot] = -1;
    slot_of_key.erase(key[slot]);
    return 0;
  }
};

}  // namespace llmh
