// Host side of the cache, native: pages, block tables and state slots of the live requests,
// and the routine that writes a step's metadata into the pinned buffer that is copied to the
// device.  Plain C++17 with a C interface (built with g++, loaded with ctypes); no CUDA here.
//
// Like the reference's KV_Pool (kv/KV_pool.h:13-102) the pool keeps, per request slot, the
// physical pages that hold its tokens, hands pages out from a LIFO free list when a request
// grows (KV_Pool::append, :40-52) and takes them back when it ends (:55-60).  Unlike it, the
// pool is split into groups: layers whose needs differ (every past key, or a window of them)
// have pages and tables of their own, and a window group gives a page back as soon as every
// later token's window has passed it.  The page size is a parameter, not the constant 16 of
// kv/KV_Layout.h:2, and contracts are checked, not asserted.  Requests are known here by their
// slot (the row id that the reference uses to index its tables, kv/KV_pool.h:31-37), which is
// also the index of a request's fixed-size state.
#include "page_pool.h"

using namespace llmh;

LLMH_API void* llmh_pool_create(int n_groups, const int* kinds, const int* page_sizes, const int* num_pages,
                                const int* windows, int max_requests, int max_seq_len) {
  if (n_groups < 0 || max_requests <= 0 || max_seq_len <= 0) return nullptr;
  Pool* p = new Pool();
  p->max_requests = max_requests;
  p->max_seq_len = max_seq_len;
  for (int g = 0; g < n_groups; ++g) {
    if (page_sizes[g] <= 0 || num_pages[g] < 0 || (kinds[g] != KIND_FULL && kinds[g] != KIND_WINDOW) ||
        (kinds[g] == KIND_WINDOW && windows[g] <= 0)) {
      delete p;
      return nullptr;
    }
    Group grp;
    grp.kind = kinds[g];
    grp.page_size = page_sizes[g];
    grp.num_pages = num_pages[g];
    grp.window = windows[g];
    grp.width = grp.pages_for(max_seq_len);
    grp.free.resize(num_pages[g]);
    for (int i = 0; i < num_pages[g]; ++i) grp.free[i] = num_pages[g] - 1 - i;      // page 0 is handed out first
    grp.table.assign((size_t)max_requests * grp.width, -1);
    grp.n_pages.assign(max_requests, 0);
    grp.first_live.assign(max_requests, 0);
    p->groups.push_back(std::move(grp));
  }
  p->free_slots.resize(max_requests);
  for (int i = 0; i < max_requests; ++i) p->free_slots[i] = max_requests - 1 - i;
  p->len.assign(max_requests, -1);
  p->key.assign(max_requests, 0);
  p->freed.resize(n_groups);
  return p;
}

LLMH_API void llmh_pool_destroy(void* h) { delete static_cast<Pool*>(h); }
LLMH_API const char* llmh_pool_error(void* h) { return static_cast<Pool*>(h)->error; }
LLMH_API int llmh_pool_table_width(void* h, int g) { return static_cast<Pool*>(h)->groups[g].width; }
LLMH_API int llmh_pool_free_pages(void* h, int g) { return (int)static_cast<Pool*>(h)->groups[g].free.size(); }
LLMH_API int llmh_pool_free_slots(void* h) { return (int)static_cast<Pool*>(h)->free_slots.size(); }
LLMH_API int llmh_pool_length(void* h, int slot) {
  Pool* p = static_cast<Pool*>(h);
  return p->live(slot) ? p->len[slot] : p->fail(ERR_CONTRACT, "slot %d is not live", slot);
}

// slot -1: a request not yet admitted; length -1: the slot's current length
LLMH_API int llmh_pool_pages_needed(void* h, int slot, int length, int n_new, int* out) {
  Pool* p = static_cast<Pool*>(h);
  if (slot >= 0 && !p->live(slot)) return p->fail(ERR_CONTRACT, "slot %d is not live", slot);
  const int cur = length >= 0 ? length : (slot >= 0 ? p->len[slot] : 0);
  p->pages_needed(slot, cur, n_new, out);
  return 0;
}

// A new request, known to the caller by `key`, takes a state slot; returns the slot.
LLMH_API int llmh_pool_admit(void* h, long long key) { return static_cast<Pool*>(h)->admit(key); }
// The slot of a live request, or -1.
LLMH_API int llmh_pool_slot(void* h, long long key) { return static_cast<Pool*>(h)->slot_of(key); }
// The keys of the live requests into out (up to capacity); returns their number.
LLMH_API int llmh_pool_live_keys(void* h, long long* out, int capacity) {
  Pool* p = static_cast<Pool*>(h);
  int n = 0;
  for (int slot = 0; slot < p->max_requests; ++slot)
    if (p->len[slot] >= 0) {
      if (n < capacity) out[n] = p->key[slot];
      ++n;
    }
  return n;
}

LLMH_API int llmh_pool_take_fresh(void* h, int* out, int capacity) {
  Pool* p = static_cast<Pool*>(h);
  const int n = std::min((int)p->fresh.size(), capacity);
  std::copy(p->fresh.begin(), p->fresh.begin() + n, out);
  p->fresh.clear();
  return n;
}

// The request is about to write n_new tokens: give back window pages that are out of sight,
// take the pages that the new tokens need, return the position of the first new token.
LLMH_API int llmh_pool_extend(void* h, int slot, int n_new) {
  Pool* p = static_cast<Pool*>(h);
  if (!p->live(slot)) return p->fail(ERR_CONTRACT, "slot %d is not live", slot);
  if (n_new <= 0) return p->fail(ERR_CONTRACT, "extend needs at least one token");
  const int cur = p->len[slot];
  if (cur + n_new > p->max_seq_len)
    return p->fail(ERR_CONTRACT, "slot %d: %d+%d tokens exceed max_seq_len %d", slot, cur, n_new, p->max_seq_len);
  int needs[64];
  if (p->groups.size() > 64) return p->fail(ERR_CONTRACT, "too many cache groups");
  p->pages_needed(slot, cur, n_new, needs);
  for (size_t g = 0; g < p->groups.size(); ++g)
    if (needs[g] > (int)p->groups[g].free.size())
      return p->fail(ERR_OUT_OF_PAGES, "group %d: slot %d needs %d pages, %d free", (int)g, slot, needs[g], (int)p->groups[g].free.size());
  p->give_back_window(slot, cur);
  for (Group& grp : p->groups) {
    int* row = grp.table.data() + (size_t)slot * grp.width;
    const int want = grp.pages_for(cur + n_new);
    for (int i = grp.n_pages[slot]; i < want; ++i) {
      row[i] = grp.free.back();
      grp.free.pop_back();
    }
    grp.n_pages[slot] = want;
  }
  p->len[slot] = cur + n_new;
  return cur;
}

// The request ended: all its pages and its slot go back.
LLMH_API int llmh_pool_release(void* h, int slot) { return static_cast<Pool*>(h)->release(slot); }

// The start of a step, all or nothing: entries b = 0..B-1 are requests (by key; new ones are
// admitted) that bring counts[b] tokens each.  First sees that every entry fits (request slots,
// max_seq_len, pages of every group), before any page moves; then every entry gives back the
// window pages that are out of its sight, and only then the entries are admitted and take their
// pages in order, so that an entry ahead of one that frees pages can already use them (the sum
// that was checked counts them).  slots[b]
// and starts[b] get the request's slot and the position of its first new token.  Returns 0,
// ERR_CONTRACT (*bad = the entry at fault, or -1) or ERR_OUT_OF_PAGES (*bad = the group).
LLMH_API int llmh_pool_begin_step(void* h, int B, const long long* keys, const int* counts, int* slots, int* starts,
                                  int* bad) {
  Pool* p = static_cast<Pool*>(h);
  const int G = (int)p->groups.size();
  if (G > 64) return p->fail(ERR_CONTRACT, "too many cache groups");
  int need[64] = {0}, k[64];
  int fresh = 0;
  *bad = -1;
  for (int b = 0; b < B; ++b) {
    const int slot = p->slot_of(keys[b]);
    const int cur = slot >= 0 ? p->len[slot] : 0;
    fresh += slot < 0;
    if (counts[b] <= 0 || cur + counts[b] > p->max_seq_len) {
      *bad = b;
      return p->fail(ERR_CONTRACT, "%d+%d tokens exceed max_seq_len %d", cur, counts[b], p->max_seq_len);
    }
    p->pages_needed(slot, cur, counts[b], k);
    for (int g = 0; g < G; ++g) need[g] += k[g];
  }
  if (fresh > (int)p->free_slots.size())
    return p->fail(ERR_CONTRACT, "%d new requests but only %d request slots free", fresh, (int)p->free_slots.size());
  for (int g = 0; g < G; ++g)
    if (need[g] > (int)p->groups[g].free.size()) {
      *bad = g;
      return p->fail(ERR_OUT_OF_PAGES, "cache group %d: the step needs %d pages, %d free", g, need[g], (int)p->groups[g].free.size());
    }
  for (int b = 0; b < B; ++b) {
    const int slot = p->slot_of(keys[b]);
    if (slot >= 0) p->give_back_window(slot, p->len[slot]);
  }
  for (int b = 0; b < B; ++b) {
    int slot = p->slot_of(keys[b]);
    if (slot < 0) slot = p->admit(keys[b]);
    if (slot < 0) return slot;
    slots[b] = slot;
    starts[b] = llmh_pool_extend(h, slot, counts[b]);
    if (starts[b] < 0) return starts[b];
  }
  return 0;
}

// Debug aid: with on != 0 the pool remembers every page that goes back to a free list (a request
// ended, was preempted, or a window passed the page) until llmh_pool_take_freed collects them, so
// that the device side can overwrite them and a read of a stale page shows.
LLMH_API void llmh_pool_log_freed(void* h, int on) {
  Pool* p = static_cast<Pool*>(h);
  p->log_freed = on != 0;
  for (auto& v : p->freed) v.clear();
}

// The pages of group g freed since the last call, into out (up to capacity); returns their
// number and forgets them.
LLMH_API int llmh_pool_take_freed(void* h, int g, int* out, int capacity) {
  Pool* p = static_cast<Pool*>(h);
  std::vector<int>& v = p->freed[g];
  const int n = std::min((int)v.size(), capacity);
  std::copy(v.begin(), v.begin() + n, out);
  v.erase(v.begin(), v.begin() + n);
  return n;
}

// The slot's table row in group g (width entries; -1 where no page is held), the number of
// logical pages in it and the first one still held.
LLMH_API const int* llmh_pool_table(void* h, int g, int slot, int* n_pages, int* first_live) {
  Pool* p = static_cast<Pool*>(h);
  const Group& grp = p->groups[g];
  *n_pages = grp.n_pages[slot];
  *first_live = grp.first_live[slot];
  return grp.table.data() + (size_t)slot * grp.width;
}

// No page lost, held twice or free twice; no slot lost or shared; tables match lengths.
LLMH_API int llmh_pool_check(void* h) {
  Pool* p = static_cast<Pool*>(h);
  for (size_t g = 0; g < p->groups.size(); ++g) {
    const Group& grp = p->groups[g];
    std::vector<int> seen(grp.num_pages, 0);
    for (int page : grp.free) {
      if (page < 0 || page >= grp.num_pages) return p->fail(ERR_CONTRACT, "group %d: page %d on the free list", (int)g, page);
      ++seen[page];
    }
    for (int slot = 0; slot < p->max_requests; ++slot) {
      if (p->len[slot] < 0) continue;
      if (grp.n_pages[slot] != grp.pages_for(p->len[slot]))
        return p->fail(ERR_CONTRACT, "group %d: table of slot %d does not match its length", (int)g, slot);
      const int* row = grp.table.data() + (size_t)slot * grp.width;
      for (int i = grp.first_live[slot]; i < grp.n_pages[slot]; ++i) {
        if (row[i] < 0 || row[i] >= grp.num_pages)
          return p->fail(ERR_CONTRACT, "group %d: a live table entry is marked as given back", (int)g);
        ++seen[row[i]];
      }
    }
    for (int page = 0; page < grp.num_pages; ++page) {
      if (seen[page] > 1) return p->fail(ERR_CONTRACT, "group %d: a page is held twice or free twice (page %d)", (int)g, page);
      if (seen[page] == 0) return p->fail(ERR_CONTRACT, "group %d: pages lost (page %d)", (int)g, page);
    }
  }
  std::vector<int> slots(p->max_requests, 0);
  for (int s : p->free_slots) ++slots[s];
  for (int s = 0; s < p->max_requests; ++s)
    if ((p->len[s] >= 0) + slots[s] != 1) return p->fail(ERR_CONTRACT, "a request slot is lost or shared (slot %d)", s);
  size_t live = 0;
  for (int s = 0; s < p->max_requests; ++s)
    if (p->len[s] >= 0) {
      ++live;
      if (p->slot_of(p->key[s]) != s) return p->fail(ERR_CONTRACT, "slot %d and its request's key disagree", s);
    }
  if (live != p->slot_of_key.size()) return p->fail(ERR_CONTRACT, "two requests share a slot");
  return 0;
}

// ---- a step's metadata ---------------------------------------------------------------------
// Offsets (in int32 words) of the arrays inside the metadata block; block_table and slot_map
// have one entry per cache group.
struct StepLayout {
  int token_ids, positions, token_entry, cu_tokens, kv_lens, state_slots, logit_rows, feed_dst, feed_src;
  int n_groups;
  int block_table[16], slot_map[16];
};

// Entries b = 0..B-1: slot, number of new tokens, position of the first (what extend returned);
// tokens: all entries' token ids back to back (a fed entry's token is a placeholder);
// want_counts/wants: per entry the wanted places among its tokens; feeds: per entry the row of
// the feed source or -1.  Writes the block (int32) and returns the number of fed entries, or a
// negative code.
LLMH_API int llmh_prepare_step(void* h, const StepLayout* lay, int32_t* block, int B, const int* slots,
                               const int* n_tokens, const int* starts, const int* tokens, const int* want_counts,
                               const int* wants, const int* feeds) {
  Pool* p = static_cast<Pool*>(h);
  if (lay->n_groups != (int)p->groups.size() || lay->n_groups > 16) return p->fail(ERR_CONTRACT, "layout and pool disagree on the groups");
  int t = 0, r = 0, w_at = 0, n_feed = 0;
  block[lay->cu_tokens] = 0;
  for (int b = 0; b < B; ++b) {
    const int slot = slots[b], n = n_tokens[b], start = starts[b];
    if (!p->live(slot) || p->len[slot] != start + n) return p->fail(ERR_CONTRACT, "entry %d: slot %d does not hold %d tokens", b, slot, start + n);
    for (int i = 0; i < n; ++i) {
      block[lay->token_ids + t + i] = tokens[t + i];
      block[lay->positions + t + i] = start + i;
      block[lay->token_entry + t + i] = b;
    }
    for (int g = 0; g < lay->n_groups; ++g) {
      const Group& grp = p->groups[g];
      const int* row = grp.table.data() + (size_t)slot * grp.width;
      int32_t* bt = block + lay->block_table[g] + (size_t)b * grp.width;
      std::copy(row, row + grp.width, bt);
      int32_t* sm = block + lay->slot_map[g] + t;
      for (int i = 0; i < n; ++i) {
        const int pos = start + i;
        sm[i] = row[pos / grp.page_size] * grp.page_size + pos % grp.page_size;
      }
    }
    for (int i = 0; i < want_counts[b]; ++i) block[lay->logit_rows + r++] = t + wants[w_at + i];
    w_at += want_counts[b];
    if (feeds[b] >= 0) {
      block[lay->feed_dst + n_feed] = t;
      block[lay->feed_src + n_feed] = feeds[b];
      ++n_feed;
    }
    block[lay->kv_lens + b] = start + n;
    block[lay->state_slots + b] = slot;
    t += n;
    block[lay->cu_tokens + b + 1] = t;
  }
  return n_feed;
}
