// The scheduler, native: admits requests, cuts prompts into portions under a token budget,
// decodes, finishes and frees.  Plain C++17 with a C interface on top of the page pool
// (page_pool.h); the Python class llm_b200.engine.scheduler.Scheduler is its face.
//
// Rules are those of the reference's Scheduler (runtime/Scheduler.h:81-283) with one change: a
// step is one mixed batch instead of a prefill batch or a decode batch (:103-108).  Decoding
// requests come first, one token each; what is left of max_num_batched_tokens is filled with
// prompt portions in arrival order, a long prompt cut to the budget and several short ones
// sharing it (:155-191).  A portion is scheduled only if the free pages cover it plus a reserve
// of one page for every running request that will sit on a page boundary (:170-171,222-232); a
// request that does not fit stops the walk (head-of-line blocking, :171).
//
// When pages run out: prompts wait; if the decoding requests themselves cannot all take their
// next token, the one queued last is preempted: its pages and slot are given back and it returns
// to the head of the prompt queue with everything it has produced so far as its prompt, to be
// recomputed (:194,234-246).  A request whose prompt plus max_new_tokens can never fit is refused
// when it is added (:89-91).
//
// The pages themselves are taken when the step is prepared, as the reference takes them in
// Engine::prepare (runtime/Engine.h:57); the scheduler only does the arithmetic, group by group,
// and gives pages back (preemption, the end of a request).
#include <deque>
#include <unordered_map>

#include "page_pool.h"

using namespace llmh;

namespace {

constexpr int PENDING_TOKEN = -1;      // stands for a token that is sampled but not read back yet
enum : int { PREFILL = 0, DECODE = 1 };

struct Request {
  long long id = 0;
  std::vector<int> tokens;             // prompt, then what was generated
  int prompt_len = 0, max_new = 0;
  int phase = PREFILL;
  int cached_len = 0;                  // tokens whose keys and values are in the cache
  int num_preemptions = 0;
  bool ignore_eos = false;
  bool ended = false;                  // its end was found after the next step had already been launched
};

struct Entry {
  long long id;
  int start, count;                    // position of the first token, number of tokens
  int offset;                          // of its tokens in the batch's token buffer
  bool samples;                        // the step's last token of this entry yields the next token
};

struct Scheduler {
  Pool* pool;
  int max_num_seqs, max_tokens, eos;
  long long next_id = 0;
  long long num_preemptions = 0;
  std::unordered_map<long long, Request> requests;
  std::deque<long long> prefill_ready, decode_ready;
  // the batch of the last schedule()
  std::vector<Entry> entries;
  std::vector<int> batch_tokens;
  // the requests that the last update() finished
  std::vector<Request> finished;
  std::vector<int> promised, needs, reserve, scratch;

  int G() const { return (int)pool->groups.size(); }
  bool live(long long id) const { return pool->slot_of(id) >= 0; }

  void release(long long id) {
    const int slot = pool->slot_of(id);
    if (slot >= 0) pool->release(slot);
  }

  // pages that `count` more tokens of request `id` take, per group, into out; the request is at
  // `length` tokens (-1: where the pool has it)
  void pages_needed(long long id, bool is_live, int length, int count, int* out) const {
    const int slot = is_live ? pool->slot_of(id) : -1;
    const int cur = length >= 0 ? length : (slot >= 0 ? pool->len[slot] : 0);
    pool->pages_needed(slot, cur, count, out);
  }

  bool fits(const int* need, const int* extra) const {
    for (int g = 0; g < G(); ++g)
      if ((int)pool->groups[g].free.size() - promised[g] < need[g] + (extra ? extra[g] : 0)) return false;
    return true;
  }

  void preempt_last_decode() {
    const long long id = decode_ready.back();
    decode_ready.pop_back();
    Request& r = requests.at(id);
    release(id);
    r.cached_len = 0;
    r.phase = PREFILL;
    ++r.num_preemptions;
    prefill_ready.push_front(id);
    ++num_preemptions;
  }

  int new_in_batch() const {
    int n = 0;
    for (const Entry& e : entries) n += !live(e.id);
    return n;
  }

  // one page per request that, after this step, decodes from a page boundary
  void decode_reserve(int* out) const {
    for (int g = 0; g < G(); ++g) out[g] = 0;
    for (const auto& kv : requests) {
      const Request& r = kv.second;
      int after = r.cached_len;
      bool runs_on = r.phase == DECODE;
      for (const Entry& e : entries)
        if (e.id == r.id) {
          after = e.start + e.count;
          runs_on = e.samples;
          break;
        }
      if (runs_on && after > 0)
        for (int g = 0; g < G(); ++g) out[g] += after % pool->groups[g].page_size == 0;
    }
  }

  void schedule_once() {
    entries.clear();
    batch_tokens.clear();
    const int n_groups = G();
    promised.assign(n_groups, 0);
    needs.assign(n_groups, 0);
    reserve.assign(n_groups, 0);
    scratch.assign(n_groups, 0);

    // Decoding requests first; preempt from the back while they do not all fit.
    while (!decode_ready.empty()) {
      std::fill(needs.begin(), needs.end(), 0);
      const size_t first = std::min(decode_ready.size(), (size_t)max_num_seqs);
      for (size_t i = 0; i < first; ++i) {
        pages_needed(decode_ready[i], true, -1, 1, scratch.data());
        for (int g = 0; g < n_groups; ++g) needs[g] += std::max(scratch[g], 0);
      }
      if (fits(needs.data(), nullptr)) break;
      preempt_last_decode();
    }
    int budget = max_tokens;
    for (int taken = 0; taken < max_num_seqs && !decode_ready.empty(); ++taken) {
      const long long id = decode_ready.front();
      decode_ready.pop_front();
      const Request& r = requests.at(id);
      pages_needed(id, true, -1, 1, scratch.data());
      for (int g = 0; g < n_groups; ++g) promised[g] += scratch[g];
      entries.push_back({id, r.cached_len, 1, (int)batch_tokens.size(), true});
      batch_tokens.push_back(r.tokens.back());
      --budget;
    }

    // Prompt portions in arrival order.
    while (!prefill_ready.empty() && budget > 0 && (int)entries.size() < max_num_seqs) {
      const long long id = prefill_ready.front();
      const Request& r = requests.at(id);
      const int target = (int)r.tokens.size();
      const int chunk = std::min(target - r.cached_len, budget);
      const bool is_final = r.cached_len + chunk == target;
      const bool is_live = live(id);
      if (!is_live && (int)pool->free_slots.size() - new_in_batch() <= 0) break;
      pages_needed(id, is_live, r.cached_len, chunk, needs.data());
      decode_reserve(reserve.data());
      if (is_final)                    // this request decodes next and may start on a fresh page
        for (int g = 0; g < n_groups; ++g) reserve[g] += target % pool->groups[g].page_size == 0;
      if (!fits(needs.data(), reserve.data())) break;
      for (int g = 0; g < n_groups; ++g) promised[g] += needs[g];
      entries.push_back({id, r.cached_len, chunk, (int)batch_tokens.size(), is_final});
      batch_tokens.insert(batch_tokens.end(), r.tokens.begin() + r.cached_len, r.tokens.begin() + r.cached_len + chunk);
      budget -= chunk;
      if (!is_final) break;            // the rest of this prompt comes in the next step; nothing may overtake it
      prefill_ready.pop_front();
    }
  }

  // The next step's batch.  If nothing can run although requests wait, prompts that hold pages
  // behind the head of the queue give them back (they are recomputed later), which always lets
  // the head run: admission made sure that it fits alone.
  void schedule() {
    schedule_once();
    if (!entries.empty() || requests.empty() || prefill_ready.empty()) return;
    const long long head = prefill_ready.front();
    bool freed = false;
    for (auto it = prefill_ready.rbegin(); it != prefill_ready.rend(); ++it) {
      if (*it == head || !live(*it)) continue;
      release(*it);
      Request& r = requests.at(*it);
      r.cached_len = 0;
      ++r.num_preemptions;
      ++num_preemptions;
      freed = true;
    }
    if (freed) schedule_once();
  }

  bool is_finished(const Request& r, int tok) const {
    const bool hit_eos = eos >= 0 && tok == eos && !r.ignore_eos;
    return hit_eos || (int)r.tokens.size() - r.prompt_len >= r.max_new;
  }

  void retire(long long id) {
    release(id);
    auto it = requests.find(id);
    finished.push_back(std::move(it->second));
    requests.erase(it);
  }
};

}  // namespace

LLMH_API void* llmh_sched_create(void* pool, int max_num_seqs, int max_tokens, int eos_token_id) {
  Pool* p = static_cast<Pool*>(pool);
  if (!p || max_num_seqs <= 0 || max_num_seqs > max_tokens || max_num_seqs > p->max_requests) return nullptr;
  Scheduler* s = new Scheduler();
  s->pool = p;
  s->max_num_seqs = max_num_seqs;
  s->max_tokens = max_tokens;
  s->eos = eos_token_id;
  return s;
}

LLMH_API void llmh_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

// The new request's id, or -1 if it can never run: empty prompt, longer than max_seq_len with its
// new tokens, or more pages than a whole group holds.
LLMH_API long long llmh_sched_add(void* h, const int* prompt, int n, int max_new_tokens, int ignore_eos) {
  Scheduler* s = static_cast<Scheduler*>(h);
  const long long worst = (long long)n + max_new_tokens;
  if (n <= 0 || max_new_tokens <= 0 || worst > s->pool->max_seq_len) return -1;
  std::vector<int> need(s->G());
  s->pool->pages_needed(-1, 0, (int)worst, need.data());
  for (int g = 0; g < s->G(); ++g)
    if (need[g] > s->pool->groups[g].num_pages) return -1;
  Request r;
  r.id = s->next_id++;
  r.tokens.assign(prompt, prompt + n);
  r.prompt_len = n;
  r.max_new = max_new_tokens;
  r.ignore_eos = ignore_eos != 0;
  s->prefill_ready.push_back(r.id);
  const long long id = r.id;
  s->requests.emplace(id, std::move(r));
  return id;
}

LLMH_API int llmh_sched_num_requests(void* h) { return (int)static_cast<Scheduler*>(h)->requests.size(); }
LLMH_API long long llmh_sched_num_preemptions(void* h) { return static_cast<Scheduler*>(h)->num_preemptions; }

// Makes the next step's batch and returns its number of entries; *n_tokens gets its tokens.
LLMH_API int llmh_sched_schedule(void* h, int* n_tokens) {
  Scheduler* s = static_cast<Scheduler*>(h);
  s->schedule();
  *n_tokens = (int)s->batch_tokens.size();
  return (int)s->entries.size();
}

// The batch of the last schedule: per entry its request, the position of its first token, its
// number of tokens and whether it samples; returns the tokens of all entries back to back.
LLMH_API const int* llmh_sched_batch(void* h, long long* ids, int* starts, int* counts, int* samples) {
  Scheduler* s = static_cast<Scheduler*>(h);
  for (size_t i = 0; i < s->entries.size(); ++i) {
    ids[i] = s->entries[i].id;
    starts[i] = s->entries[i].start;
    counts[i] = s->entries[i].count;
    samples[i] = s->entries[i].samples;
  }
  return s->batch_tokens.data();
}

// Accounts for a finished step: entries as llmh_sched_batch gave them, new_tokens[i] the next
// token of entry i where it samples (PENDING_TOKEN: not read back yet).  Returns how many
// requests finished; their pages are free again and llmh_sched_finished gives them.
LLMH_API int llmh_sched_update(void* h, int n, const long long* ids, const int* starts, const int* counts,
                               const int* samples, const int* new_tokens) {
  Scheduler* s = static_cast<Scheduler*>(h);
  s->finished.clear();
  for (int i = 0; i < n; ++i) {
    auto it = s->requests.find(ids[i]);
    if (it == s->requests.end()) continue;
    Request& r = it->second;
    r.cached_len = starts[i] + counts[i];
    if (!samples[i]) continue;
    if (r.ended) {                     // ran one step too far: that step's token is dropped
      s->retire(r.id);
      continue;
    }
    const int tok = new_tokens[i];
    r.tokens.push_back(tok);
    if (tok != PENDING_TOKEN && s->is_finished(r, tok)) {
      s->retire(r.id);
    } else {
      r.phase = DECODE;
      s->decode_ready.push_back(r.id);
    }
  }
  return (int)s->finished.size();
}

// The i-th request that the last update finished: its tokens (prompt, then generated).
LLMH_API const int* llmh_sched_finished(void* h, int i, long long* id, int* prompt_len, int* n_tokens,
                                        int* num_preemptions) {
  Scheduler* s = static_cast<Scheduler*>(h);
  if (i < 0 || i >= (int)s->finished.size()) return nullptr;
  const Request& r = s->finished[i];
  *id = r.id;
  *prompt_len = r.prompt_len;
  *n_tokens = (int)r.tokens.size();
  *num_preemptions = r.num_preemptions;
  return r.tokens.data();
}

// Whether the step after this batch can be scheduled before the batch's tokens are known: only
// decoding requests, nobody waiting to be admitted, nobody at its last token, and pages for one
// more token of each without preempting anyone.
LLMH_API int llmh_sched_can_look_ahead(void* h, int n, const long long* ids, const int* samples) {
  Scheduler* s = static_cast<Scheduler*>(h);
  if (!s->prefill_ready.empty() || n == 0) return 0;
  std::vector<int> need(s->G(), 0), k(s->G(), 0);
  for (int i = 0; i < n; ++i) {
    auto it = s->requests.find(ids[i]);
    if (it == s->requests.end() || !samples[i] || it->second.ended) return 0;
    const Request& r = it->second;
    if ((int)r.tokens.size() - r.prompt_len + 2 > r.max_new) return 0;       // this step's token would be its last
    const int slot = s->pool->slot_of(r.id);
    if (slot < 0 || s->pool->len[slot] + 1 > s->pool->max_seq_len) return 0;
    s->pool->pages_needed(slot, s->pool->len[slot], 1, k.data());
    for (int g = 0; g < s->G(); ++g) need[g] += std::max(k[g], 0);
  }
  for (int g = 0; g < s->G(); ++g)
    if (need[g] > (int)s->pool->groups[g].free.size()) return 0;
  return 1;
}

// The tokens of a step that was accounted with placeholders have arrived.  A request that ends
// with its token is marked: it is already part of the step in flight and retires when that step
// is accounted.  Returns 0, or -1 if a request has no placeholder to resolve.
LLMH_API int llmh_sched_resolve(void* h, int n, const long long* ids, const int* new_tokens) {
  Scheduler* s = static_cast<Scheduler*>(h);
  for (int i = 0; i < n; ++i) {
    auto it = s->requests.find(ids[i]);
    if (it == s->requests.end()) continue;
    Request& r = it->second;
    int at = (int)r.tokens.size() - 1;
    while (at >= r.prompt_len && r.tokens[at] != PENDING_TOKEN) --at;
    if (at < r.prompt_len) return -1;
    const int tok = new_tokens[i];
    r.tokens[at] = tok;
    if (s->eos >= 0 && tok == s->eos && !r.ignore_eos) {
      r.tokens.resize(at + 1);
      r.ended = true;
    }
  }
  return 0;
}

// A waiting or running request's tokens, or null if there is none of that id; fields:
// prompt_len, max_new_tokens, phase (0 prompt, 1 decoding), cached_len, num_preemptions, ended.
LLMH_API const int* llmh_sched_request(void* h, long long id, int* n_tokens, int* fields) {
  Scheduler* s = static_cast<Scheduler*>(h);
  auto it = s->requests.find(id);
  if (it == s->requests.end()) return nullptr;
  const Request& r = it->second;
  *n_tokens = (int)r.tokens.size();
  fields[0] = r.prompt_len;
  fields[1] = r.max_new;
  fields[2] = r.phase;
  fields[3] = r.cached_len;
  fields[4] = r.num_preemptions;
  fields[5] = r.ended;
  return r.tokens.data();
}

// The ids in the prompt queue (which = 0) or the decode queue (1), front first; returns their number.
LLMH_API int llmh_sched_queue(void* h, int which, long long* out, int capacity) {
  Scheduler* s = static_cast<Scheduler*>(h);
  const std::deque<long long>& q = which ? s->decode_ready : s->prefill_ready;
  int n = 0;
  for (long long id : q) {
    if (n < capacity) out[n] = id;
    ++n;
  }
  return n;
}
