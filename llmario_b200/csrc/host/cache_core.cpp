// The bookkeeping of the paged cache, on the host: which pages are free, which pages each
// request holds in each group of layers, when a window has passed a page, and which cells of the
// device block tables have changed since they were last sent.  No GPU code: plain C++17 with a C
// interface, compiled by g++ and opened with ctypes like the kernels.
//
// What the reference does (crates/engine/kv/src/lib.rs:36-176; crates/engine/model/src/kv.rs:
// 402-497, 715-827): a pool of fixed-size blocks with a first-freed-first-reused queue, a table of
// block ids per sequence, all-or-nothing allocation that refuses with "needed / free" before it
// changes anything, and separate classes of storage for layers that keep every key and layers that
// keep a window of them.  Here every group of layers with the same need has a pool and a table of
// its own; a group with a window gives a page back as soon as no later query can reach a key in it.
//
// Requests are named by 64-bit keys that the caller chooses.  Every function returns 0 or a
// count on success and a negative code on misuse (the caller turns it into an exception); nothing
// is changed when a call fails.
#include <cstdint>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

namespace {

enum Error {
  E_UNKNOWN = -1,         // no such request
  E_OPEN_TWICE = -2,      // the request is already open
  E_NO_SLOT = -3,         // every request slot is taken
  E_TWICE_IN_STEP = -4,   // a request appears twice in one reserve call
  E_EMPTY_ENTRY = -5,     // a step entry of zero tokens
  E_CONTEXT = -6,         // the request would outgrow the context
  E_PAST_RESERVED = -7,   // advance beyond the pages that were reserved
  E_LENGTHEN = -8,        // truncate to more than the request holds
  E_STATE_REWIND = -9,    // a request with fixed-size state cannot be rewound
  E_WINDOW_GONE = -10,    // truncate into pages a window has already given back
  E_NOT_HELD = -11,       // a page released that is not held
  E_ARGUMENT = -12,
  // check(): what is wrong
  E_HELD_TWICE = -20, E_FREE_AND_HELD = -21, E_FREE_TWICE = -22, E_LOST = -23, E_COUNT_OFF = -24,
  E_SLOT_TWICE = -25, E_SLOT_LOST = -26,
};

struct Pool {
  int n = 0;
  std::deque<int> free;          // the page freed longest ago is handed out first
  std::vector<char> held;
  int n_held = 0;
  explicit Pool(int pages) : n(pages), held(pages, 0) {
    for (int p = 0; p < pages; ++p) free.push_back(p);
  }
  bool alloc(int k, std::vector<int>* out) {      // all or nothing
    if (k > (int)free.size()) return false;
    for (int i = 0; i < k; ++i) {
      const int p = free.front();
      free.pop_front();
      held[p] = 1;
      out->push_back(p);
    }
    n_held += k;
    return true;
  }
  int release(const int* pages, int k) {
    for (int i = 0; i < k; ++i)
      if (pages[i] < 0 || pages[i] >= n || !held[pages[i]]) return E_NOT_HELD;
    for (int i = 0; i < k; ++i) {
      // (a page named twice in one call would be freed twice: refuse the second)
      if (!held[pages[i]]) return E_NOT_HELD;
      held[pages[i]] = 0;
      free.push_back(pages[i]);
      --n_held;
    }
    return 0;
  }
};

struct Request {
  int slot = 0;
  int length = 0;
  std::vector<std::vector<int>> pages;   // per group, by page index; -1 = given back
  std::vector<int> first_live;           // per group, first page index not given back
};

struct Group {
  Pool pool;
  int window;                            // 0: every key is kept
  // changes of the device table not yet taken: one value per cell, the last one wins
  std::vector<int> pending;              // [max_requests * pages_per_request]
  std::vector<char> dirty;
  std::vector<int> dirty_cells;
  Group(int pages, int w, int cells) : pool(pages), window(w), pending(cells, -1), dirty(cells, 0) {}
  void set(int cell, int value) {
    pending[cell] = value;
    if (!dirty[cell]) {
      dirty[cell] = 1;
      dirty_cells.push_back(cell);
    }
  }
};

struct Core {
  int page_size, max_requests, max_context, pages_per_request, has_state;
  std::vector<Group> groups;
  std::unordered_map<int64_t, Request> requests;
  std::deque<int> free_slots;
  std::vector<int> fresh_slots;          // opened since they were last taken
  long long counters[4] = {0, 0, 0, 0};  // pages allocated, released, released by a window, refusals

  int first_needed_page(const Group& g, int length) const {
    if (g.window <= 0) return 0;
    const int first_key = length - g.window + 1;
    return (first_key > 0 ? first_key : 0) / page_size;
  }
  void needed(const Request& r, int new_tokens, int* out) const {
    const int want = (r.length + new_tokens + page_size - 1) / page_size;
    for (size_t g = 0; g < groups.size(); ++g) {
      const int have = (int)r.pages[g].size();
      out[g] = want > have ? want - have : 0;
    }
  }
};

}  // namespace

extern "C" {

Core* llm_cache_new(int n_groups, const int* n_pages, const int* window, int page_size, int max_requests,
                    int max_context, int has_state) {
  if (n_groups < 0 || page_size <= 0 || max_requests <= 0 || max_context <= 0) return nullptr;
  for (int g = 0; g < n_groups; ++g)
    if (n_pages[g] <= 0) return nullptr;
  Core* c = new Core();
  c->page_size = page_size;
  c->max_requests = max_requests;
  c->max_context = max_context;
  c->pages_per_request = (max_context + page_size - 1) / page_size;
  c->has_state = has_state;
  for (int g = 0; g < n_groups; ++g)
    c->groups.emplace_back(n_pages[g], window[g], max_requests * c->pages_per_request);
  for (int s = 0; s < max_requests; ++s) c->free_slots.push_back(s);
  return c;
}

void llm_cache_delete(Core* c) { delete c; }

int llm_cache_open(Core* c, int64_t key) {
  if (c->requests.count(key)) return E_OPEN_TWICE;
  if (c->free_slots.empty()) return E_NO_SLOT;
  Request r;
  r.slot = c->free_slots.front();
  c->free_slots.pop_front();
  r.pages.resize(c->groups.size());
  r.first_live.assign(c->groups.size(), 0);
  c->fresh_slots.push_back(r.slot);
  const int slot = r.slot;
  c->requests.emplace(key, std::move(r));
  return slot;
}

int llm_cache_has(Core* c, int64_t key) { return c->requests.count(key) ? 1 : 0; }

// slot and length of one request
int llm_cache_info(Core* c, int64_t key, int* slot, int* length) {
  auto it = c->requests.find(key);
  if (it == c->requests.end()) return E_UNKNOWN;
  *slot = it->second.slot;
  *length = it->second.length;
  return 0;
}

// the same for n requests at once; returns the index of the first unknown one as -(100 + i)
int llm_cache_info_many(Core* c, int n, const int64_t* keys, int* slots, int* lengths) {
  for (int i = 0; i < n; ++i) {
    auto it = c->requests.find(keys[i]);
    if (it == c->requests.end()) return -(100 + i);
    slots[i] = it->second.slot;
    lengths[i] = it->second.length;
  }
  return 0;
}

int llm_cache_free_slots(Core* c) { return (int)c->free_slots.size(); }

void llm_cache_free_pages(Core* c, int* out) {
  for (size_t g = 0; g < c->groups.size(); ++g) out[g] = (int)c->groups[g].pool.free.size();
}

// pages each group must add so that the request can grow by new_tokens
int llm_cache_pages_needed(Core* c, int64_t key, int new_tokens, int* out) {
  auto it = c->requests.find(key);
  if (it == c->requests.end()) return E_UNKNOWN;
  c->needed(it->second, new_tokens, out);
  return 0;
}

// Room for every (request, new tokens) of a step, or nothing changed.  Returns 0; 1 when the
// pages do not suffice (info = group, needed, free); a negative code on misuse (info[0] = index
// of the offending entry, info[1], info[2] = its length and count where that helps).
int llm_cache_reserve(Core* c, int n, const int64_t* keys, const int* counts, int* info) {
  const int G = (int)c->groups.size();
  std::vector<int> need(G, 0), k(G, 0);
  std::vector<Request*> reqs(n);
  for (int i = 0; i < n; ++i) {
    info[0] = i;
    for (int j = 0; j < i; ++j)
      if (keys[j] == keys[i]) return E_TWICE_IN_STEP;
    auto it = c->requests.find(keys[i]);
    if (it == c->requests.end()) return E_UNKNOWN;
    reqs[i] = &it->second;
    if (counts[i] <= 0) return E_EMPTY_ENTRY;
    if (reqs[i]->length + counts[i] > c->max_context) {
      info[1] = reqs[i]->length;
      info[2] = counts[i];
      return E_CONTEXT;
    }
    c->needed(*reqs[i], counts[i], k.data());
    for (int g = 0; g < G; ++g) need[g] += k[g];
  }
  for (int g = 0; g < G; ++g)
    if (need[g] > (int)c->groups[g].pool.free.size()) {
      ++c->counters[3];
      info[0] = g;
      info[1] = need[g];
      info[2] = (int)c->groups[g].pool.free.size();
      return 1;
    }
  std::vector<int> got;
  for (int i = 0; i < n; ++i) {
    Request& r = *reqs[i];
    c->needed(r, counts[i], k.data());
    for (int g = 0; g < G; ++g) {
      if (!k[g]) continue;
      got.clear();
      c->groups[g].pool.alloc(k[g], &got);       // cannot fail: the sum was checked above
      c->counters[0] += k[g];
      for (int p : got) {
        c->groups[g].set(r.slot * c->pages_per_request + (int)r.pages[g].size(), p);
        r.pages[g].push_back(p);
      }
    }
  }
  return 0;
}

// The request now holds n more tokens; pages that a window has passed go back.
int llm_cache_advance(Core* c, int64_t key, int n) {
  auto it = c->requests.find(key);
  if (it == c->requests.end()) return E_UNKNOWN;
  Request& r = it->second;
  for (size_t g = 0; g < c->groups.size(); ++g)
    if ((long long)r.length + n > (long long)r.pages[g].size() * c->page_size) return E_PAST_RESERVED;
  r.length += n;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    Group& grp = c->groups[g];
    int keep_from = c->first_needed_page(grp, r.length);
    if (keep_from > (int)r.pages[g].size()) keep_from = (int)r.pages[g].size();
    if (keep_from > r.first_live[g]) {
      const int gone = keep_from - r.first_live[g];
      const int rc = grp.pool.release(r.pages[g].data() + r.first_live[g], gone);
      if (rc) return rc;
      c->counters[1] += gone;
      c->counters[2] += gone;
      for (int j = r.first_live[g]; j < keep_from; ++j) {
        r.pages[g][j] = -1;
        grp.set(r.slot * c->pages_per_request + j, -1);
      }
      r.first_live[g] = keep_from;
    }
  }
  return 0;
}

// Forget everything past `length` tokens (kv.rs:792-816).  A group that has given pages back to
// its window cannot be rewound into them.  info[0] = the group at fault.
int llm_cache_truncate(Core* c, int64_t key, int length, int* info) {
  auto it = c->requests.find(key);
  if (it == c->requests.end()) return E_UNKNOWN;
  Request& r = it->second;
  if (length > r.length || length < 0) return E_LENGTHEN;
  if (c->has_state && length < r.length) return E_STATE_REWIND;
  for (size_t g = 0; g < c->groups.size(); ++g)
    if (c->first_needed_page(c->groups[g], length) < r.first_live[g]) {
      info[0] = (int)g;
      return E_WINDOW_GONE;
    }
  const int keep = (length + c->page_size - 1) / c->page_size;
  std::vector<int> gone;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    Group& grp = c->groups[g];
    gone.clear();
    for (int j = keep; j < (int)r.pages[g].size(); ++j) {
      if (r.pages[g][j] >= 0) gone.push_back(r.pages[g][j]);
      grp.set(r.slot * c->pages_per_request + j, -1);
    }
    const int rc = grp.pool.release(gone.data(), (int)gone.size());
    if (rc) return rc;
    c->counters[1] += (long long)gone.size();
    if ((int)r.pages[g].size() > keep) r.pages[g].resize(keep);
  }
  r.length = length;
  return 0;
}

// The request is over: its pages and its slot go back.
int llm_cache_close(Core* c, int64_t key) {
  auto it = c->requests.find(key);
  if (it == c->requests.end()) return E_UNKNOWN;
  Request& r = it->second;
  std::vector<int> gone;
  for (size_t g = 0; g < c->groups.size(); ++g) {
    Group& grp = c->groups[g];
    gone.clear();
    for (int j = 0; j < (int)r.pages[g].size(); ++j)
      if (r.pages[g][j] >= 0) {
        gone.push_back(r.pages[g][j]);
        grp.set(r.slot * c->pages_per_request + j, -1);
      }
    const int rc = grp.pool.release(gone.data(), (int)gone.size());
    if (rc) return rc;
    c->counters[1] += (long long)gone.size();
  }
  c->free_slots.push_back(r.slot);
  for (size_t i = 0; i < c->fresh_slots.size(); ++i)
    if (c->fresh_slots[i] == r.slot) {
      c->fresh_slots.erase(c->fresh_slots.begin() + i);
      break;
    }
  c->requests.erase(it);
  return 0;
}

int llm_cache_pending_updates(Core* c, int group) { return (int)c->groups[group].dirty_cells.size(); }

// The (request slot, page index, page id) triples of a group since the last call, one per table
// cell (the last value wins), into out[3 * n]; returns n and forgets them.
int llm_cache_take_updates(Core* c, int group, int* out) {
  Group& g = c->groups[group];
  int n = 0;
  for (int cell : g.dirty_cells) {
    out[3 * n] = cell / c->pages_per_request;
    out[3 * n + 1] = cell % c->pages_per_request;
    out[3 * n + 2] = g.pending[cell];
    g.dirty[cell] = 0;
    ++n;
  }
  g.dirty_cells.clear();
  return n;
}

// The request slots opened since the last call (their fixed-size state must be zeroed).
int llm_cache_take_fresh(Core* c, int* out, int cap) {
  const int n = (int)c->fresh_slots.size() < cap ? (int)c->fresh_slots.size() : cap;
  for (int i = 0; i < n; ++i) out[i] = c->fresh_slots[i];
  c->fresh_slots.erase(c->fresh_slots.begin(), c->fresh_slots.begin() + n);
  return n;
}

// The page ids of a request in a group by page index (-1 = given back); returns how many there are.
int llm_cache_pages_of(Core* c, int64_t key, int group, int* out, int cap) {
  auto it = c->requests.find(key);
  if (it == c->requests.end()) return E_UNKNOWN;
  if (group < 0 || group >= (int)c->groups.size()) return E_ARGUMENT;
  const std::vector<int>& p = it->second.pages[group];
  for (int i = 0; i < (int)p.size() && i < cap; ++i) out[i] = p[i];
  return (int)p.size();
}

int llm_cache_live(Core* c, int64_t* out, int cap) {
  int n = 0;
  for (auto& kv : c->requests) {
    if (n < cap) out[n] = kv.first;
    ++n;
  }
  return n;
}

void llm_cache_counters(Core* c, long long* out) { memcpy(out, c->counters, sizeof(c->counters)); }

// No page lost, none held twice, none both free and held; the same for request slots.
// Returns 0 or the code of what is wrong, with the group in info[0].
int llm_cache_check(Core* c, int* info) {
  for (size_t g = 0; g < c->groups.size(); ++g) {
    info[0] = (int)g;
    const Pool& pool = c->groups[g].pool;
    std::vector<int> count(pool.n, 0);
    int held = 0;
    for (auto& kv : c->requests)
      for (int p : kv.second.pages[g])
        if (p >= 0) {
          if (p >= pool.n || count[p]) return E_HELD_TWICE;
          count[p] = 1;
          ++held;
        }
    std::vector<char> in_free(pool.n, 0);
    for (int p : pool.free) {
      if (p < 0 || p >= pool.n) return E_LOST;
      if (count[p]) return E_FREE_AND_HELD;
      if (in_free[p]) return E_FREE_TWICE;
      in_free[p] = 1;
    }
    if ((int)pool.free.size() + held != pool.n) return E_LOST;
    if (pool.n_held != held) return E_COUNT_OFF;
  }
  std::vector<char> slot(c->max_requests, 0);
  for (auto& kv : c->requests) {
    const int s = kv.second.slot;
    if (s < 0 || s >= c->max_requests || slot[s]) return E_SLOT_TWICE;
    slot[s] = 1;
  }
  for (int s : c->free_slots) {
    if (s < 0 || s >= c->max_requests || slot[s]) return E_SLOT_TWICE;
    slot[s] = 1;
  }
  if (c->requests.size() + c->free_slots.size() != (size_t)c->max_requests) return E_SLOT_LOST;
  return 0;
}

// ---- the pool alone (what the tests of the pool drive)
Pool* llm_pool_new(int n_pages) { return n_pages > 0 ? new Pool(n_pages) : nullptr; }
void llm_pool_delete(Pool* p) { delete p; }
int llm_pool_free(Pool* p) { return (int)p->free.size(); }
int llm_pool_held(Pool* p) { return p->n_held; }
// k pages into out, or -1 with nothing changed
int llm_pool_alloc(Pool* p, int k, int* out) {
  std::vector<int> got;
  if (k < 0 || !p->alloc(k, &got)) return -1;
  for (int i = 0; i < k; ++i) out[i] = got[i];
  return k;
}
int llm_pool_release(Pool* p, const int* pages, int k) { return p->release(pages, k); }

}  // extern "C"
