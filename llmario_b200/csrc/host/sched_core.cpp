// The scheduler's decisions, on the host: which requests run, which tokens of which request the
// next step feeds, who gives way when pages run out.  Plain C++17 with a C interface, in the same
// library as the cache bookkeeping, which it asks through that library's own C functions.  It
// sees requests as lengths and limits; the token ids stay with the caller.
//
// Rules, after the reference's step loop (crates/engine/server/src/engine.rs:621-710, 780-994):
//   * waiting requests are served first come, first served, while a request slot is free;
//   * a step first gives one token to every running request that is decoding, then fills what is
//     left of the token budget with prompt portions, oldest request first; the last portion of
//     one prompt may share a step with the first portion of the next (engine.rs:893-911);
//   * a request finishes on an end-of-sequence token ("stop"), after max_tokens generated tokens
//     or when its context is full ("length") (engine.rs:1185-1216).
// When pages run out (the reference fails the newest job, engine.rs:940-963; its unused policy
// crate retracts a running request and recomputes it later, crates/engine/sched/src/lib.rs:
// 148-174): prompt portions are shortened or left out of the step first; if even the decoding
// requests do not fit, the most recently admitted running request is preempted: its pages are
// given back and it returns to the head of the waiting queue, to be recomputed once all of it fits
// the free pages.  A request that cannot fit even alone is failed.
#include <algorithm>
#include <cstdint>
#include <deque>
#include <unordered_map>
#include <unordered_set>
#include <vector>

struct Core;
extern "C" {
int llm_cache_has(Core* c, int64_t key);
int llm_cache_info(Core* c, int64_t key, int* slot, int* length);
int llm_cache_free_slots(Core* c);
void llm_cache_free_pages(Core* c, int* out);
int llm_cache_pages_needed(Core* c, int64_t key, int new_tokens, int* out);
int llm_cache_close(Core* c, int64_t key);
int llm_cache_pages_of(Core* c, int64_t key, int group, int* out, int cap);
}

namespace {

enum State { WAITING = 0, RUNNING = 1, FINISHED = 2 };
enum Reason { R_NONE = 0, R_STOP = 1, R_LENGTH = 2, R_ERROR = 3, R_ABORTED = 4 };
enum Counter { C_ADMITTED, C_FINISHED, C_PREEMPTIONS, C_FAILED, C_STEPS, C_PROMPT_TOKENS, C_DECODE_TOKENS,
               C_STEPS_AHEAD, N_COUNTERS };

struct Req {
  int64_t key = 0;
  int prompt_len = 0, out_len = 0;
  int computed = 0;              // tokens of prompt + output whose keys are in the cache
  int max_tokens = 0;
  bool ignore_eos = false, penalties = false;
  int state = WAITING, reason = R_NONE, preemptions = 0;
  // What a step that is still running will have added when it ends (no end-of-sequence token
  // assumed); non-zero only while the step after it is being planned.
  int fly_count = 0, fly_samples = 0;
  int done() const { return computed + fly_count; }         // tokens in the cache, the running step's included
  int outs() const { return out_len + fly_samples; }
  int seq() const { return prompt_len + out_len + fly_samples; }
};

struct Entry { int64_t key; int start, count, samples; };

struct Sched {
  Core* cache;
  int n_groups, page_size, budget, max_context;
  std::unordered_map<int64_t, Req> reqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;              // in order of admission
  std::unordered_set<int> eos;
  long long counters[N_COUNTERS] = {};

  std::vector<int> pages_for(const Req& r, int count, bool opened) {
    std::vector<int> need(n_groups);
    if (opened && llm_cache_has(cache, r.key)) {
      llm_cache_pages_needed(cache, r.key, count, need.data());
    } else {
      for (int g = 0; g < n_groups; ++g) need[g] = (count + page_size - 1) / page_size;
    }
    return need;
  }
  static bool fits(const std::vector<int>& need, const std::vector<int>& free) {
    for (size_t g = 0; g < need.size(); ++g)
      if (need[g] > free[g]) return false;
    return true;
  }
  static void take(const std::vector<int>& need, std::vector<int>* free) {
    for (size_t g = 0; g < need.size(); ++g) (*free)[g] -= need[g];
  }
  // largest count <= n whose pages fit in `free`
  int fit(const Req& r, int n, const std::vector<int>& free, bool opened) {
    if (n <= 0) return 0;
    opened = opened && llm_cache_has(cache, r.key);
    if (fits(pages_for(r, n, opened), free)) return n;
    if (n_groups == 0) return n;
    int have = 0, held = 0, slot = 0;
    if (opened) {
      llm_cache_info(cache, r.key, &slot, &have);
      held = llm_cache_pages_of(cache, r.key, 0, nullptr, 0);
    }
    const int least = *std::min_element(free.begin(), free.end());
    const long long room = (long long)(held + least) * page_size - have;
    return (int)std::max<long long>(0, std::min<long long>(n, room));
  }
  void drop_running(int64_t key) {
    running.erase(std::remove(running.begin(), running.end(), key), running.end());
  }
  void close_pages(int64_t key) {
    if (llm_cache_has(cache, key)) llm_cache_close(cache, key);
  }
  void preempt(Req& r) {
    drop_running(r.key);
    close_pages(r.key);
    r.computed = 0;
    r.state = WAITING;
    ++r.preemptions;
    ++counters[C_PREEMPTIONS];
    waiting.push_front(r.key);
  }
  void fail(Req& r) {
    drop_running(r.key);
    close_pages(r.key);
    r.state = FINISHED;
    r.reason = R_ERROR;
    ++counters[C_FAILED];
  }
  void finish(Req& r, int reason) {
    drop_running(r.key);
    close_pages(r.key);
    r.state = FINISHED;
    r.reason = reason;
    ++counters[C_FINISHED];
  }
};

struct Plan {
  std::vector<Entry> entries;
  std::vector<int64_t> preempted, failed, admitted;
};

// ahead: the plan is made while a step is still running (its contribution stands in the
// requests' fly_* fields).  Then nothing may be decided that needs the tokens it draws: where a
// request would have to give way, or the step would be empty, the answer is false and nothing
// has changed.
bool make_plan(Sched& s, Plan* plan, bool ahead = false) {
  for (;;) {
    std::vector<int> free(s.n_groups);
    llm_cache_free_pages(s.cache, free.data());
    int used = 0;
    std::vector<Entry> entries;
    bool ok = true;
    // 1. decoding requests, one token each
    for (int64_t key : s.running) {
      Req& r = s.reqs[key];
      if (r.done() == r.seq() - 1 && r.outs() > 0) {
        if (ahead) {
          // its last token is the one in flight: it ends with the running step
          if (r.outs() >= r.max_tokens || r.seq() >= s.max_context) continue;
        }
        const std::vector<int> need = s.pages_for(r, 1, true);
        if (used >= s.budget) break;
        if (!Sched::fits(need, free)) {
          if (ahead) return false;      // someone has to go: decided with all facts known
          ok = false;
          break;
        }
        Sched::take(need, &free);
        entries.push_back({key, r.done(), 1, 1});
        ++used;
      }
    }
    if (!ok) {      // the newest running request gives way, or a lone one fails
      Req& victim = s.reqs[s.running.back()];
      if (s.running.size() == 1) {
        s.fail(victim);
        plan->failed.push_back(victim.key);
      } else {
        s.preempt(victim);
        plan->preempted.push_back(victim.key);
      }
      continue;
    }
    // 2. prompt portions of running requests, oldest first
    for (int64_t key : s.running) {
      if (used >= s.budget) break;
      Req& r = s.reqs[key];
      if (r.outs() > 0 && r.done() == r.seq() - 1) continue;
      const int left = r.seq() - r.done();
      const int n = s.fit(r, std::min(left, s.budget - used), free, true);
      if (n <= 0) continue;
      Sched::take(s.pages_for(r, n, true), &free);
      entries.push_back({key, r.done(), n, r.done() + n == r.seq() ? 1 : 0});
      used += n;
    }
    // 3. admission
    while (!s.waiting.empty() && used < s.budget) {
      int planned_new = 0;
      for (const Entry& e : entries)
        if (!llm_cache_has(s.cache, e.key)) ++planned_new;
      if (llm_cache_free_slots(s.cache) - planned_new <= 0) break;
      Req& r = s.reqs[s.waiting.front()];
      const int left = r.seq() - r.computed;
      if (r.preemptions) {
        // a request that lost its pages comes back only when all of it fits: otherwise it would
        // take the pages the older requests are about to need and be preempted again
        if (!plan->preempted.empty() || !Sched::fits(s.pages_for(r, left + 1, false), free)) break;
      }
      const int n = s.fit(r, std::min(left, s.budget - used), free, false);
      if (n <= 0) break;
      s.waiting.pop_front();
      r.state = RUNNING;
      s.running.push_back(r.key);
      ++s.counters[C_ADMITTED];
      plan->admitted.push_back(r.key);
      Sched::take(s.pages_for(r, n, false), &free);
      entries.push_back({r.key, r.computed, n, r.computed + n == r.seq() ? 1 : 0});
      used += n;
    }
    if (entries.empty() && ahead) return false;
    if (entries.empty() && !s.running.empty()) {
      // nothing fits although requests are running: a prompt portion is stuck for want of pages
      Req& victim = s.reqs[s.running.back()];
      if (s.running.size() == 1) {
        s.fail(victim);
        plan->failed.push_back(victim.key);
      } else {
        s.preempt(victim);
        plan->preempted.push_back(victim.key);
      }
      continue;
    }
    if (entries.empty() && !s.waiting.empty() && s.running.empty()) {
      Req& r = s.reqs[s.waiting.front()];
      s.waiting.pop_front();
      s.fail(r);
      plan->failed.push_back(r.key);
      continue;
    }
    plan->entries = entries;
    break;
  }
  ++s.counters[C_STEPS];
  return true;
}

}  // namespace

extern "C" {

// Error codes of llm_sched_add.
enum { S_EMPTY_PROMPT = -1, S_PROMPT_TOO_LONG = -2, S_KEY_IN_USE = -3, S_UNKNOWN = -4, S_ARGUMENT = -5 };

Sched* llm_sched_new(Core* cache, int n_groups, int page_size, int token_budget, int max_context) {
  if (!cache || n_groups < 0 || page_size <= 0 || token_budget <= 0 || max_context <= 0) return nullptr;
  Sched* s = new Sched();
  s->cache = cache;
  s->n_groups = n_groups;
  s->page_size = page_size;
  s->budget = token_budget;
  s->max_context = max_context;
  return s;
}
void llm_sched_delete(Sched* s) { delete s; }

void llm_sched_set_eos(Sched* s, int n, const int* ids) {
  s->eos.clear();
  for (int i = 0; i < n; ++i) s->eos.insert(ids[i]);
}

// Queue a request.  An empty prompt, or one that leaves no room in the context, is refused
// (engine.rs:788-798).
int llm_sched_add(Sched* s, int64_t key, int prompt_len, int max_tokens, int ignore_eos, int penalties) {
  if (prompt_len <= 0) return S_EMPTY_PROMPT;
  if (prompt_len >= s->max_context) return S_PROMPT_TOO_LONG;
  auto it = s->reqs.find(key);
  if (it != s->reqs.end() && it->second.state != FINISHED) return S_KEY_IN_USE;
  Req r;
  r.key = key;
  r.prompt_len = prompt_len;
  r.max_tokens = max_tokens;
  r.ignore_eos = ignore_eos != 0;
  r.penalties = penalties != 0;
  s->reqs[key] = r;
  s->waiting.push_back(key);
  return 0;
}

// Forget a finished request (its key may be used again).
int llm_sched_forget(Sched* s, int64_t key) {
  auto it = s->reqs.find(key);
  if (it == s->reqs.end()) return S_UNKNOWN;
  if (it->second.state != FINISHED) return S_ARGUMENT;
  s->reqs.erase(it);
  return 0;
}

int llm_sched_has_work(Sched* s) { return (!s->waiting.empty() || !s->running.empty()) ? 1 : 0; }
int llm_sched_sizes(Sched* s, int* waiting, int* running) {
  *waiting = (int)s->waiting.size();
  *running = (int)s->running.size();
  return 0;
}

// out: computed, output length, state, reason, preemptions
int llm_sched_request(Sched* s, int64_t key, int* out) {
  auto it = s->reqs.find(key);
  if (it == s->reqs.end()) return S_UNKNOWN;
  const Req& r = it->second;
  out[0] = r.computed, out[1] = r.out_len, out[2] = r.state, out[3] = r.reason, out[4] = r.preemptions;
  return 0;
}

// Decide the next step.  Changes the queues (admission, preemption, failure) but feeds nothing:
// the caller runs the step and reports back with llm_sched_complete.
// entries: keys and (start, count, samples) triples; events: keys of the requests preempted,
// failed and admitted by this call, in that order, their numbers in n_events[0..2].  cap: room
// in keys / triples (entries) and in events; it must be at least the number of waiting and running
// requests (S_ARGUMENT otherwise, before anything is decided).  Returns the number of entries.
int llm_sched_plan(Sched* s, int cap, int64_t* keys, int* triples, int64_t* events, int* n_events) {
  if (cap < (int)(s->waiting.size() + s->running.size())) return S_ARGUMENT;
  Plan plan;
  make_plan(*s, &plan);
  for (size_t i = 0; i < plan.entries.size(); ++i) {
    keys[i] = plan.entries[i].key;
    triples[3 * i] = plan.entries[i].start;
    triples[3 * i + 1] = plan.entries[i].count;
    triples[3 * i + 2] = plan.entries[i].samples;
  }
  // (a request is preempted, failed or admitted at most once by one call, and never both
  // preempted and admitted: there are no more events than requests)
  int at = 0;
  for (int64_t k : plan.preempted) events[at++] = k;
  for (int64_t k : plan.failed) events[at++] = k;
  for (int64_t k : plan.admitted) events[at++] = k;
  n_events[0] = (int)plan.preempted.size();
  n_events[1] = (int)plan.failed.size();
  n_events[2] = (int)plan.admitted.size();
  return (int)plan.entries.size();
}

// The step after `flying` (n entries: keys and (start, count, samples) triples; flying_events: how
// many requests that plan preempted or failed), decided while it is still running and the tokens
// it draws are unknown.  The planner runs as for any step, on the requests as they will stand
// when the flying step ends without an end-of-sequence token: decoding requests get one more
// token (the one in flight is their input), prompts their next portions, waiting requests are
// admitted into free slots.  A request whose last token is in flight (max_tokens or the context
// reached) is left out; it keeps its slot and pages until the flying step is reported.  Returns
// the number of entries, with the admitted requests in events / n_events[2], or -1 when the step
// cannot be known yet: the flying plan preempted or failed someone, pages are short so that a
// request would have to give way, or nothing could run.  (Penalties do not stand in the way: the
// sampler counts the token in flight on the device.)  A request that does end on an end-of-sequence token drawn by the flying
// step has a row too many in this one; llm_sched_complete passes over it.
int llm_sched_plan_ahead(Sched* s, int n, const int64_t* fkeys, const int* ftriples, int flying_events,
                         int cap, int64_t* keys, int* triples, int64_t* events, int* n_events) {
  if (flying_events || n <= 0) return -1;
  if (cap < (int)(s->waiting.size() + s->running.size())) return S_ARGUMENT;
  std::vector<Req*> touched;
  for (int i = 0; i < n; ++i) {
    auto it = s->reqs.find(fkeys[i]);
    if (it == s->reqs.end() || it->second.state != RUNNING) continue;     // gone meanwhile (aborted)
    it->second.fly_count = ftriples[3 * i + 1];
    it->second.fly_samples = ftriples[3 * i + 2] ? 1 : 0;
    touched.push_back(&it->second);
  }
  Plan plan;
  const bool known = make_plan(*s, &plan, true);
  for (Req* r : touched) r->fly_count = r->fly_samples = 0;
  if (!known) return -1;
  ++s->counters[C_STEPS_AHEAD];
  for (size_t i = 0; i < plan.entries.size(); ++i) {
    keys[i] = plan.entries[i].key;
    triples[3 * i] = plan.entries[i].start;
    triples[3 * i + 1] = plan.entries[i].count;
    triples[3 * i + 2] = plan.entries[i].samples;
  }
  int at = 0;
  for (int64_t k : plan.admitted) events[at++] = k;
  n_events[0] = n_events[1] = 0;
  n_events[2] = (int)plan.admitted.size();
  return (int)plan.entries.size();
}

// The step ran.  tokens[i]: the token drawn for entry i (read only where the entry samples).
// finished: keys of the requests that ended, reasons: why (1 stop, 2 length).  Returns their number.
int llm_sched_complete(Sched* s, int n, const int64_t* keys, const int* triples, const int* tokens,
                       int64_t* finished, int* reasons) {
  int done = 0;
  for (int i = 0; i < n; ++i) {
    auto it = s->reqs.find(keys[i]);
    if (it == s->reqs.end()) continue;
    Req& r = it->second;
    if (r.state != RUNNING) continue;      // it ended while this step, planned ahead, was already running
    const int count = triples[3 * i + 1], samples = triples[3 * i + 2];
    r.computed += count;
    if (r.out_len > 0 && count == 1 && samples) ++s->counters[C_DECODE_TOKENS];
    else s->counters[C_PROMPT_TOKENS] += count;
    if (!samples) continue;
    ++r.out_len;
    if (s->eos.count(tokens[i]) && !r.ignore_eos) s->finish(r, R_STOP);             // engine.rs:1185-1188
    else if (r.out_len >= r.max_tokens) s->finish(r, R_LENGTH);                    // engine.rs:1211-1213
    else if (r.seq() >= s->max_context) s->finish(r, R_LENGTH);                    // engine.rs:1214-1216
    if (r.state == FINISHED) {
      finished[done] = r.key;
      reasons[done] = r.reason;
      ++done;
    }
  }
  return done;
}

// Drop a request wherever it is (a client that went away, engine.rs:695-703).
int llm_sched_abort(Sched* s, int64_t key) {
  auto it = s->reqs.find(key);
  if (it == s->reqs.end()) return S_UNKNOWN;
  Req& r = it->second;
  s->waiting.erase(std::remove(s->waiting.begin(), s->waiting.end(), key), s->waiting.end());
  s->drop_running(key);
  s->close_pages(key);
  r.state = FINISHED;
  r.reason = R_ABORTED;
  return 0;
}

// End a request as failed wherever it is: the step that held it could not be trusted (the
// reference turns such a failure into an error event for the job, engine.rs:1140).
int llm_sched_fail(Sched* s, int64_t key) {
  const int rc = llm_sched_abort(s, key);
  if (rc != 0) return rc;
  s->reqs.find(key)->second.reason = R_ERROR;
  ++s->counters[C_FAILED];
  return 0;
}

// waiting keys then running keys, in their order; returns -1 when cap is too small
int llm_sched_queues(Sched* s, int cap, int64_t* out, int* n_waiting, int* n_running) {
  *n_waiting = (int)s->waiting.size();
  *n_running = (int)s->running.size();
  if (*n_waiting + *n_running > cap) return -1;
  int at = 0;
  for (int64_t k : s->waiting) out[at++] = k;
  for (int64_t k : s->running) out[at++] = k;
  return at;
}

void llm_sched_counters(Sched* s, long long* out) {
  for (int i = 0; i < N_COUNTERS; ++i) out[i] = s->counters[i];
}

}  // extern "C"
