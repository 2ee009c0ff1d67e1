// Host runtime: page pools, cache bookkeeping, scheduler, step packing.  See runtime.h.
//
// Page pool after the reference's BlockTable (include/tge/models/block_table.hpp:21-130): allocate
// pops a LIFO free list and sets the count to one, a full pool is an error, share adds a reference,
// release drops one and returns the page at zero, every misuse is an error.  The scheduler keeps the
// shape of the reference's only scheduler, the loop of `bench continuous` (apps/cli/main.cpp:1451-1644:
// live decodes first, then prompt work), and adds what a paged cache needs: a token budget, portions,
// admission by free pages, and preemption with recompute when pages run out.
#include "runtime.h"

#include "random_weights.h"

#include <algorithm>
#include <cstring>
#include <thread>
#include <cstdarg>
#include <cstdio>
#include <deque>
#include <memory>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

thread_local std::string g_error;

int fail(int code, const char* format, ...) {
  char buffer[512];
  va_list args;
  va_start(args, format);
  vsnprintf(buffer, sizeof(buffer), format, args);
  va_end(args);
  g_error = buffer;
  return code;
}

constexpr int NO_PAGE = -1;

}  // namespace

// ------------------------------------------------------------------------------------------------------
struct TgeRtPool {
  std::vector<int> refcount;
  std::vector<int> free_list;      // back = next page handed out

  explicit TgeRtPool(int pages) : refcount(pages, 0) {
    free_list.reserve(pages);
    for (int page = pages - 1; page >= 0; --page) free_list.push_back(page);   // page 0 is handed out first
  }
  int capacity() const { return (int)refcount.size(); }
  int free_count() const { return (int)free_list.size(); }
  int live(int page) const {
    if (page < 0 || page >= capacity()) return fail(TGE_RT_PAGE_ERROR, "page pool: page id %d out of range", page);
    if (refcount[page] <= 0) return fail(TGE_RT_PAGE_ERROR, "page pool: page %d is not live", page);
    return 0;
  }
  int allocate() {
    if (free_list.empty()) return fail(TGE_RT_EXHAUSTED, "page pool: no free page");
    const int page = free_list.back();
    free_list.pop_back();
    refcount[page] = 1;
    return page;
  }
  int share(int page) {
    if (int rc = live(page)) return rc;
    ++refcount[page];
    return 0;
  }
  int release(int page) {
    if (int rc = live(page)) return rc;
    if (--refcount[page] == 0) {
      free_list.push_back(page);
      return 1;
    }
    return 0;
  }
  int check() const {
    std::vector<char> seen(capacity(), 0);
    for (int page : free_list) {
      if (seen[page]) return fail(TGE_RT_PAGE_ERROR, "page pool: page %d is on the free list twice", page);
      seen[page] = 1;
      if (refcount[page] != 0) return fail(TGE_RT_PAGE_ERROR, "page pool: free page %d has references", page);
    }
    for (int page = 0; page < capacity(); ++page) {
      if (refcount[page] < 0) return fail(TGE_RT_PAGE_ERROR, "page pool: page %d has a negative count", page);
      if (refcount[page] == 0 && !seen[page])
        return fail(TGE_RT_PAGE_ERROR, "page pool: page %d is lost (neither free nor referenced)", page);
    }
    return 0;
  }
};

// ------------------------------------------------------------------------------------------------------
struct TgeRtCache {
  struct Group {
    int window;                                              // < 0: none
    std::unique_ptr<TgeRtPool> pool;
    std::unordered_map<int64_t, std::vector<int>> tables;    // request -> logical page -> physical id
  };
  struct Live {
    int slot, tokens, computed;
    long long order;
  };
  int page_size, max_requests;
  std::vector<Group> groups;
  std::vector<int> free_slots;
  std::unordered_map<int64_t, Live> live;
  long long admissions = 0;

  TgeRtCache(int page, int requests) : page_size(page), max_requests(requests) {
    for (int slot = requests - 1; slot >= 0; --slot) free_slots.push_back(slot);
  }
  int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
  const Live* find(int64_t request) const {
    auto it = live.find(request);
    return it == live.end() ? nullptr : &it->second;
  }
  int first_needed_page(const Group& group, int computed_tokens) const {
    if (group.window < 0) return 0;
    const int first_key = std::max(computed_tokens - group.window + 1, 0);
    return first_key / page_size;
  }
  int missing(const Group& group, int64_t request, int total_tokens) const {
    auto it = group.tables.find(request);
    const int have = it == group.tables.end() ? 0 : (int)it->second.size();
    return std::max(pages_for(total_tokens) - have, 0);
  }
  bool can_grow(int64_t request, int total_tokens) const {
    for (const Group& group : groups)
      if (missing(group, request, total_tokens) > group.pool->free_count()) return false;
    return true;
  }
  bool fits_empty_pool(int total_tokens) const {
    for (const Group& group : groups)
      if (pages_for(total_tokens) > group.pool->capacity()) return false;
    return true;
  }
  int admit(int64_t request) {
    if (live.count(request)) return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is already live", (long long)request);
    if (free_slots.empty()) return fail(TGE_RT_EXHAUSTED, "cache manager: no free state slot");
    const int slot = free_slots.back();
    free_slots.pop_back();
    live[request] = Live{slot, 0, 0, admissions++};
    for (Group& group : groups) group.tables[request].clear();
    return slot;
  }
  int grow(int64_t request, int total_tokens) {
    auto it = live.find(request);
    if (it == live.end()) return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is not live", (long long)request);
    for (const Group& group : groups) {
      const int need = missing(group, request, total_tokens);
      if (need > group.pool->free_count())
        return fail(TGE_RT_EXHAUSTED, "cache manager: request %lld needs %d more pages, %d are free", (long long)request,
                    need, group.pool->free_count());
    }
    for (Group& group : groups) {
      const int need = missing(group, request, total_tokens);
      std::vector<int>& table = group.tables[request];
      for (int i = 0; i < need; ++i) table.push_back(group.pool->allocate());
    }
    it->second.tokens = std::max(it->second.tokens, total_tokens);
    return 0;
  }
  int release_behind_window(int64_t request, int computed_tokens) {
    int released = 0;
    for (Group& group : groups) {
      auto it = group.tables.find(request);
      if (it == group.tables.end()) continue;
      std::vector<int>& table = it->second;
      const int end = std::min(first_needed_page(group, computed_tokens), (int)table.size());
      for (int index = 0; index < end; ++index) {
        if (table[index] != NO_PAGE) {
          group.pool->release(table[index]);
          table[index] = NO_PAGE;
          ++released;
        }
      }
    }
    return released;
  }
  int set_computed(int64_t request, int tokens) {
    auto it = live.find(request);
    if (it == live.end()) return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is not live", (long long)request);
    if (tokens > it->second.tokens)
      return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld computed %d tokens but holds pages for %d",
                  (long long)request, tokens, it->second.tokens);
    if (tokens > it->second.computed) it->second.computed = tokens;
    release_behind_window(request, it->second.computed);
    return 0;
  }
  int free_request(int64_t request) {
    auto it = live.find(request);
    if (it == live.end())
      return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is not live (freed twice?)", (long long)request);
    for (Group& group : groups) {
      auto table = group.tables.find(request);
      if (table == group.tables.end()) continue;
      for (int page : table->second)
        if (page != NO_PAGE) group.pool->release(page);
      group.tables.erase(table);
    }
    free_slots.push_back(it->second.slot);
    live.erase(it);
    return 0;
  }
  int check() const {
    for (const Group& group : groups) {
      if (int rc = group.pool->check()) return rc;
      std::vector<int> held(group.pool->capacity(), 0);
      for (const auto& entry : group.tables) {
        if (!live.count(entry.first))
          return fail(TGE_RT_PAGE_ERROR, "cache manager: a table exists for dead request %lld", (long long)entry.first);
        for (int page : entry.second)
          if (page != NO_PAGE) {
            if (page < 0 || page >= group.pool->capacity())
              return fail(TGE_RT_PAGE_ERROR, "cache manager: a table holds page id %d outside the pool", page);
            ++held[page];
          }
      }
      for (int page = 0; page < group.pool->capacity(); ++page)
        if (group.pool->refcount[page] != held[page])
          return fail(TGE_RT_PAGE_ERROR, "cache manager: page %d is held %d times but counts %d references", page,
                      held[page], group.pool->refcount[page]);
    }
    std::vector<char> taken(max_requests, 0);
    for (const auto& entry : live) {
      const int slot = entry.second.slot;
      if (slot < 0 || slot >= max_requests || taken[slot]) return fail(TGE_RT_PAGE_ERROR, "cache manager: a state slot is held twice");
      taken[slot] = 1;
    }
    for (int slot : free_slots) {
      if (slot < 0 || slot >= max_requests || taken[slot]) return fail(TGE_RT_PAGE_ERROR, "cache manager: a state slot is held twice");
      taken[slot] = 1;
    }
    if ((int)live.size() + (int)free_slots.size() != max_requests) return fail(TGE_RT_PAGE_ERROR, "cache manager: a state slot is lost");
    return 0;
  }
};

// ------------------------------------------------------------------------------------------------------
// One step's packing.  `Source` yields for portion i its request, tokens and wanted places.
namespace {

struct PortionView {
  int64_t request;
  const int* tokens;
  int count;
  const int* wants;
  int want_count;
};

int pack_step(TgeRtCache* cache, const std::vector<PortionView>& portions, int vocab_size, int max_model_len,
              int fixed_width, int pad_rows, bool reserve, int* out, long long capacity, TgeRtStepLayout* layout) {
  int S = (int)portions.size();
  if (S == 0) return fail(TGE_RT_VALUE_ERROR, "step: no portions");
  if ((int)cache->groups.size() > 8) return fail(TGE_RT_VALUE_ERROR, "step: more than 8 cache groups");
  // validate before touching anything
  {
    std::unordered_set<int64_t> seen;
    for (const PortionView& p : portions) {
      if (!seen.insert(p.request).second)
        return fail(TGE_RT_VALUE_ERROR, "request %lld appears twice in one step", (long long)p.request);
      if (p.count <= 0) return fail(TGE_RT_VALUE_ERROR, "request %lld: a portion needs at least one token", (long long)p.request);
      if (p.count > 1 && pad_rows > S)
        return fail(TGE_RT_VALUE_ERROR, "step: only a step of single tokens can be padded (%d portions to %d)", S, pad_rows);
      for (int i = 0; i < p.count; ++i)
        if (p.tokens[i] < 0 || p.tokens[i] >= vocab_size)
          return fail(TGE_RT_VALUE_ERROR, "request %lld: token %d is outside the vocabulary of %d", (long long)p.request,
                      p.tokens[i], vocab_size);
      for (int i = 0; i < p.want_count; ++i)
        if (p.wants[i] < 0 || p.wants[i] >= p.count)
          return fail(TGE_RT_VALUE_ERROR, "request %lld: wanted place %d is outside its %d tokens", (long long)p.request,
                      p.wants[i], p.count);
    }
  }
  if (reserve) {
    // Everything is counted before anything is taken, so a step either runs whole or changes nothing:
    // state slots for the requests that start here, and per group the pages all portions lack in sum.
    const int G = (int)cache->groups.size();
    std::vector<int> lacking(G, 0);
    int starting = 0;
    for (const PortionView& p : portions) {
      const TgeRtCache::Live* live = cache->find(p.request);
      const int total = (live ? live->computed : 0) + p.count;
      if (total > max_model_len)
        return fail(TGE_RT_VALUE_ERROR, "request %lld: %d tokens exceed the context of %d", (long long)p.request, total,
                    max_model_len);
      if (!live) ++starting;
      for (int g = 0; g < G; ++g) lacking[g] += cache->missing(cache->groups[g], p.request, total);
    }
    if (starting > (int)cache->free_slots.size())
      return fail(TGE_RT_EXHAUSTED, "cache manager: the step starts %d requests, %d state slots are free", starting,
                  (int)cache->free_slots.size());
    for (int g = 0; g < G; ++g)
      if (lacking[g] > cache->groups[g].pool->free_count())
        return fail(TGE_RT_EXHAUSTED, "cache manager: the step needs %d more pages of group %d, %d are free", lacking[g], g,
                    cache->groups[g].pool->free_count());
    for (const PortionView& p : portions) {
      if (!cache->find(p.request))
        if (int rc = cache->admit(p.request); rc < 0) return rc;
      if (int rc = cache->grow(p.request, cache->find(p.request)->computed + p.count); rc < 0) return rc;
    }
  }
  TgeRtStepLayout L{};
  int T = 0, R = 0, max_q = 0, max_ctx = 0;
  for (const PortionView& p : portions) {
    const TgeRtCache::Live* live = cache->find(p.request);
    if (!live) return fail(TGE_RT_PAGE_ERROR, "step: request %lld is not live", (long long)p.request);
    T += p.count;
    R += p.want_count;
    max_q = std::max(max_q, p.count);
    max_ctx = std::max(max_ctx, live->computed + p.count);
  }
  // A step padded to more portions than it has gets idle ones behind the real ones: one token (id 0) at
  // position 0 of the group's scratch page, its state in the scratch slot.  They read and write nothing
  // that a request holds, and nobody asks for their logits.
  const int idle = std::max(0, pad_rows - S);
  const int real_tokens = T;
  S += idle;
  T += idle;
  const int G = (int)cache->groups.size();
  int cursor = 0;
  auto section = [&](int count) { const int at = cursor; cursor += count; return at; };
  L.num_tokens = T; L.num_seqs = S; L.num_rows = R; L.max_q_len = max_q; L.max_ctx_len = max_ctx;
  L.token_ids = section(T); L.positions = section(T); L.seq_of_token = section(T); L.q_start = section(S + 1);
  L.start_pos = section(S); L.ctx_len = section(S); L.slots = section(S); L.logit_rows = section(std::max(R, pad_rows));
  for (int g = 0; g < G; ++g) {
    int width = fixed_width;
    if (width <= 0) {
      width = 1;
      for (const PortionView& p : portions) {
        auto it = cache->groups[g].tables.find(p.request);
        if (it != cache->groups[g].tables.end()) width = std::max(width, (int)it->second.size());
      }
    }
    L.width[g] = width;
    L.table[g] = section(S * width);
  }
  L.total_ints = cursor;
  if (cursor > capacity) return fail(TGE_RT_VALUE_ERROR, "step: %d index values do not fit a buffer of %lld", cursor, capacity);
  int token = 0, row = 0;
  out[L.q_start] = 0;
  for (int i = R; i < pad_rows; ++i) out[L.logit_rows + i] = 0;
  for (int s = 0; s < S - idle; ++s) {
    const PortionView& p = portions[s];
    const TgeRtCache::Live* live = cache->find(p.request);
    const int start = live->computed;
    for (int i = 0; i < p.count; ++i, ++token) {
      out[L.token_ids + token] = p.tokens[i];
      out[L.positions + token] = start + i;
      out[L.seq_of_token + token] = s;
    }
    for (int i = 0; i < p.want_count; ++i) out[L.logit_rows + row++] = token - p.count + p.wants[i];
    out[L.q_start + s + 1] = token;
    out[L.start_pos + s] = start;
    out[L.ctx_len + s] = start + p.count;
    out[L.slots + s] = live->slot;
    for (int g = 0; g < G; ++g) {
      int* dst = out + L.table[g] + (size_t)s * L.width[g];
      auto it = cache->groups[g].tables.find(p.request);
      const int have = it == cache->groups[g].tables.end() ? 0 : (int)it->second.size();
      if (have > L.width[g])
        return fail(TGE_RT_VALUE_ERROR, "step: request %lld holds %d pages, the table is %d wide", (long long)p.request, have,
                    L.width[g]);
      for (int i = 0; i < have; ++i) dst[i] = it->second[i];
      for (int i = have; i < L.width[g]; ++i) dst[i] = NO_PAGE;
    }
  }
  for (int s = S - idle, token = real_tokens; s < S; ++s, ++token) {
    out[L.token_ids + token] = 0;
    out[L.positions + token] = 0;
    out[L.seq_of_token + token] = s;
    out[L.q_start + s + 1] = token + 1;
    out[L.start_pos + s] = 0;
    out[L.ctx_len + s] = 1;
    out[L.slots + s] = cache->max_requests;
    for (int g = 0; g < G; ++g) {
      int* dst = out + L.table[g] + (size_t)s * L.width[g];
      dst[0] = cache->groups[g].pool->capacity();
      for (int i = 1; i < L.width[g]; ++i) dst[i] = NO_PAGE;
    }
  }
  if (layout) *layout = L;
  return cursor;
}

}  // namespace

// ------------------------------------------------------------------------------------------------------
struct TgeRtScheduler {
  enum State { WAITING = 0, RUNNING = 1, FINISHED = 2 };
  struct Request {
    int64_t id;
    std::vector<int> tokens;       // prompt, then what was generated
    int prompt_len, max_new_tokens;
    int state = WAITING, computed = 0, preemptions = 0, reason = -1;
    int generated() const { return (int)tokens.size() - prompt_len; }
  };
  struct Item {
    Request* request;
    int start, count;
    bool samples;
  };
  TgeRtCache* cache;
  int max_batch_tokens, max_requests, max_model_len, chunk;
  std::unordered_set<int> end_tokens;
  std::unordered_map<int64_t, std::unique_ptr<Request>> requests;
  std::deque<Request*> waiting;
  std::vector<Request*> running;           // in admission order
  std::vector<Item> plan;
  std::vector<int64_t> preempted;
  std::vector<int> want_last;              // scratch for packing
  long long counters[5] = {0, 0, 0, 0, 0};

  int planned_tokens() const {
    int total = 0;
    for (const Item& item : plan) total += item.count;
    return total;
  }
  int portion_size(const Request* r, int budget) const {
    int count = std::min((int)r->tokens.size() - r->computed, budget);
    if (chunk > 0) count = std::min(count, chunk);
    return count;
  }
  void preempt(Request* victim) {
    cache->free_request(victim->id);
    running.erase(std::find(running.begin(), running.end(), victim));
    victim->state = WAITING;
    victim->computed = 0;
    ++victim->preemptions;
    waiting.push_front(victim);
    preempted.push_back(victim->id);
    plan.erase(std::remove_if(plan.begin(), plan.end(), [&](const Item& item) { return item.request == victim; }), plan.end());
    ++counters[2];
  }
  int schedule() {
    plan.clear();
    preempted.clear();
    int budget = max_batch_tokens;
    // running requests first, in admission order; each reserves its pages as it is planned
    size_t index = 0;
    while (index < running.size()) {
      Request* r = running[index];
      int count = portion_size(r, budget);
      if (count <= 0) { ++index; continue; }
      while (!cache->can_grow(r->id, r->computed + count)) {
        Request* victim = running.back();
        preempt(victim);
        budget = max_batch_tokens - planned_tokens();     // the victim's planned tokens go back to the budget
        if (victim == r) break;
      }
      if (r->state != RUNNING) continue;                   // it preempted itself; same index, shorter list
      count = portion_size(r, budget);
      if (int rc = cache->grow(r->id, r->computed + count)) return rc;
      plan.push_back(Item{r, r->computed, count, r->computed + count == (int)r->tokens.size()});
      budget -= count;
      ++index;
    }
    // then new requests in arrival order, unless this step had to preempt (or preemption left nothing
    // to run: then the head of the queue starts over at once)
    while (!waiting.empty() && (preempted.empty() || plan.empty()) && budget > 0 && (int)running.size() < max_requests &&
           !cache->free_slots.empty()) {
      Request* r = waiting.front();
      const int count = portion_size(r, budget);
      const int pages = cache->pages_for(count);
      bool fits = true;
      for (const auto& group : cache->groups) fits = fits && pages <= group.pool->free_count();
      if (!fits) break;
      waiting.pop_front();
      if (int rc = cache->admit(r->id); rc < 0) return rc;
      if (int rc = cache->grow(r->id, count)) return rc;
      r->state = RUNNING;
      r->computed = 0;
      running.push_back(r);
      ++counters[3];
      plan.push_back(Item{r, 0, count, count == (int)r->tokens.size()});
      budget -= count;
    }
    if (plan.empty() && (!waiting.empty() || !running.empty()))
      return fail(TGE_RT_STUCK, "scheduler: nothing can run although requests are waiting "
                                "(the page pool is too small for the oldest request's next portion)");
    ++counters[0];
    counters[1] += planned_tokens();
    return (int)plan.size();
  }
  int update(const int* sampled, int count, int64_t* finished, int* reasons, int capacity) {
    int cursor = 0, done = 0;
    int sampling = 0;
    for (const Item& item : plan) sampling += item.samples ? 1 : 0;
    if (sampling != count) return fail(TGE_RT_VALUE_ERROR, "scheduler: %d sampled tokens for %d sampling portions", count, sampling);
    for (const Item& item : plan) {
      Request* r = item.request;
      r->computed = item.start + item.count;
      if (int rc = cache->set_computed(r->id, r->computed)) return rc;
      if (!item.samples) continue;
      const int token = sampled[cursor++];
      r->tokens.push_back(token);
      int reason = -1;
      if (end_tokens.count(token)) reason = 0;
      else if (r->generated() >= r->max_new_tokens) reason = 1;
      else if ((int)r->tokens.size() >= max_model_len) reason = 2;
      if (reason >= 0) {
        r->state = FINISHED;
        r->reason = reason;
        cache->free_request(r->id);
        running.erase(std::find(running.begin(), running.end(), r));
        ++counters[4];
        if (done < capacity) {
          finished[done] = r->id;
          reasons[done] = reason;
        }
        ++done;
      }
    }
    plan.clear();
    return done;
  }
};

// ------------------------------------------------------------------------------------------------------
extern "C" {

const char* tge_rt_last_error(void) { return g_error.c_str(); }

TgeRtPool* tge_rt_pool_create(int num_pages) {
  if (num_pages <= 0) {
    fail(TGE_RT_VALUE_ERROR, "page pool: the number of pages must be positive");
    return nullptr;
  }
  return new TgeRtPool(num_pages);
}
void tge_rt_pool_destroy(TgeRtPool* pool) { delete pool; }
int tge_rt_pool_capacity(const TgeRtPool* pool) { return pool->capacity(); }
int tge_rt_pool_free_count(const TgeRtPool* pool) { return pool->free_count(); }
int tge_rt_pool_allocate(TgeRtPool* pool) { return pool->allocate(); }
int tge_rt_pool_share(TgeRtPool* pool, int page) { return pool->share(page); }
int tge_rt_pool_release(TgeRtPool* pool, int page) { return pool->release(page); }
int tge_rt_pool_refcount(const TgeRtPool* pool, int page) {
  if (page < 0 || page >= pool->capacity()) return fail(TGE_RT_PAGE_ERROR, "page pool: page id %d out of range", page);
  return pool->refcount[page];
}
int tge_rt_pool_check(const TgeRtPool* pool) { return pool->check(); }

TgeRtCache* tge_rt_cache_create(int page_size, int max_requests) {
  if (page_size <= 0 || max_requests <= 0) {
    fail(TGE_RT_VALUE_ERROR, "cache manager: page_size and max_requests must be positive");
    return nullptr;
  }
  return new TgeRtCache(page_size, max_requests);
}
void tge_rt_cache_destroy(TgeRtCache* cache) { delete cache; }
int tge_rt_cache_add_group(TgeRtCache* cache, int window) {
  if (cache->groups.size() >= 8) return fail(TGE_RT_VALUE_ERROR, "cache manager: at most 8 groups");
  TgeRtCache::Group group;
  group.window = window;
  group.pool.reset(new TgeRtPool(1));
  cache->groups.push_back(std::move(group));
  return (int)cache->groups.size() - 1;
}
int tge_rt_cache_set_pool_size(TgeRtCache* cache, int group, int num_pages) {
  if (group < 0 || group >= (int)cache->groups.size()) return fail(TGE_RT_VALUE_ERROR, "cache manager: no group %d", group);
  if (num_pages <= 0) return fail(TGE_RT_VALUE_ERROR, "page pool: the number of pages must be positive");
  if (!cache->live.empty()) return fail(TGE_RT_PAGE_ERROR, "cache manager: pools cannot be resized while requests are live");
  cache->groups[group].pool.reset(new TgeRtPool(num_pages));
  return 0;
}
TgeRtPool* tge_rt_cache_pool(TgeRtCache* cache, int group) {
  if (group < 0 || group >= (int)cache->groups.size()) return nullptr;
  return cache->groups[group].pool.get();
}
int tge_rt_cache_groups(const TgeRtCache* cache) { return (int)cache->groups.size(); }
int tge_rt_cache_free_slots(const TgeRtCache* cache) { return (int)cache->free_slots.size(); }
int tge_rt_cache_live_count(const TgeRtCache* cache) { return (int)cache->live.size(); }
int tge_rt_cache_live_requests(const TgeRtCache* cache, int64_t* out, int capacity) {
  std::vector<std::pair<long long, int64_t>> ordered;
  for (const auto& entry : cache->live) ordered.emplace_back(entry.second.order, entry.first);
  std::sort(ordered.begin(), ordered.end());
  for (int i = 0; i < (int)ordered.size() && i < capacity; ++i) out[i] = ordered[i].second;
  return (int)ordered.size();
}
int tge_rt_cache_is_live(const TgeRtCache* cache, int64_t request) { return cache->find(request) ? 1 : 0; }

#define TGE_RT_LIVE_OR_FAIL(var)                                                                                   \
  const TgeRtCache::Live* var = cache->find(request);                                                              \
  if (!var) return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is not live", (long long)request)

int tge_rt_cache_slot_of(const TgeRtCache* cache, int64_t request) { TGE_RT_LIVE_OR_FAIL(live); return live->slot; }
int tge_rt_cache_tokens_of(const TgeRtCache* cache, int64_t request) { TGE_RT_LIVE_OR_FAIL(live); return live->tokens; }
int tge_rt_cache_computed(const TgeRtCache* cache, int64_t request) { TGE_RT_LIVE_OR_FAIL(live); return live->computed; }
int tge_rt_cache_admit(TgeRtCache* cache, int64_t request) { return cache->admit(request); }
int tge_rt_cache_can_grow(const TgeRtCache* cache, int64_t request, int total_tokens) {
  return cache->can_grow(request, total_tokens) ? 1 : 0;
}
int tge_rt_cache_fits_empty_pool(const TgeRtCache* cache, int total_tokens) { return cache->fits_empty_pool(total_tokens) ? 1 : 0; }
int tge_rt_cache_pages_missing(const TgeRtCache* cache, int64_t request, int total_tokens, int* per_group) {
  for (size_t g = 0; g < cache->groups.size(); ++g) per_group[g] = cache->missing(cache->groups[g], request, total_tokens);
  return (int)cache->groups.size();
}
int tge_rt_cache_grow(TgeRtCache* cache, int64_t request, int total_tokens) { return cache->grow(request, total_tokens); }
int tge_rt_cache_set_computed(TgeRtCache* cache, int64_t request, int tokens) { return cache->set_computed(request, tokens); }
int tge_rt_cache_release_behind_window(TgeRtCache* cache, int64_t request, int computed_tokens) {
  TGE_RT_LIVE_OR_FAIL(live);
  (void)live;
  return cache->release_behind_window(request, computed_tokens);
}
int tge_rt_cache_free(TgeRtCache* cache, int64_t request) { return cache->free_request(request); }
int tge_rt_cache_table_length(const TgeRtCache* cache, int group, int64_t request) {
  if (group < 0 || group >= (int)cache->groups.size()) return fail(TGE_RT_VALUE_ERROR, "cache manager: no group %d", group);
  auto it = cache->groups[group].tables.find(request);
  if (it == cache->groups[group].tables.end())
    return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is not live", (long long)request);
  return (int)it->second.size();
}
int tge_rt_cache_table(const TgeRtCache* cache, int group, int64_t request, int* out, int capacity) {
  const int length = tge_rt_cache_table_length(cache, group, request);
  if (length < 0) return length;
  const std::vector<int>& table = cache->groups[group].tables.find(request)->second;
  for (int i = 0; i < length && i < capacity; ++i) out[i] = table[i];
  return length;
}
int tge_rt_cache_fill_block_table(const TgeRtCache* cache, int group, const int64_t* requests, int count, int* out,
                                  int width) {
  if (group < 0 || group >= (int)cache->groups.size()) return fail(TGE_RT_VALUE_ERROR, "cache manager: no group %d", group);
  for (int row = 0; row < count; ++row) {
    auto it = cache->groups[group].tables.find(requests[row]);
    if (it == cache->groups[group].tables.end())
      return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is not live", (long long)requests[row]);
    const int have = (int)it->second.size();
    if (have > width) return fail(TGE_RT_VALUE_ERROR, "cache manager: a table of %d pages does not fit a width of %d", have, width);
    int* dst = out + (size_t)row * width;
    for (int i = 0; i < have; ++i) dst[i] = it->second[i];
    for (int i = have; i < width; ++i) dst[i] = NO_PAGE;
  }
  return 0;
}
int tge_rt_cache_check(const TgeRtCache* cache) { return cache->check(); }
int tge_rt_cache_max_context(const TgeRtCache* cache, const int64_t* requests, const int* add, int count) {
  int most = 0;
  for (int i = 0; i < count; ++i) {
    const TgeRtCache::Live* live = cache->find(requests[i]);
    most = std::max(most, (live ? live->computed : 0) + add[i]);
  }
  return most;
}
int tge_rt_cache_advance(TgeRtCache* cache, const int64_t* requests, const int* add, int count) {
  for (int i = 0; i < count; ++i) {
    const TgeRtCache::Live* live = cache->find(requests[i]);
    if (!live) return fail(TGE_RT_PAGE_ERROR, "cache manager: request %lld is not live", (long long)requests[i]);
    if (int rc = cache->set_computed(requests[i], live->computed + add[i])) return rc;
  }
  return 0;
}

int tge_rt_step_pack(TgeRtCache* cache, int count, const int64_t* requests, const int* const* tokens,
                     const int* token_counts, const int* const* wants, const int* want_counts, int vocab_size,
                     int max_model_len, int fixed_width, int pad_rows, int* out, long long capacity,
                     TgeRtStepLayout* layout) {
  std::vector<PortionView> portions(count > 0 ? count : 0);
  for (int i = 0; i < count; ++i)
    portions[i] = PortionView{requests[i], tokens[i], token_counts[i], wants ? wants[i] : nullptr, want_counts ? want_counts[i] : 0};
  return pack_step(cache, portions, vocab_size, max_model_len, fixed_width, pad_rows, true, out, capacity, layout);
}

TgeRtScheduler* tge_rt_sched_create(TgeRtCache* cache, int max_batch_tokens, int max_requests, int max_model_len,
                                    int chunk, const int* end_tokens, int num_end_tokens) {
  if (max_batch_tokens <= 0 || max_requests <= 0 || max_model_len <= 0) {
    fail(TGE_RT_VALUE_ERROR, "scheduler: limits must be positive");
    return nullptr;
  }
  if (chunk < 0) {
    fail(TGE_RT_VALUE_ERROR, "scheduler: chunk must be positive");
    return nullptr;
  }
  TgeRtScheduler* s = new TgeRtScheduler();
  s->cache = cache;
  s->max_batch_tokens = max_batch_tokens;
  s->max_requests = std::min(max_requests, cache->max_requests);
  s->max_model_len = max_model_len;
  s->chunk = chunk;
  for (int i = 0; i < num_end_tokens; ++i) s->end_tokens.insert(end_tokens[i]);
  return s;
}
void tge_rt_sched_destroy(TgeRtScheduler* s) { delete s; }

int tge_rt_sched_add(TgeRtScheduler* s, int64_t request, const int* prompt, int prompt_len, int max_new_tokens) {
  if (prompt_len <= 0) return fail(TGE_RT_VALUE_ERROR, "request %lld: at least one prompt token is required", (long long)request);
  if (max_new_tokens <= 0) return fail(TGE_RT_VALUE_ERROR, "request %lld: max_new_tokens must be positive", (long long)request);
  if (prompt_len + 1 > s->max_model_len)
    return fail(TGE_RT_VALUE_ERROR, "request %lld: %d prompt tokens leave no room in a context of %d", (long long)request,
                prompt_len, s->max_model_len);
  // the last generated token is never fed back, so a request caches at most prompt + new - 1 tokens
  const int most = std::min(prompt_len + max_new_tokens - 1, s->max_model_len);
  if (!s->cache->fits_empty_pool(most))
    return fail(TGE_RT_VALUE_ERROR, "request %lld: %d tokens do not fit the page pool even when it is empty", (long long)request, most);
  auto it = s->requests.find(request);
  if (it != s->requests.end()) {
    if (it->second->state != TgeRtScheduler::FINISHED)
      return fail(TGE_RT_VALUE_ERROR, "request id %lld is already in use", (long long)request);
    s->requests.erase(it);
  }
  std::unique_ptr<TgeRtScheduler::Request> r(new TgeRtScheduler::Request());
  r->id = request;
  r->tokens.assign(prompt, prompt + prompt_len);
  r->prompt_len = prompt_len;
  r->max_new_tokens = max_new_tokens;
  s->waiting.push_back(r.get());
  s->requests[request] = std::move(r);
  return 0;
}
int tge_rt_sched_has_work(const TgeRtScheduler* s) { return (!s->waiting.empty() || !s->running.empty()) ? 1 : 0; }
int tge_rt_sched_waiting(const TgeRtScheduler* s, int64_t* out, int capacity) {
  int i = 0;
  for (const auto* r : s->waiting) {
    if (i < capacity) out[i] = r->id;
    ++i;
  }
  return i;
}
int tge_rt_sched_running(const TgeRtScheduler* s, int64_t* out, int capacity) {
  int i = 0;
  for (const auto* r : s->running) {
    if (i < capacity) out[i] = r->id;
    ++i;
  }
  return i;
}
int tge_rt_sched_schedule(TgeRtScheduler* s) { return s->schedule(); }
int tge_rt_sched_plan(const TgeRtScheduler* s, int64_t* requests, int* starts, int* counts, int* samples, int capacity) {
  const int n = (int)s->plan.size();
  for (int i = 0; i < n && i < capacity; ++i) {
    requests[i] = s->plan[i].request->id;
    starts[i] = s->plan[i].start;
    counts[i] = s->plan[i].count;
    samples[i] = s->plan[i].samples ? 1 : 0;
  }
  return n;
}
int tge_rt_sched_plan_preempted(const TgeRtScheduler* s, int64_t* out, int capacity) {
  const int n = (int)s->preempted.size();
  for (int i = 0; i < n && i < capacity; ++i) out[i] = s->preempted[i];
  return n;
}
int tge_rt_sched_pack(TgeRtScheduler* s, int vocab_size, int fixed_width, int pad_rows, int* out, long long capacity,
                      TgeRtStepLayout* layout) {
  std::vector<PortionView> portions(s->plan.size());
  s->want_last.resize(s->plan.size());
  for (size_t i = 0; i < s->plan.size(); ++i) {
    const TgeRtScheduler::Item& item = s->plan[i];
    s->want_last[i] = item.count - 1;
    portions[i] = PortionView{item.request->id, item.request->tokens.data() + item.start, item.count, &s->want_last[i],
                              item.samples ? 1 : 0};
  }
  // pages were reserved when the plan was made
  return pack_step(s->cache, portions, vocab_size, s->max_model_len, fixed_width, pad_rows, false, out, capacity, layout);
}
int tge_rt_sched_update(TgeRtScheduler* s, const int* sampled, int count, int64_t* finished, int* reasons, int capacity) {
  return s->update(sampled, count, finished, reasons, capacity);
}
int tge_rt_sched_request_info(const TgeRtScheduler* s, int64_t request, int* state, int* computed, int* preemptions,
                              int* num_tokens) {
  auto it = s->requests.find(request);
  if (it == s->requests.end()) return fail(TGE_RT_VALUE_ERROR, "scheduler: no request %lld", (long long)request);
  *state = it->second->state;
  *computed = it->second->computed;
  *preemptions = it->second->preemptions;
  *num_tokens = (int)it->second->tokens.size();
  return 0;
}
int tge_rt_sched_tokens(const TgeRtScheduler* s, int64_t request, int start, int count, int* out) {
  auto it = s->requests.find(request);
  if (it == s->requests.end()) return fail(TGE_RT_VALUE_ERROR, "scheduler: no request %lld", (long long)request);
  const std::vector<int>& tokens = it->second->tokens;
  if (start < 0 || count < 0 || start + count > (int)tokens.size())
    return fail(TGE_RT_VALUE_ERROR, "scheduler: tokens [%d, %d) of request %lld do not exist", start, start + count, (long long)request);
  std::copy(tokens.begin() + start, tokens.begin() + start + count, out);
  return count;
}
int tge_rt_sched_forget(TgeRtScheduler* s, int64_t request) {
  auto it = s->requests.find(request);
  if (it == s->requests.end()) return 0;
  if (it->second->state != TgeRtScheduler::FINISHED)
    return fail(TGE_RT_VALUE_ERROR, "scheduler: request %lld is still in use", (long long)request);
  s->requests.erase(it);
  return 0;
}
long long tge_rt_sched_counter(const TgeRtScheduler* s, int which) { return which >= 0 && which < 5 ? s->counters[which] : -1; }


// ------------------------------------------------------------------------------------------------------
// random weights on the host
namespace {

inline uint16_t bf16_round_nearest_even(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu)) return (uint16_t)((bits >> 16) | 0x0040u);   // NaN
  bits += 0x7FFFu + ((bits >> 16) & 1u);
  return (uint16_t)(bits >> 16);
}

void random_fill_range(void* out, int is_bf16, long long begin, long long end, long long first, uint64_t key, int kind,
                       float scale, int base, uint32_t span) {
  for (long long i = begin; i < end; ++i) {
    const uint64_t index = (uint64_t)(first + i);
    // one int-to-float conversion and one multiplication, each rounded once: nothing for a compiler to contract
    const float value = kind == TGE_RANDOM_NORMAL ? (float)tge_rw_normal_int(key, index)
                                                     : (float)tge_rw_uniform_int(key, index, base, span);
    const float result = value * (kind == TGE_RANDOM_NORMAL ? scale : 5.9604644775390625e-08f);
    if (is_bf16)
      static_cast<uint16_t*>(out)[i] = bf16_round_nearest_even(result);
    else
      static_cast<float*>(out)[i] = result;
  }
}

}  // namespace

int tge_rt_random_fill(void* out, int is_bf16, long long count, long long first, unsigned long long key, int kind,
                       float scale, int base, unsigned int span, int threads) {
  if (count < 0 || first < 0) return fail(TGE_RT_VALUE_ERROR, "random_fill: bad range first=%lld count=%lld", first, count);
  if (kind != TGE_RANDOM_NORMAL && kind != TGE_RANDOM_UNIFORM) return fail(TGE_RT_VALUE_ERROR, "random_fill: unknown kind %d", kind);
  if (out == nullptr && count > 0) return fail(TGE_RT_VALUE_ERROR, "random_fill: no output buffer");
  const long long grain = 1 << 16;
  int workers = (int)std::min<long long>(std::max(threads, 1), (count + grain - 1) / grain);
  if (workers <= 1) {
    random_fill_range(out, is_bf16, 0, count, first, key, kind, scale, base, span);
    return 0;
  }
  std::vector<std::thread> pool;
  const long long share = (count + workers - 1) / workers;
  for (int w = 0; w < workers; ++w) {
    const long long begin = w * share, end = std::min(count, begin + share);
    if (begin >= end) break;
    pool.emplace_back(random_fill_range, out, is_bf16, begin, end, first, (uint64_t)key, kind, scale, base, (uint32_t)span);
  }
  for (std::thread& t : pool) t.join();
  return 0;
}

}  // extern "C"
