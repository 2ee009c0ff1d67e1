// Host runtime of the engine, in C++: page pools, the cache manager's bookkeeping, the scheduler, and
// the packing of a step's index arrays.  No CUDA in here; the Python classes of the same names
// (cache.pages.PagePool, cache.manager.CacheManager, engine.scheduler.Scheduler) are thin views of
// these objects, and the tests of those classes are the tests of this code.
//
// Conventions: a request is a signed 64-bit handle chosen by the caller.  Functions return 0 or a
// non-negative count on success and a negative TgeRtCode on failure; tge_rt_last_error() then holds the
// message (per thread).  Objects are not thread-safe: one engine, one thread.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum TgeRtCode {
  TGE_RT_OK = 0,
  TGE_RT_EXHAUSTED = -1,   // no free page or slot: the caller may preempt or wait
  TGE_RT_PAGE_ERROR = -2,  // a page, slot or request was used in a way its state does not allow
  TGE_RT_VALUE_ERROR = -3, // an argument is out of range
  TGE_RT_STUCK = -4        // the scheduler has work but nothing can run
};

const char* tge_rt_last_error(void);

// ---- page pool: reference counts and a LIFO free list ---------------------------------------------
typedef struct TgeRtPool TgeRtPool;
TgeRtPool* tge_rt_pool_create(int num_pages);
void tge_rt_pool_destroy(TgeRtPool* pool);
int tge_rt_pool_capacity(const TgeRtPool* pool);
int tge_rt_pool_free_count(const TgeRtPool* pool);
int tge_rt_pool_allocate(TgeRtPool* pool);                 // page id
int tge_rt_pool_share(TgeRtPool* pool, int page);
int tge_rt_pool_release(TgeRtPool* pool, int page);        // 1 when the page went back to the free list
int tge_rt_pool_refcount(const TgeRtPool* pool, int page);
int tge_rt_pool_check(const TgeRtPool* pool);

// ---- cache bookkeeping: groups of layers, block tables, state slots ----------------------------------
typedef struct TgeRtCache TgeRtCache;
TgeRtCache* tge_rt_cache_create(int page_size, int max_requests);
void tge_rt_cache_destroy(TgeRtCache* cache);
int tge_rt_cache_add_group(TgeRtCache* cache, int window);            // window < 0: every key is kept; returns the group's index
int tge_rt_cache_set_pool_size(TgeRtCache* cache, int group, int num_pages);
TgeRtPool* tge_rt_cache_pool(TgeRtCache* cache, int group);          // owned by the cache
int tge_rt_cache_groups(const TgeRtCache* cache);
int tge_rt_cache_free_slots(const TgeRtCache* cache);
int tge_rt_cache_live_count(const TgeRtCache* cache);
int tge_rt_cache_live_requests(const TgeRtCache* cache, int64_t* out, int capacity);   // in admission order
int tge_rt_cache_is_live(const TgeRtCache* cache, int64_t request);
int tge_rt_cache_slot_of(const TgeRtCache* cache, int64_t request);
int tge_rt_cache_tokens_of(const TgeRtCache* cache, int64_t request);
int tge_rt_cache_computed(const TgeRtCache* cache, int64_t request);
int tge_rt_cache_admit(TgeRtCache* cache, int64_t request);          // slot
int tge_rt_cache_can_grow(const TgeRtCache* cache, int64_t request, int total_tokens);   // 0 or 1
int tge_rt_cache_fits_empty_pool(const TgeRtCache* cache, int total_tokens);             // 0 or 1
int tge_rt_cache_pages_missing(const TgeRtCache* cache, int64_t request, int total_tokens, int* per_group);
int tge_rt_cache_grow(TgeRtCache* cache, int64_t request, int total_tokens);             // all or nothing
int tge_rt_cache_set_computed(TgeRtCache* cache, int64_t request, int tokens);
int tge_rt_cache_release_behind_window(TgeRtCache* cache, int64_t request, int computed_tokens);   // pages given back
int tge_rt_cache_free(TgeRtCache* cache, int64_t request);
int tge_rt_cache_table_length(const TgeRtCache* cache, int group, int64_t request);
int tge_rt_cache_table(const TgeRtCache* cache, int group, int64_t request, int* out, int capacity);
// rows of page ids, -1 beyond each row's end; out is int32 [count, width]
int tge_rt_cache_fill_block_table(const TgeRtCache* cache, int group, const int64_t* requests, int count, int* out,
                                  int width);
int tge_rt_cache_check(const TgeRtCache* cache);
// Largest (tokens computed + tokens to add) over the requests; one not yet admitted counts from zero.
int tge_rt_cache_max_context(const TgeRtCache* cache, const int64_t* requests, const int* add, int count);
// Records for every request that `add[i]` more tokens are computed (as set_computed does, windows included).
int tge_rt_cache_advance(TgeRtCache* cache, const int64_t* requests, const int* add, int count);

// ---- a step's index arrays ------------------------------------------------------------------------------
// Sections of the packed int32 buffer, in this order; TgeRtStepLayout gives where each begins.
//   token_ids[T] positions[T] seq_of_token[T] q_start[S+1] start_pos[S] ctx_len[S] slots[S] logit_rows[R]
//   then one block table [S, width_g] per group
typedef struct TgeRtStepLayout {
  int num_tokens, num_seqs, num_rows, max_q_len, max_ctx_len, total_ints;
  int token_ids, positions, seq_of_token, q_start, start_pos, ctx_len, slots, logit_rows;
  int table[8], width[8];
} TgeRtStepLayout;

// Reserves what the step needs (admits unknown requests, grows pages; all or nothing) and packs it.
// tokens[i] / wants[i] point at the i-th portion's token ids and wanted places.  fixed_width > 0 pads
// every block table to that width; pad_rows > 0 pads a step of single tokens to that many portions and
// the logit_rows section to that many entries (a captured graph's geometry): the idle portions behind
// the real ones are one token at position 0 of each group's scratch page (id = the pool's capacity)
// with the scratch state slot (id = max_requests).  Else the widest row and the wanted places decide.
// Progress is not recorded: call tge_rt_cache_advance after the step ran.
int tge_rt_step_pack(TgeRtCache* cache, int count, const int64_t* requests, const int* const* tokens,
                     const int* token_counts, const int* const* wants, const int* want_counts, int vocab_size,
                     int max_model_len, int fixed_width, int pad_rows, int* out, long long capacity,
                     TgeRtStepLayout* layout);

// ---- scheduler -------------------------------------------------------------------------------------------
typedef struct TgeRtScheduler TgeRtScheduler;
TgeRtScheduler* tge_rt_sched_create(TgeRtCache* cache, int max_batch_tokens, int max_requests, int max_model_len,
                                    int chunk, const int* end_tokens, int num_end_tokens);
void tge_rt_sched_destroy(TgeRtScheduler* s);
int tge_rt_sched_add(TgeRtScheduler* s, int64_t request, const int* prompt, int prompt_len, int max_new_tokens);
int tge_rt_sched_has_work(const TgeRtScheduler* s);
int tge_rt_sched_waiting(const TgeRtScheduler* s, int64_t* out, int capacity);
int tge_rt_sched_running(const TgeRtScheduler* s, int64_t* out, int capacity);
// Plans the next step; returns the number of portions.  The plan stays valid until the next schedule().
int tge_rt_sched_schedule(TgeRtScheduler* s);
int tge_rt_sched_plan(const TgeRtScheduler* s, int64_t* requests, int* starts, int* counts, int* samples, int capacity);
int tge_rt_sched_plan_preempted(const TgeRtScheduler* s, int64_t* out, int capacity);
// Packs the current plan (tokens come from the scheduler's own copies); the wanted place of a portion
// that samples is its last token.
int tge_rt_sched_pack(TgeRtScheduler* s, int vocab_size, int fixed_width, int pad_rows, int* out, long long capacity,
                      TgeRtStepLayout* layout);
// Records the step: one sampled token per sampling portion, in plan order.  Returns how many requests
// finished; their handles and reasons (0 end token, 1 length, 2 context) go to the out arrays.
int tge_rt_sched_update(TgeRtScheduler* s, const int* sampled, int count, int64_t* finished, int* reasons, int capacity);
int tge_rt_sched_request_info(const TgeRtScheduler* s, int64_t request, int* state, int* computed, int* preemptions,
                              int* num_tokens);
int tge_rt_sched_tokens(const TgeRtScheduler* s, int64_t request, int start, int count, int* out);
int tge_rt_sched_forget(TgeRtScheduler* s, int64_t request);       // drops a finished request's record
long long tge_rt_sched_counter(const TgeRtScheduler* s, int which);  // 0 steps 1 tokens 2 preemptions 3 admitted 4 finished

// ---- random weights on the host (random_weights.h: the same values as the device fill kernel) -------
// Fills out[0..count) with elements first..first+count of the tensor whose key is `key`, as float32
// (is_bf16 0) or bfloat16 rounded to nearest even (1).  kind 0: normal, value = float(int) * scale;
// kind 1: uniform, value = float(base + (u32 * span >> 32)) * 2^-24.  Uses up to `threads` threads.
int tge_rt_random_fill(void* out, int is_bf16, long long count, long long first, unsigned long long key, int kind,
                       float scale, int base, unsigned int span, int threads);

#ifdef __cplusplus
}
#endif
