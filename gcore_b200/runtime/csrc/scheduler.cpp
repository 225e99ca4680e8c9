// Host runtime of the rollout decoder: reference-counted paged-KV block manager and a continuous-batching
// scheduler with prefix sharing (n samples of one prompt share the prompt's blocks, copy-on-write for the last
// partial block) and recompute-style preemption when the cache runs out.
//
// This is the part of vLLM / SGLang the reference drives through its engine wrappers
// (gpatch_v4/generation_backend/infer_engine.py:291-343: generate, abort_all_requests, flush_cache, get_load).
// Plain C ABI, no CUDA: the Python engine copies the tables this produces into device tensors once per step.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

#define RT_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct Request {
  int64_t id;
  int prompt_len;
  int max_new;
  int generated = 0;
  int cached_tokens = 0;  // tokens whose KV is in the cache
  bool prefilled = false;
  bool finished = false;
  int64_t arrival;
  std::vector<int> blocks;
};

struct Scheduler {
  int num_blocks, block_size, max_running, max_prefill_tokens;
  std::vector<int> free_list;
  std::vector<int> refcnt;
  std::unordered_map<int64_t, Request> reqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;
  int64_t clock = 0;
  int64_t preemptions = 0;

  int blocks_needed(int tokens) const { return (tokens + block_size - 1) / block_size; }
  bool alloc(Request& r, int upto_tokens) {
    const int need = blocks_needed(upto_tokens) - static_cast<int>(r.blocks.size());
    if (need <= 0) return true;
    if (static_cast<int>(free_list.size()) < need) return false;
    for (int i = 0; i < need; ++i) {
      const int b = free_list.back();
      free_list.pop_back();
      refcnt[b] = 1;
      r.blocks.push_back(b);
    }
    return true;
  }
  void release(Request& r) {
    for (int b : r.blocks) {
      if (--refcnt[b] == 0) free_list.push_back(b);
    }
    r.blocks.clear();
    r.cached_tokens = 0;
  }
};

}  // namespace

RT_EXPORT void* gkrt_sched_create(int num_blocks, int block_size, int max_running, int max_prefill_tokens) {
  auto* s = new Scheduler();
  s->num_blocks = num_blocks;
  s->block_size = block_size;
  s->max_running = max_running;
  s->max_prefill_tokens = max_prefill_tokens;
  s->refcnt.assign(num_blocks, 0);
  s->free_list.reserve(num_blocks);
  for (int b = num_blocks - 1; b >= 0; --b) s->free_list.push_back(b);
  return s;
}

RT_EXPORT void gkrt_sched_destroy(void* h) { delete static_cast<Scheduler*>(h); }

RT_EXPORT int gkrt_sched_add(void* h, int64_t id, int prompt_len, int max_new) {
  auto* s = static_cast<Scheduler*>(h);
  if (s->reqs.count(id)) return -1;
  if (s->blocks_needed(prompt_len + max_new) > s->num_blocks) return -2;  // can never fit
  Request r;
  r.id = id;
  r.prompt_len = prompt_len;
  r.max_new = max_new;
  r.arrival = s->clock++;
  s->reqs.emplace(id, std::move(r));
  s->waiting.push_back(id);
  return 0;
}

// Child shares the parent's cached prompt blocks.  The parent must have been prefilled.  Full blocks are shared by
// reference; if the prompt ends inside a block the child gets a fresh block and (*copy_src, *copy_dst) tells the
// caller which block to copy on the device.  Returns 0, or -1 when no block is free / parent unknown.
RT_EXPORT int gkrt_sched_fork(void* h, int64_t parent, int64_t child, int max_new, int* copy_src, int* copy_dst) {
  auto* s = static_cast<Scheduler*>(h);
  *copy_src = *copy_dst = -1;
  auto it = s->reqs.find(parent);
  if (it == s->reqs.end() || !it->second.prefilled || s->reqs.count(child)) return -1;
  const Request& p = it->second;
  const int shared_tokens = p.prompt_len;
  const int full = shared_tokens / s->block_size;
  const bool partial = shared_tokens % s->block_size != 0;
  if (partial && s->free_list.empty()) return -1;
  Request c;
  c.id = child;
  c.prompt_len = p.prompt_len;
  c.max_new = max_new;
  c.prefilled = true;
  c.cached_tokens = shared_tokens;
  c.arrival = s->clock++;
  for (int i = 0; i < full; ++i) {
    c.blocks.push_back(p.blocks[i]);
    ++s->refcnt[p.blocks[i]];
  }
  if (partial) {
    const int b = s->free_list.back();
    s->free_list.pop_back();
    s->refcnt[b] = 1;
    c.blocks.push_back(b);
    *copy_src = p.blocks[full];
    *copy_dst = b;
  }
  s->running.push_back(child);
  s->reqs.emplace(child, std::move(c));
  return 0;
}

// One scheduling step.
//   prefill_ids[<=cap_prefill]: requests admitted this step (their whole prompt is prefilled at once)
//   decode_ids [<=cap_decode] : running requests that decode one token this step (a block for it is reserved)
// Running requests that cannot get a block are preempted youngest-first (blocks freed, back to the wait queue).
RT_EXPORT int gkrt_sched_step(void* h, int64_t* prefill_ids, int cap_prefill, int* n_prefill, int64_t* decode_ids,
                              int cap_decode, int* n_decode) {
  auto* s = static_cast<Scheduler*>(h);
  *n_prefill = *n_decode = 0;
  // 1. reserve the next token's slot for every running request, oldest first; preempt from the back on failure
  std::sort(s->running.begin(), s->running.end(),
            [&](int64_t a, int64_t b) { return s->reqs[a].arrival < s->reqs[b].arrival; });
  size_t i = 0;
  while (i < s->running.size()) {
    Request& r = s->reqs[s->running[i]];
    if (r.finished) { ++i; continue; }
    if (!s->alloc(r, r.cached_tokens + 1)) {
      // preempt the youngest running request (possibly r itself)
      const int64_t victim = s->running.back();
      Request& v = s->reqs[victim];
      s->release(v);
      v.prefilled = false;
      v.prompt_len += v.generated;  // recompute: generated tokens become part of the prompt
      v.max_new -= v.generated;
      v.generated = 0;
      s->running.pop_back();
      s->waiting.push_front(victim);
      ++s->preemptions;
      if (victim == r.id) break;
      continue;
    }
    ++i;
  }
  for (int64_t id : s->running) {
    if (*n_decode >= cap_decode) break;
    if (!s->reqs[id].finished) decode_ids[(*n_decode)++] = id;
  }
  // 2. admit waiting requests while blocks, slots and the prefill token budget allow
  int budget = s->max_prefill_tokens;
  while (!s->waiting.empty() && *n_prefill < cap_prefill &&
         static_cast<int>(s->running.size()) < s->max_running) {
    Request& r = s->reqs[s->waiting.front()];
    if (r.prompt_len > budget && *n_prefill > 0) break;
    // keep one block of head-room per running request so decode does not immediately preempt
    const int need = s->blocks_needed(r.prompt_len + 1);
    if (static_cast<int>(s->free_list.size()) < need + static_cast<int>(s->running.size())) break;
    s->alloc(r, r.prompt_len + 1);
    budget -= r.prompt_len;
    prefill_ids[(*n_prefill)++] = r.id;
    s->running.push_back(r.id);
    s->waiting.pop_front();
  }
  return 0;
}

// Called after the device step: the prompt (prefill) or one more token (decode) is now cached.
RT_EXPORT void gkrt_sched_commit(void* h, int64_t id, int is_prefill) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return;
  Request& r = it->second;
  if (is_prefill) {
    r.prefilled = true;
    r.cached_tokens = r.prompt_len;
  } else {
    ++r.cached_tokens;
    ++r.generated;
  }
}

RT_EXPORT void gkrt_sched_count_generated(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it != s->reqs.end()) ++it->second.generated;
}

RT_EXPORT void gkrt_sched_finish(void* h, int64_t id) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return;
  s->release(it->second);
  s->running.erase(std::remove(s->running.begin(), s->running.end(), id), s->running.end());
  s->waiting.erase(std::remove(s->waiting.begin(), s->waiting.end(), id), s->waiting.end());
  s->reqs.erase(it);
}

RT_EXPORT void gkrt_sched_abort_all(void* h) {
  auto* s = static_cast<Scheduler*>(h);
  for (auto& kv : s->reqs) s->release(kv.second);
  s->reqs.clear();
  s->running.clear();
  s->waiting.clear();
}

RT_EXPORT int gkrt_sched_block_table(void* h, int64_t id, int* out, int cap) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -1;
  const int n = std::min<int>(cap, it->second.blocks.size());
  std::memcpy(out, it->second.blocks.data(), n * sizeof(int));
  return static_cast<int>(it->second.blocks.size());
}

// Fills block tables ([n, max_blocks], -1 padded) and cached-token counts for a batch of requests in one call.
RT_EXPORT int gkrt_sched_batch_tables(void* h, const int64_t* ids, int n, int* tables, int max_blocks, int* cached) {
  auto* s = static_cast<Scheduler*>(h);
  for (int i = 0; i < n; ++i) {
    auto it = s->reqs.find(ids[i]);
    if (it == s->reqs.end()) return -1;
    const Request& r = it->second;
    int* row = tables + static_cast<size_t>(i) * max_blocks;
    const int nb = std::min<int>(max_blocks, r.blocks.size());
    std::memcpy(row, r.blocks.data(), nb * sizeof(int));
    for (int j = nb; j < max_blocks; ++j) row[j] = 0;
    cached[i] = r.cached_tokens;
  }
  return 0;
}

RT_EXPORT void gkrt_sched_stats(void* h, int64_t* out) {
  auto* s = static_cast<Scheduler*>(h);
  out[0] = static_cast<int64_t>(s->free_list.size());
  out[1] = static_cast<int64_t>(s->running.size());
  out[2] = static_cast<int64_t>(s->waiting.size());
  out[3] = s->preemptions;
  out[4] = s->num_blocks;
}

// Makes sure the request owns blocks for `tokens` more tokens beyond what is cached (multi-step decode reserves a
// whole interval at once).  Returns 0, or -1 when the cache cannot provide them.
RT_EXPORT int gkrt_sched_reserve(void* h, int64_t id, int tokens) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return -2;
  return s->alloc(it->second, it->second.cached_tokens + tokens) ? 0 : -1;
}

// `tokens` decode steps have run: their KV is cached.
RT_EXPORT void gkrt_sched_advance(void* h, int64_t id, int tokens) {
  auto* s = static_cast<Scheduler*>(h);
  auto it = s->reqs.find(id);
  if (it == s->reqs.end()) return;
  it->second.cached_tokens += tokens;
  it->second.generated += tokens;
}
