// C++ host runtime of the rollout engine and the data path (C ABI, used through ctypes).
//
//   BlockManager  paged-KV block allocator with reference counts; sequences that share a prompt
//                 (the n samples of one request) share its full blocks, each gets a private tail.
//   Scheduler     continuous batching: FIFO admission while blocks last, one decode slot per
//                 running sequence, preemption-by-recompute of the youngest sequence when the
//                 cache runs out.
//   pack_rows     greedy first-fit packing of variable-length examples into token-budgeted rows
//                 written straight into caller-provided (pinned) buffers with cu_seqlens.
//   numa_bind     pin the calling thread to the CPUs of one NUMA node (reads sysfs, no libnuma).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <fstream>
#include <list>
#include <mutex>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include <sched.h>

namespace {

struct Seq {
  int64_t id = 0;
  int64_t group = 0;          // request id: sequences of one group share prompt blocks
  int prompt_len = 0;
  int len = 0;                // tokens whose K/V are (or will be after this step) in the cache
  int max_len = 0;
  std::vector<int> blocks;
  bool running = false;
  bool needs_prefill = true;
  int64_t arrival = 0;
  std::vector<int> tokens;    // prompt token ids (prefix cache only)
  int cached_tokens = 0;      // tokens at the start of the sequence whose K/V were found in the prefix cache at admission
};

struct Engine {
  int block_size = 64;
  int num_blocks = 0;
  int max_running = 256;
  std::vector<int> refcnt;
  std::vector<int> free_list;
  std::unordered_map<int64_t, Seq> seqs;
  std::deque<int64_t> waiting;
  std::vector<int64_t> running;
  std::unordered_map<int64_t, std::vector<int>> group_prompt_blocks;  // full prompt blocks shared inside a group
  std::unordered_map<int64_t, int> group_users;
  int64_t clock = 0;
  int64_t preemptions = 0;
  std::mutex mu;

  // ---- prefix cache: full blocks keep their content after their last user is gone.  A block is identified by the chain
  // hash of all tokens up to and including its own (so equal hashes mean equal PREFIXES), verified against the stored
  // parent hash and token ids on every hit; unreferenced cached blocks wait in an LRU list and are taken back only when
  // the free list is empty.
  bool prefix_cache = false;
  std::vector<uint64_t> block_hash;              // 0 = not cached
  std::vector<uint64_t> block_parent;
  std::vector<std::vector<int>> block_tokens;
  std::unordered_map<uint64_t, int> cached;      // chain hash -> block
  std::list<int> evictable;                      // cached blocks with no user, least recently released first
  std::unordered_map<int, std::list<int>::iterator> ev_pos;
  int64_t cache_queries = 0, cache_hits = 0, cache_evictions = 0;   // in blocks

  static uint64_t chain_hash(uint64_t parent, const int* tok, int n) {
    uint64_t h = 1469598103934665603ull ^ (parent * 0x9E3779B97F4A7C15ull);
    for (int i = 0; i < n; ++i) {
      h ^= static_cast<uint32_t>(tok[i]);
      h *= 1099511628211ull;
    }
    return h ? h : 1;
  }
  void uncache(int b) {
    auto it = cached.find(block_hash[b]);
    if (it != cached.end() && it->second == b) cached.erase(it);
    block_hash[b] = 0;
    block_tokens[b].clear();
  }
  int alloc_block() {
    int b;
    if (!free_list.empty()) {
      b = free_list.back();
      free_list.pop_back();
    } else if (!evictable.empty()) {
      b = evictable.front();
      evictable.pop_front();
      ev_pos.erase(b);
      uncache(b);
      cache_evictions++;
    } else {
      return -1;
    }
    refcnt[b] = 1;
    return b;
  }
  int available_blocks() const { return static_cast<int>(free_list.size() + evictable.size()); }
  void release_block(int b) {
    if (--refcnt[b] != 0) return;
    if (prefix_cache && block_hash[b] != 0) {
      evictable.push_back(b);
      ev_pos[b] = std::prev(evictable.end());
    } else {
      free_list.push_back(b);
    }
  }
  // one more user of a cached block (it may have been waiting in the LRU list)
  void retain_cached(int b) {
    if (refcnt[b]++ == 0) {
      auto it = ev_pos.find(b);
      if (it != ev_pos.end()) {
        evictable.erase(it->second);
        ev_pos.erase(it);
      }
    }
  }
  // Blocks of the longest cached prefix of `tok` (whole blocks only, at most `max_blocks`).
  std::vector<int> lookup_prefix(const std::vector<int>& tok, int max_blocks) {
    std::vector<int> out;
    uint64_t parent = 0;
    for (int i = 0; i < max_blocks; ++i) {
      const int* t = tok.data() + static_cast<size_t>(i) * block_size;
      const uint64_t h = chain_hash(parent, t, block_size);
      cache_queries++;
      auto it = cached.find(h);
      if (it == cached.end()) break;
      const int b = it->second;
      if (block_parent[b] != parent || !std::equal(block_tokens[b].begin(), block_tokens[b].end(), t)) break;  // hash collision
      out.push_back(b);
      parent = h;
    }
    cache_hits += static_cast<int64_t>(out.size());
    return out;
  }
  // The first `n_tokens` tokens of `s` have their K/V in `s.blocks`: make its full blocks findable.
  void publish_blocks(const Seq& s, const int* tok, int n_tokens) {
    if (!prefix_cache) return;
    const int full = std::min<int>(n_tokens / block_size, static_cast<int>(s.blocks.size()));
    uint64_t parent = 0;
    for (int i = 0; i < full; ++i) {
      const int* t = tok + static_cast<size_t>(i) * block_size;
      const uint64_t h = chain_hash(parent, t, block_size);
      const int b = s.blocks[i];
      if (block_hash[b] == 0 && cached.find(h) == cached.end()) {
        block_hash[b] = h;
        block_parent[b] = parent;
        block_tokens[b].assign(t, t + block_size);
        cached.emplace(h, b);
      }
      parent = h;
    }
  }
  int blocks_needed(int tokens) const { return (tokens + block_size - 1) / block_size; }

  void free_seq_blocks(Seq& s) {
    for (int b : s.blocks) release_block(b);
    s.blocks.clear();
  }
  void drop_group_ref(int64_t g) {
    auto it = group_users.find(g);
    if (it == group_users.end()) return;
    if (--it->second == 0) {
      for (int b : group_prompt_blocks[g]) release_block(b);
      group_prompt_blocks.erase(g);
      group_users.erase(it);
    }
  }
};

}  // namespace

extern "C" {

void* b200_engine_create(int num_blocks, int block_size, int max_running) {
  auto* e = new Engine();
  e->num_blocks = num_blocks;
  e->block_size = block_size;
  e->max_running = max_running;
  e->refcnt.assign(num_blocks, 0);
  e->block_hash.assign(num_blocks, 0);
  e->block_parent.assign(num_blocks, 0);
  e->block_tokens.resize(num_blocks);
  e->free_list.reserve(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) e->free_list.push_back(i);
  return e;
}

void b200_engine_destroy(void* h) { delete static_cast<Engine*>(h); }

int b200_engine_free_blocks(void* h) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  return e->available_blocks();
}

// Prefix cache on / off (off also forgets everything cached).
int b200_engine_enable_prefix_cache(void* h, int on) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  e->prefix_cache = on != 0;
  if (!on) {
    for (int b : e->evictable) { e->uncache(b); e->free_list.push_back(b); }
    e->evictable.clear();
    e->ev_pos.clear();
    for (size_t b = 0; b < e->block_hash.size(); ++b)
      if (e->block_hash[b]) e->uncache(static_cast<int>(b));
  }
  return 0;
}

// Forget every cached prefix (after a weight update: K/V computed with older weights must not serve new requests).
// Blocks in use stay with their users and return to the free list when released.
int b200_engine_reset_prefix_cache(void* h) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  for (int b : e->evictable) { e->uncache(b); e->free_list.push_back(b); }
  e->evictable.clear();
  e->ev_pos.clear();
  for (size_t b = 0; b < e->block_hash.size(); ++b)
    if (e->block_hash[b]) e->uncache(static_cast<int>(b));
  return 0;
}

// out[0..2] = block lookups, block hits, evictions since creation; out[3] = cached blocks now
int b200_engine_prefix_cache_stats(void* h, int64_t* out) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  out[0] = e->cache_queries;
  out[1] = e->cache_hits;
  out[2] = e->cache_evictions;
  out[3] = static_cast<int64_t>(e->cached.size());
  return 0;
}

// Prompt token ids of a queued sequence (needed for prefix-cache lookups; call right after b200_engine_add).
int b200_engine_set_tokens(void* h, int64_t seq_id, const int* tokens, int n) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  auto it = e->seqs.find(seq_id);
  if (it == e->seqs.end()) return -1;
  it->second.tokens.assign(tokens, tokens + n);
  return 0;
}

// Tokens at the start of the sequence that need no prompt pass (their K/V came from the prefix cache at admission).
int b200_engine_cached_tokens(void* h, int64_t seq_id) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  auto it = e->seqs.find(seq_id);
  return it == e->seqs.end() ? -1 : it->second.cached_tokens;
}

// A sequence is done and `tokens[0..n)` is everything it holds (prompt + generated): the full blocks whose K/V were
// written (all but the last sampled token) become findable, then the sequence is removed like b200_engine_finish.
int b200_engine_finish_tokens(void* h, int64_t seq_id, const int* tokens, int n);

int64_t b200_engine_preemptions(void* h) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  return e->preemptions;
}

// Queue a sequence.  `group` ties the samples of one prompt together for prefix sharing.
int b200_engine_add(void* h, int64_t seq_id, int64_t group, int prompt_len, int max_len) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  if (e->seqs.count(seq_id)) return -1;
  if (e->blocks_needed(max_len) > e->num_blocks) return -2;  // can never fit
  Seq s;
  s.id = seq_id;
  s.group = group;
  s.prompt_len = prompt_len;
  s.len = prompt_len;
  s.max_len = max_len;
  s.arrival = e->clock++;
  e->seqs.emplace(seq_id, std::move(s));
  e->waiting.push_back(seq_id);
  e->group_users[group] += 1;
  return 0;
}

// Remove a finished (or aborted) sequence and free what only it was using.
int b200_engine_finish(void* h, int64_t seq_id) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  auto it = e->seqs.find(seq_id);
  if (it == e->seqs.end()) return -1;
  Seq& s = it->second;
  e->free_seq_blocks(s);
  e->running.erase(std::remove(e->running.begin(), e->running.end(), seq_id), e->running.end());
  e->waiting.erase(std::remove(e->waiting.begin(), e->waiting.end(), seq_id), e->waiting.end());
  e->drop_group_ref(s.group);
  e->seqs.erase(it);
  return 0;
}

int b200_engine_finish_tokens(void* h, int64_t seq_id, const int* tokens, int n) {
  {
    auto* e = static_cast<Engine*>(h);
    std::lock_guard<std::mutex> g(e->mu);
    auto it = e->seqs.find(seq_id);
    if (it == e->seqs.end()) return -1;
    const Seq& s = it->second;
    if (s.running && !s.needs_prefill && n > 1) e->publish_blocks(s, tokens, std::min(n, s.len) - 1);
  }
  return b200_engine_finish(h, seq_id);
}

// One scheduling step.
//   1. every running sequence gets room for one more token (a new block when it crosses a block
//      boundary); if the cache is full the youngest running sequence (possibly the one that asks) is preempted:
//      its blocks are freed and it goes back to the head of the waiting queue to be recomputed.  A sequence that
//      was already given its decode slot in this step is never the victim.
//   2. waiting sequences are admitted in FIFO order while their (prompt + 1 token) blocks fit and
//      the running set is below max_running.  Full prompt blocks are shared inside a group.
// Outputs: prefill_ids (sequences admitted this step, needing a prompt pass), decode_ids (sequences
// that decode one token this step), preempted_ids.  Returns 0.
int b200_engine_schedule(void* h, int64_t* prefill_ids, int* n_prefill, int64_t* decode_ids, int* n_decode,
                         int64_t* preempted_ids, int* n_preempted, int cap) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  *n_prefill = *n_decode = *n_preempted = 0;
  // ---- 1. growth of running sequences (oldest first)
  std::vector<int64_t> order = e->running;
  {
    // admission order is arrival order except after a preemption: look the arrivals up once, sort only if needed
    std::vector<std::pair<int64_t, int64_t>> keyed(order.size());
    for (size_t i = 0; i < order.size(); ++i) keyed[i] = {e->seqs[order[i]].arrival, order[i]};
    if (!std::is_sorted(keyed.begin(), keyed.end())) {
      std::sort(keyed.begin(), keyed.end());
      for (size_t i = 0; i < order.size(); ++i) order[i] = keyed[i].second;
    }
  }
  for (size_t i = 0; i < order.size(); ++i) {
    Seq& s = e->seqs[order[i]];
    if (!s.running) continue;  // preempted below
    const int need = e->blocks_needed(s.len + 1) - static_cast<int>(s.blocks.size());
    bool ok = true;
    for (int k = 0; k < need && ok; ++k) {
      int b = e->alloc_block();
      while (b < 0) {
        // The cache is full: the YOUNGEST running sequence gives its blocks back and is recomputed later.  Sequences
        // are visited oldest first, so the victim is either this sequence itself or one that has not been given its
        // decode slot yet - a sequence already listed in decode_ids is never taken apart afterwards.
        int64_t victim = -1;
        for (auto rit = order.rbegin(); rit != order.rend(); ++rit) {
          if (e->seqs[*rit].running) { victim = *rit; break; }
        }
        if (victim < 0) { ok = false; break; }
        Seq& v = e->seqs[victim];
        e->free_seq_blocks(v);
        v.running = false;
        v.needs_prefill = true;
        e->running.erase(std::remove(e->running.begin(), e->running.end(), victim), e->running.end());
        e->waiting.push_front(victim);
        e->preemptions++;
        if (*n_preempted < cap) preempted_ids[(*n_preempted)++] = victim;
        if (victim == s.id) { ok = false; break; }  // this sequence was the youngest: it waits, nothing to grow
        b = e->alloc_block();
      }
      if (!ok) break;
      s.blocks.push_back(b);
    }
    if (ok && *n_decode < cap) decode_ids[(*n_decode)++] = s.id;
  }
  // ---- 2. admission
  while (!e->waiting.empty() && static_cast<int>(e->running.size()) < e->max_running && *n_prefill < cap) {
    Seq& s = e->seqs[e->waiting.front()];
    const int full_prompt_blocks = s.prompt_len / e->block_size;
    auto shared = e->group_prompt_blocks.find(s.group);
    const bool can_share = shared != e->group_prompt_blocks.end() && s.len == s.prompt_len;
    const int total_needed = e->blocks_needed(s.len + 1);
    std::vector<int> hit;
    if (e->prefix_cache && !can_share && !s.tokens.empty()) {
      // whole blocks of the prompt, leaving at least one token to compute (its logits start the generation)
      const int known = std::min<int>(static_cast<int>(s.tokens.size()), s.len);
      hit = e->lookup_prefix(s.tokens, std::max(0, (known - 1) / e->block_size));
    }
    const int fresh = can_share ? total_needed - full_prompt_blocks : total_needed - static_cast<int>(hit.size());
    int hit_waiting = 0;  // hit blocks that sit in the LRU list are not available as fresh blocks
    for (int b : hit) hit_waiting += e->refcnt[b] == 0;
    if (fresh > e->available_blocks() - hit_waiting) break;
    s.blocks.clear();
    s.cached_tokens = 0;
    if (can_share) {
      for (int b : shared->second) { e->refcnt[b]++; s.blocks.push_back(b); }
    } else {
      for (int b : hit) { e->retain_cached(b); s.blocks.push_back(b); }
      s.cached_tokens = static_cast<int>(hit.size()) * e->block_size;
    }
    while (static_cast<int>(s.blocks.size()) < total_needed) s.blocks.push_back(e->alloc_block());
    if (!can_share && s.len == s.prompt_len && full_prompt_blocks > 0 && e->group_users[s.group] > 1) {
      // first sequence of its group: publish its full prompt blocks (the group holds its own reference)
      std::vector<int> pub(s.blocks.begin(), s.blocks.begin() + full_prompt_blocks);
      for (int b : pub) e->refcnt[b]++;
      e->group_prompt_blocks[s.group] = std::move(pub);
    }
    s.running = true;
    e->running.push_back(s.id);
    e->waiting.pop_front();
    prefill_ids[(*n_prefill)++] = s.id;
  }
  return 0;
}

// After the engine produced one token for `seq_id` (prefill's first token or a decode step).
int b200_engine_advance(void* h, int64_t seq_id, int new_tokens) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  auto it = e->seqs.find(seq_id);
  if (it == e->seqs.end()) return -1;
  Seq& s = it->second;
  if (s.needs_prefill && !s.tokens.empty())  // the prompt pass has written these K/V: later requests may start from them
    e->publish_blocks(s, s.tokens.data(), std::min<int>(static_cast<int>(s.tokens.size()), s.len));
  s.len += new_tokens;
  s.needs_prefill = false;
  return s.len;
}

// Block ids of a sequence; returns the count (or -1).  `shared_prefix_tokens` = tokens whose K/V
// were already written by another member of the group (no need to write them again).
int b200_engine_blocks(void* h, int64_t seq_id, int* out, int cap, int* shared_prefix_tokens) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  auto it = e->seqs.find(seq_id);
  if (it == e->seqs.end()) return -1;
  const Seq& s = it->second;
  const int n = static_cast<int>(s.blocks.size());
  for (int i = 0; i < n && i < cap; ++i) out[i] = s.blocks[i];
  if (shared_prefix_tokens) {
    int shared = 0;
    auto sh = e->group_prompt_blocks.find(s.group);
    if (sh != e->group_prompt_blocks.end() && !sh->second.empty() && !s.blocks.empty() && s.blocks[0] == sh->second[0])
      shared = static_cast<int>(sh->second.size()) * e->block_size;
    *shared_prefix_tokens = shared;
  }
  return n;
}

// Inputs of one decode step for `n` sequences, written straight into the caller's (pinned) staging arrays: position of
// the new token, its cache slot, context length, sampled-token counter and the zero-padded block table (row stride =
// widest table rounded up to `round_to`, returned in *max_blocks).  One call replaces a per-sequence round trip.
// Returns 0; -1 unknown sequence; -2 table does not fit `bt_cap` ints.
int b200_engine_pack_decode(void* h, const int64_t* ids, int n, int round_to, int64_t* pos, int64_t* slots, int32_t* ctx,
                            int32_t* ctr, int32_t* bt, int64_t bt_cap, int* max_blocks) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  std::vector<const Seq*> ss(n);
  int need = 1;
  for (int i = 0; i < n; ++i) {
    auto it = e->seqs.find(ids[i]);
    if (it == e->seqs.end() || it->second.len < 1) return -1;
    ss[i] = &it->second;
    need = std::max(need, static_cast<int>(it->second.blocks.size()));
  }
  if (round_to > 1) need = (need + round_to - 1) / round_to * round_to;
  if (static_cast<int64_t>(n) * need > bt_cap) return -2;
  *max_blocks = need;
  const int bs = e->block_size;
  for (int i = 0; i < n; ++i) {
    const Seq& s = *ss[i];
    const int last = s.len - 1;
    if (last / bs >= static_cast<int>(s.blocks.size())) return -1;
    pos[i] = last;
    slots[i] = static_cast<int64_t>(s.blocks[last / bs]) * bs + last % bs;
    ctx[i] = s.len;
    ctr[i] = s.len - s.prompt_len;
    int32_t* row = bt + static_cast<int64_t>(i) * need;
    const int nb = static_cast<int>(s.blocks.size());
    for (int k = 0; k < nb; ++k) row[k] = s.blocks[k];
    for (int k = nb; k < need; ++k) row[k] = 0;
  }
  return 0;
}

// One new token for each of `n` sequences (the batched form of b200_engine_advance).
int b200_engine_advance_many(void* h, const int64_t* ids, int n) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  for (int i = 0; i < n; ++i) {
    auto it = e->seqs.find(ids[i]);
    if (it == e->seqs.end()) return -1;
    Seq& s = it->second;
    if (s.needs_prefill && !s.tokens.empty())
      e->publish_blocks(s, s.tokens.data(), std::min<int>(static_cast<int>(s.tokens.size()), s.len));
    s.len += 1;
    s.needs_prefill = false;
  }
  return 0;
}

int b200_engine_counts(void* h, int* waiting, int* running) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  *waiting = static_cast<int>(e->waiting.size());
  *running = static_cast<int>(e->running.size());
  return 0;
}

// ---------------------------------------------------------------------------------------- packer
// Greedy first-fit in arrival order: example i (length lens[i]) goes into the current row unless it
// would exceed `budget` tokens (or `max_per_row` examples); rows are emitted into flat buffers:
//   row_of[i]      row index of example i
//   Returns the number of rows.
int b200_pack_plan(const int* lens, int n, int budget, int max_per_row, int* row_of) {
  int row = 0, used = 0, cnt = 0;
  for (int i = 0; i < n; ++i) {
    if (cnt > 0 && (used + lens[i] > budget || (max_per_row > 0 && cnt >= max_per_row))) {
      ++row;
      used = 0;
      cnt = 0;
    }
    row_of[i] = row;
    used += lens[i];
    ++cnt;
  }
  return n > 0 ? row + 1 : 0;
}

// Copy examples [first, last) (token ids + labels, concatenated in `tokens`/`labels` with offsets
// `starts`) into one packed row: ids, labels (first token of every document masked to -100),
// shifted labels, position ids, cu_seqlens.  Returns the row length.
int b200_pack_row(const int64_t* tokens, const int64_t* labels, const int64_t* starts, int first, int last, int64_t* out_ids,
                  int64_t* out_labels, int64_t* out_shifted, int64_t* out_pos, int32_t* out_cu) {
  int64_t o = 0;
  out_cu[0] = 0;
  for (int i = first; i < last; ++i) {
    const int64_t a = starts[i], b = starts[i + 1], n = b - a;
    std::memcpy(out_ids + o, tokens + a, sizeof(int64_t) * n);
    std::memcpy(out_labels + o, labels ? labels + a : tokens + a, sizeof(int64_t) * n);
    if (n > 0) out_labels[o] = -100;
    for (int64_t k = 0; k < n; ++k) out_pos[o + k] = k;
    o += n;
    out_cu[i - first + 1] = static_cast<int32_t>(o);
  }
  for (int64_t k = 0; k + 1 < o; ++k) out_shifted[k] = out_labels[k + 1];
  if (o > 0) out_shifted[o - 1] = -100;
  return static_cast<int>(o);
}

// ---------------------------------------------------------------------------------------- NUMA
// Bind the calling thread to the CPUs of `node` as listed by /sys/devices/system/node/nodeN/cpulist.
// Returns the number of CPUs in the mask, 0 if the node is unknown, -1 on failure.
int b200_numa_bind(int node) {
  std::ifstream f("/sys/devices/system/node/node" + std::to_string(node) + "/cpulist");
  if (!f.good()) return 0;
  std::string line;
  std::getline(f, line);
  cpu_set_t set;
  CPU_ZERO(&set);
  int count = 0;
  std::stringstream ss(line);
  std::string part;
  while (std::getline(ss, part, ',')) {
    const size_t dash = part.find('-');
    int a = std::stoi(part.substr(0, dash));
    int b = dash == std::string::npos ? a : std::stoi(part.substr(dash + 1));
    for (int c = a; c <= b && c < CPU_SETSIZE; ++c) { CPU_SET(c, &set); ++count; }
  }
  if (count == 0) return 0;
  return sched_setaffinity(0, sizeof(set), &set) == 0 ? count : -1;
}

}  // extern "C"
