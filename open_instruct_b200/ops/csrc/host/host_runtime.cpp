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

  int alloc_block() {
    if (free_list.empty()) return -1;
    int b = free_list.back();
    free_list.pop_back();
    refcnt[b] = 1;
    return b;
  }
  void release_block(int b) {
    if (--refcnt[b] == 0) free_list.push_back(b);
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
  e->free_list.reserve(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) e->free_list.push_back(i);
  return e;
}

void b200_engine_destroy(void* h) { delete static_cast<Engine*>(h); }

int b200_engine_free_blocks(void* h) {
  auto* e = static_cast<Engine*>(h);
  std::lock_guard<std::mutex> g(e->mu);
  return static_cast<int>(e->free_list.size());
}

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
    const int fresh = can_share ? total_needed - full_prompt_blocks : total_needed;
    if (fresh > static_cast<int>(e->free_list.size())) break;
    s.blocks.clear();
    if (can_share) {
      for (int b : shared->second) { e->refcnt[b]++; s.blocks.push_back(b); }
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
  it->second.len += new_tokens;
  it->second.needs_prefill = false;
  return it->second.len;
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
    it->second.len += 1;
    it->second.needs_prefill = false;
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
