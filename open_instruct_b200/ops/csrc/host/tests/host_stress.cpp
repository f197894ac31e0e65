// Sanitizer stress of the C++ host runtime (block manager + scheduler + packer), built together with host_runtime.cpp
// under -fsanitize=address,undefined and under -fsanitize=thread by tests/test_host_sanitizers_cpu.py.
//
// Part 1 drives one engine the way the rollout engine does, from several threads at once: a loop thread that schedules,
// advances and finishes sequences, producer threads that add requests (n samples sharing a prompt), and an observer that
// polls the counters - the mix `EngineWorker` produces with its loop thread, RPC threads and the actor manager.
// Invariants are checked along the way: blocks are conserved, nothing is scheduled twice in a step, a tiny cache
// forces preemption-by-recompute and still finishes everything.
// Part 2 packs ragged examples with the native packer into exactly sized buffers (any write past the end is an ASan report)
// from several threads and checks the packed rows against a plain restatement.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <random>
#include <set>
#include <thread>
#include <vector>

extern "C" {
void* b200_engine_create(int num_blocks, int block_size, int max_running);
void b200_engine_destroy(void* h);
int b200_engine_free_blocks(void* h);
int64_t b200_engine_preemptions(void* h);
int b200_engine_add(void* h, int64_t seq_id, int64_t group, int prompt_len, int max_len);
int b200_engine_finish(void* h, int64_t seq_id);
int b200_engine_schedule(void* h, int64_t* prefill_ids, int* n_prefill, int64_t* decode_ids, int* n_decode, int64_t* preempted_ids,
                         int* n_preempted, int cap);
int b200_engine_advance(void* h, int64_t seq_id, int new_tokens);
int b200_engine_blocks(void* h, int64_t seq_id, int* out, int cap, int* shared_prefix_tokens);
int b200_engine_counts(void* h, int* waiting, int* running);
int b200_engine_enable_prefix_cache(void* h, int on);
int b200_engine_reset_prefix_cache(void* h);
int b200_engine_prefix_cache_stats(void* h, int64_t* out);
int b200_engine_set_tokens(void* h, int64_t seq_id, const int* tokens, int n);
int b200_engine_cached_tokens(void* h, int64_t seq_id);
int b200_engine_finish_tokens(void* h, int64_t seq_id, const int* tokens, int n);
int b200_pack_plan(const int* lens, int n, int budget, int max_per_row, int* row_of);
int b200_pack_row(const int64_t* tokens, const int64_t* labels, const int64_t* starts, int first, int last, int64_t* out_ids,
                  int64_t* out_labels, int64_t* out_shifted, int64_t* out_pos, int32_t* out_cu);
int b200_numa_bind(int node);
}

#define CHECK(cond)                                                            \
  do {                                                                         \
    if (!(cond)) {                                                             \
      std::fprintf(stderr, "CHECK failed: %s (line %d)\n", #cond, __LINE__);  \
      std::exit(3);                                                            \
    }                                                                          \
  } while (0)

// `prefix_cache`: prompts are cut from five shared documents, so later requests start from blocks earlier ones left behind;
// sequences finish with their whole token list; an observer thread resets the cache now and then.
static void engine_stress(int num_blocks, int requests_per_producer, bool prefix_cache = false) {
  constexpr int BS = 16, PRODUCERS = 3, SAMPLES = 4;
  void* e = b200_engine_create(num_blocks, BS, 24);
  if (prefix_cache) b200_engine_enable_prefix_cache(e, 1);
  std::vector<std::vector<int>> toks(PRODUCERS * requests_per_producer * SAMPLES);
  std::mutex toks_mu;
  std::atomic<int64_t> next_seq{0};
  std::atomic<int> added{0}, finished{0};
  std::atomic<bool> producing{true};
  std::vector<int> target(PRODUCERS * requests_per_producer * SAMPLES, 0);  // generated tokens wanted per sequence

  auto producer = [&](int p) {
    std::mt19937 rng(100 + p);
    for (int r = 0; r < requests_per_producer; ++r) {
      const int prompt = 5 + rng() % 60, gen = 1 + rng() % 40;
      const int64_t group = p * 100000 + r;
      for (int s = 0; s < SAMPLES; ++s) {
        const int64_t id = next_seq.fetch_add(1);
        target[id] = gen;
        while (b200_engine_add(e, id, group, prompt, prompt + gen) != 0) std::this_thread::yield();
        if (prefix_cache) {
          std::vector<int> t(prompt);
          const int doc = static_cast<int>(group % 5);
          for (int i = 0; i < prompt; ++i) t[i] = (doc * 131 + i * 7) % 1000;
          b200_engine_set_tokens(e, id, t.data(), prompt);
          std::lock_guard<std::mutex> g(toks_mu);
          toks[id] = std::move(t);
        }
        added.fetch_add(1);
      }
      if (r % 7 == 0) std::this_thread::yield();
    }
  };
  auto observer = [&]() {
    while (producing.load() || finished.load() < added.load()) {
      int w = 0, r = 0;
      b200_engine_counts(e, &w, &r);
      CHECK(w >= 0 && r >= 0 && r <= 24);
      CHECK(b200_engine_free_blocks(e) <= num_blocks);
      if (prefix_cache) {
        int64_t st[4];
        b200_engine_prefix_cache_stats(e, st);
        CHECK(st[1] <= st[0] && st[3] >= 0 && st[3] <= num_blocks);
        if ((st[0] & 63) == 63) b200_engine_reset_prefix_cache(e);
      }
      std::this_thread::yield();
    }
  };
  auto loop = [&]() {
    std::vector<int64_t> pre(4096), dec(4096), pmt(4096);
    std::vector<int> produced(target.size(), 0);
    std::vector<int> blk(4096);
    const int total = static_cast<int>(target.size());
    long guard = 0;
    while (finished.load() < total) {
      CHECK(++guard < 50000000);
      int np = 0, nd = 0, nx = 0;
      b200_engine_schedule(e, pre.data(), &np, dec.data(), &nd, pmt.data(), &nx, 4096);
      std::set<int64_t> seen;
      for (int i = 0; i < np; ++i) CHECK(seen.insert(pre[i]).second);
      for (int i = 0; i < nd; ++i) CHECK(seen.insert(dec[i]).second);
      for (int i = 0; i < np + nd; ++i) {
        const int64_t id = i < np ? pre[i] : dec[i - np];
        int shared = 0;
        const int nb = b200_engine_blocks(e, id, blk.data(), 4096, &shared);
        CHECK(nb > 0 && shared >= 0);
        for (int b = 0; b < nb; ++b) CHECK(blk[b] >= 0 && blk[b] < num_blocks);
        if (prefix_cache && i < np) {
          const int c = b200_engine_cached_tokens(e, id);
          std::lock_guard<std::mutex> g(toks_mu);
          CHECK(c >= 0 && c % BS == 0 && c < static_cast<int>(toks[id].size()) + produced[id] + 1);
        }
        b200_engine_advance(e, id, 1);
        if (prefix_cache) {
          std::lock_guard<std::mutex> g(toks_mu);
          toks[id].push_back(static_cast<int>(id % 997));  // the "sampled" token
        }
        if (++produced[id] >= target[id]) {
          if (prefix_cache) {
            std::vector<int> all;
            {
              std::lock_guard<std::mutex> g(toks_mu);
              all = toks[id];
            }
            b200_engine_finish_tokens(e, id, all.data(), static_cast<int>(all.size()));
          } else {
            b200_engine_finish(e, id);
          }
          finished.fetch_add(1);
        }
      }
      for (int i = 0; i < nx; ++i) produced[pmt[i]] = produced[pmt[i]];  // preempted: recomputed later, progress kept by the caller
      if (np + nd == 0) std::this_thread::yield();
    }
  };
  std::vector<std::thread> ts;
  ts.emplace_back(loop);
  ts.emplace_back(observer);
  for (int p = 0; p < PRODUCERS; ++p) ts.emplace_back(producer, p);
  for (size_t i = 2; i < ts.size(); ++i) ts[i].join();
  producing.store(false);
  ts[0].join();
  ts[1].join();
  int w = 0, r = 0;
  b200_engine_counts(e, &w, &r);
  CHECK(w == 0 && r == 0);
  CHECK(b200_engine_free_blocks(e) == num_blocks);  // every block came back
  std::printf("engine: %d sequences, %lld preemptions, %d blocks\n", finished.load(), static_cast<long long>(b200_engine_preemptions(e)), num_blocks);
  b200_engine_destroy(e);
}

static void packer_stress(int seed) {
  std::mt19937 rng(seed);
  const int n = 200 + rng() % 100, budget = 256;
  std::vector<int> lens(n);
  std::vector<int64_t> starts(n + 1, 0);
  for (int i = 0; i < n; ++i) {
    lens[i] = 1 + rng() % 200;
    starts[i + 1] = starts[i] + lens[i];
  }
  std::vector<int64_t> tok(starts[n]), lab(starts[n]);
  for (auto& t : tok) t = rng() % 50000;
  for (size_t i = 0; i < lab.size(); ++i) lab[i] = (rng() % 3) ? tok[i] : -100;
  std::vector<int> row_of(n);
  const int rows = b200_pack_plan(lens.data(), n, budget, 5, row_of.data());
  CHECK(rows > 0 && row_of[n - 1] == rows - 1);
  int first = 0;
  for (int r = 0; r < rows; ++r) {
    int last = first;
    while (last < n && row_of[last] == r) ++last;
    const int64_t T = starts[last] - starts[first];
    CHECK(last - first <= 5 && (T <= budget || last - first == 1));
    std::vector<int64_t> ids(T), labels(T), shifted(T), pos(T);  // exactly sized: an overrun is a sanitizer report
    std::vector<int32_t> cu(last - first + 1);
    const int got = b200_pack_row(tok.data(), lab.data(), starts.data(), first, last, ids.data(), labels.data(), shifted.data(), pos.data(), cu.data());
    CHECK(got == T && cu.back() == T);
    int64_t o = 0;
    for (int i = first; i < last; ++i)
      for (int64_t k = 0; k < lens[i]; ++k, ++o) {
        CHECK(ids[o] == tok[starts[i] + k] && pos[o] == k);
        CHECK(labels[o] == (k == 0 ? -100 : lab[starts[i] + k]));
      }
    for (int64_t k = 0; k + 1 < T; ++k) CHECK(shifted[k] == labels[k + 1]);
    CHECK(T == 0 || shifted[T - 1] == -100);
    first = last;
  }
}

int main() {
  engine_stress(4096, 60);  // roomy cache
  engine_stress(40, 25);    // tiny cache: admission stalls and preemption-by-recompute
  engine_stress(4096, 40, true);  // prefix cache with room: hits, resets from another thread
  engine_stress(48, 25, true);    // prefix cache under pressure: eviction before preemption
  std::vector<std::thread> ts;
  for (int t = 0; t < 4; ++t) ts.emplace_back([t] { for (int k = 0; k < 20; ++k) packer_stress(1000 * t + k); });
  for (auto& t : ts) t.join();
  (void)b200_numa_bind(0);
  (void)b200_numa_bind(4096);  // unknown node: reports 0 and touches nothing
  std::printf("HOST_STRESS_OK\n");
  return 0;
}
