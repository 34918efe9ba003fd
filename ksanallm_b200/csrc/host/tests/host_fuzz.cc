// Randomised driver for the host runtime (block manager + prefix tree, continuous-batching scheduler, draft trie),
// meant to be built with -fsanitize=address,undefined: thousands of steps of a simulated serving loop under memory
// pressure (tiny block pools) with shared prefixes, chunked prefill, speculative drafts, forks, aborts, swap and
// recompute pre-emption. Beyond what the sanitizers report, it checks that every block is back in the pool (free or
// cached) once all requests are done, that each step respects the token and batch caps, and that the packed step
// buffer stays inside its capacity.
//
//   g++ -std=c++17 -O1 -g -fsanitize=address,undefined -fno-sanitize-recover=all -I.. host_fuzz.cc -o host_fuzz
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <set>
#include <stdexcept>
#include <vector>

#include "draft_trie.h"
#include "scheduler.h"

using namespace ksana;

#define CHECK(cond)                                                              \
  do {                                                                           \
    if (!(cond)) {                                                               \
      std::fprintf(stderr, "CHECK failed at line %d: %s (round %d)\n", __LINE__, #cond, g_round); \
      std::exit(2);                                                              \
    }                                                                            \
  } while (0)

static int g_round = 0;
static long g_steps = 0, g_swaps = 0, g_recomputes = 0, g_prefix_hits = 0, g_flexible_hits = 0, g_accepted = 0,
            g_finished = 0, g_forks = 0;

static void OneRound(uint32_t seed) {
  std::mt19937 rng(seed);
  auto rnd = [&](int lo, int hi) { return lo + static_cast<int>(rng() % static_cast<uint32_t>(hi - lo + 1)); };
  SchedulerConfig cfg;
  cfg.block_size = 4 << rnd(0, 2);
  cfg.max_batch_size = rnd(2, 12);
  cfg.max_step_tokens = rnd(32, 160);
  cfg.max_token_len = 200;
  cfg.split_fuse_token_num = rnd(0, 1) ? rnd(8, 48) : 0;
  const int host_blocks = rnd(0, 1) ? rnd(8, 64) : 0;
  cfg.preempt_mode = host_blocks ? rnd(0, 1) : 1;
  cfg.max_draft_tokens = rnd(0, 1) ? rnd(1, 3) : 0;
  cfg.lookahead_slots = cfg.max_draft_tokens ? rnd(0, 2) : 0;
  cfg.decode_token_threshold = 1 + cfg.max_draft_tokens;
  cfg.min_flexible_cache_num = rnd(0, 3) == 0 ? 2 * cfg.block_size : 0;
  cfg.ptp_mode = cfg.max_draft_tokens > 0 && rnd(0, 3) == 0;  // register tokens: every position yields a token
  const int micro_batches = rnd(0, 2) == 0 ? rnd(2, 3) : 1;   // pipeline micro-batches taking turns
  cfg.pp_wb_strategy = micro_batches > 1 ? rnd(0, 4) : 0;
  const int dev_blocks = rnd(200 / cfg.block_size + 4, 400 / cfg.block_size + 24);
  auto cache = std::make_shared<KVCacheManager>(dev_blocks, host_blocks, cfg.block_size, rnd(0, 3) != 0);
  Scheduler sched(cfg, cache);
  DraftTrie trie(8, 1 << 12);

  std::vector<std::vector<int32_t>> stems;  // shared prompt beginnings -> prefix hits
  for (int i = 0; i < 4; ++i) {
    std::vector<int32_t> s(rnd(4, 60));
    for (auto& t : s) t = rnd(1, 50);
    stems.push_back(s);
  }
  std::set<int64_t> live, paused;
  int64_t next_id = 1, now = 0;
  const int total_requests = rnd(20, 80);
  int issued = 0;
  std::vector<int32_t> buf(1 << 18);

  for (int step = 0; step < 20000 && (issued < total_requests || !live.empty()); ++step) {
    now += 5;
    while (issued < total_requests && rnd(0, 2) == 0) {  // arrivals
      Sequence s;
      s.id = next_id++;
      s.group_id = s.id;
      s.tokens = stems[rnd(0, 3)];
      if (rnd(0, 1)) {  // a stem somewhere in the middle: candidate for non-prefix reuse
        std::vector<int32_t> head(rnd(1, 9));
        for (auto& t : head) t = rnd(51, 99);
        head.insert(head.end(), s.tokens.begin(), s.tokens.end());
        s.tokens = head;
      }
      for (int k = rnd(0, 30); k > 0; --k) s.tokens.push_back(rnd(1, 99));
      s.prompt_len = static_cast<int>(s.tokens.size());
      s.max_new_tokens = rnd(1, 40);
      s.ignore_eos = rnd(0, 1);
      s.eos_ids = {7};
      s.stop_ids = {8};
      s.no_cache = rnd(0, 9) == 0;
      s.arrival_ms = now;
      if (sched.Enqueue(s) == 0) live.insert(s.id);
      ++issued;
    }
    if (!live.empty() && rnd(0, 40) == 0) {  // a client goes away
      auto it = live.begin();
      std::advance(it, rnd(0, static_cast<int>(live.size()) - 1));
      sched.Abort(*it);
    }
    if (!live.empty() && rnd(0, 30) == 0) {  // parallel sampling / beam: fork a running sequence
      auto it = live.begin();
      std::advance(it, rnd(0, static_cast<int>(live.size()) - 1));
      const Sequence* p = sched.Get(*it);
      if (p != nullptr && p->state == SEQ_RUNNING && p->num_generated() > 0) {
        if (sched.Fork(*it, next_id)) {
          live.insert(next_id);
          ++g_forks;
        }
        ++next_id;
      }
    }
    if (!live.empty() && rnd(0, 50) == 0) {  // stop string found by the detokenizer / beam pruned: finished from outside
      auto it = live.begin();
      std::advance(it, rnd(0, static_cast<int>(live.size()) - 1));
      const Sequence* p = sched.Get(*it);
      if (p != nullptr && p->state == SEQ_RUNNING && sched.Finish(*it, FINISH_ABORTED)) {
        sched.Forget(*it);
        live.erase(it);
      }
    }
    if (!live.empty() && rnd(0, 20) == 0) {  // beam search rewrites the token it just got
      auto it = live.begin();
      std::advance(it, rnd(0, static_cast<int>(live.size()) - 1));
      const Sequence* p = sched.Get(*it);
      if (p != nullptr && p->state == SEQ_RUNNING && p->num_generated() > 0) sched.ReplaceLastToken(*it, rnd(1, 99));
    }
    if (!live.empty() && rnd(0, 6) == 0) {  // a beam ahead of its siblings is held back for a few steps
      auto it = live.begin();
      std::advance(it, rnd(0, static_cast<int>(live.size()) - 1));
      if (sched.SetPaused(*it, true)) paused.insert(*it);
    }
    if (step % 5 == 0) {
      for (int64_t id : paused) sched.SetPaused(id, false);
      paused.clear();
    }
    sched.SetHoldWaiting(rnd(0, 15) == 0);  // the data-parallel balancer holds admissions back for a step
    for (int64_t id : live) {  // drafts from the trie for decoding sequences
      const Sequence* s = sched.Get(id);
      if (cfg.max_draft_tokens && s != nullptr && s->state == SEQ_RUNNING && s->num_generated() > 0 && rnd(0, 1)) {
        std::vector<int32_t> d = trie.Propose(cfg.max_draft_tokens);
        if (d.empty()) d.assign(static_cast<size_t>(rnd(1, cfg.max_draft_tokens)), rnd(1, 99));
        sched.SetDrafts(id, d);
      }
    }
    if (micro_batches > 1) sched.SetMicroBatch(step % micro_batches, micro_batches);
    StepPlan plan = sched.Schedule(now);
    for (const auto& ev : plan.dropped) {
      live.erase(ev.seq_id);
      sched.Forget(ev.seq_id);
    }
    if (plan.empty()) continue;
    CHECK(plan.total_tokens <= cfg.max_step_tokens + cfg.max_batch_size * cfg.max_draft_tokens);
    CHECK(static_cast<int>(plan.entries.size()) <= cfg.max_batch_size);
    CHECK(plan.flexible.size() % 4 == 0);
    int logits = 0;
    for (const auto& e : plan.entries) {
      CHECK(e.q_len > 0 && e.n_drafts <= e.q_len && e.num_logits <= e.q_len);
      CHECK(cache->NumBlocks(e.seq_id) * cfg.block_size >= e.q_start + e.q_len);
      logits += e.num_logits;
    }
    CHECK(logits == plan.total_logits);
    PackedLayout l = sched.Pack(plan, buf.data(), static_cast<int64_t>(buf.size()), 1);
    CHECK(l.total_words > 0 && l.total_words <= static_cast<int32_t>(buf.size()));
    for (int t = 0; t < plan.total_tokens; ++t) {
      int slot = buf[l.off_slot_mapping + t];
      CHECK(slot >= -1 && slot < dev_blocks * cfg.block_size);
    }
    std::vector<int32_t> sampled(static_cast<size_t>(plan.total_logits));
    for (auto& t : sampled) t = rnd(1, 60);  // 7 = EOS, 8 = stop id turn up regularly
    for (const auto& r : sched.Update(plan, sampled, now)) {
      for (int32_t t : r.new_tokens) trie.FeedOne(t);
      if (r.finish_reason != FINISH_NONE) {
        live.erase(r.seq_id);
        sched.Forget(r.seq_id);
      }
    }
  }
  CHECK(live.empty());
  g_steps += sched.stats().steps;
  g_swaps += sched.stats().preempt_swap;
  g_recomputes += sched.stats().preempt_recompute;
  g_accepted += sched.stats().draft_accepted;
  g_finished += sched.stats().finished;
  g_prefix_hits += cache->stats().prefix_hit_tokens;
  g_flexible_hits += cache->stats().flexible_hit_tokens;
  CHECK(sched.num_running() == 0 && sched.num_waiting() == 0);
  CHECK(cache->num_free_blocks() + cache->num_cached_blocks() == dev_blocks);
  CHECK(cache->num_free_host_blocks() == host_blocks);
  cache->ClearUnreferenced();
  CHECK(cache->num_free_blocks() == dev_blocks);
}

int main(int argc, char** argv) {
  const int rounds = argc > 1 ? std::atoi(argv[1]) : 200;
  const uint32_t seed0 = argc > 2 ? static_cast<uint32_t>(std::atoll(argv[2])) : 1u;
  for (g_round = 0; g_round < rounds; ++g_round) {
    try {
      OneRound(seed0 + static_cast<uint32_t>(g_round));
    } catch (const std::exception& e) {
      std::fprintf(stderr, "round %d (seed %u): %s\n", g_round, seed0 + static_cast<uint32_t>(g_round), e.what());
      return 3;
    }
  }
  std::printf("host_fuzz: %d rounds ok (steps %ld, finished %ld, forks %ld, swap pre-emptions %ld, recompute pre-emptions %ld, "
              "prefix-hit tokens %ld, flexible-hit tokens %ld, accepted drafts %ld)\n",
              rounds, g_steps, g_finished, g_forks, g_swaps, g_recomputes, g_prefix_hits, g_flexible_hits, g_accepted);
  return 0;
}
