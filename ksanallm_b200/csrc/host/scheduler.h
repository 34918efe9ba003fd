// Continuous-batching scheduler core.
//
// Capability parity with the reference's BatchScheduler + ContinuousBatchingStrategy
// (src/ksana_llm/batch_scheduler/batch_scheduler.cpp:118-421,
//  strategy/continuous_batching.cpp:102-141, 391-605, 607-899) and the per-sequence state
// machine of InferRequest (src/ksana_llm/runtime/infer_request.cpp:173-446), redesigned around
// one flat "step plan" that is serialised into a single int32 staging buffer (one H2D per step).
//
// Per step:
//   1. running sequences get their next tokens (1 for decode, +drafts for speculative decoding,
//      a chunk for an unfinished prefill); blocks are grown; on exhaustion the most recently
//      admitted sequences are pre-empted (swap to host, or recompute);
//   2. swapped sequences come back while memory allows;
//   3. waiting sequences are admitted (prefix match, chunked prefill = split_fuse_token_num,
//      token / batch / launch-threshold caps, queue timeouts).
// After the model ran, Update() applies sampled tokens (including draft verification), commits
// filled blocks to the prefix tree and applies the finish rules.
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <memory>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "kv_cache.h"

namespace ksana {

enum RetCode : int {
  RET_SUCCESS = 0,
  RET_EXCEED_CAPACITY = 1,        // waiting queue full
  RET_INPUT_LENGTH_EXCEEDED = 2,  // prompt longer than max_token_len
  RET_INVALID_ARGUMENT = 3,
  RET_REQUEST_TIMEOUT = 4,
  RET_REQUEST_ABORTED = 5,
  RET_OUT_OF_MEMORY = 6,
};

enum FinishReason : int {
  FINISH_NONE = 0,
  FINISH_EOS = 1,
  FINISH_STOP_TOKEN = 2,
  FINISH_LENGTH = 3,
  FINISH_ABORTED = 4,
  FINISH_TIMEOUT = 5,
  FINISH_STOP_STRING = 6,
  FINISH_ERROR = 7,
};

enum SeqState : int { SEQ_WAITING = 0, SEQ_RUNNING = 1, SEQ_SWAPPED = 2, SEQ_FINISHED = 3 };

struct SchedulerConfig {
  int block_size = 16;
  int max_batch_size = 128;
  int max_step_tokens = 4096;
  int max_token_len = 2048;
  int max_waiting_queue_len = 1200;
  int64_t waiting_timeout_ms = 3600000;
  int split_fuse_token_num = 0;  // 0: a prompt is prefilled in one step if it fits the token cap
  int preempt_mode = 0;          // 0 swap, 1 recompute
  double launch_block_threshold = 2.0;
  double swapin_block_threshold = 2.0;
  int max_draft_tokens = 0;       // speculative tokens verified per decode step
  // Parallel token prediction: the "drafts" are register tokens appended after the sequence's last real tokens; the
  // model answers every register position with one more token, all of them are kept (nothing is verified) and the
  // registers' own KV entries are dropped. The reference: runtime/draft_generator/ptp_generator.cpp,
  // runtime/ptp_generation_controller.cpp.
  bool ptp_mode = false;
  // Non-prefix cache reuse: a run of at least this many tokens found elsewhere in the prefix tree is copied (keys
  // re-rotated) instead of being computed; 0 turns the search off (reference: min_flexible_cache_num).
  int min_flexible_cache_num = 0;
  // Pipeline micro-batch workload balancing (reference: batch_scheduler/workload_balance/pp_multibatch_balancer.cpp):
  // 0 = none (waiting sequences go to whichever micro-batch admits them), 1 = new sequences go to the least loaded
  // micro-batch, one unit per sequence; 2 = the same plus moving work off a micro-batch that exceeds 1.2x the mean;
  // 3 = like 2 with a sequence weighing 1 + (tokens to compute) / 200; 4 = like 2 weighing the tokens to compute.
  int pp_wb_strategy = 0;
  // Extra KV slots reserved past the tokens of a step: a multi-step draft module writes its own cache entries for
  // the positions it drafts ahead of (mtp_step_num - 1).
  int lookahead_slots = 0;
  int decode_token_threshold = 1;  // q_len <= threshold with cached KV counts as a decode entry
};

struct Sequence {
  int64_t id = 0;
  int64_t group_id = 0;
  std::vector<int32_t> tokens;  // prompt + generated
  int prompt_len = 0;
  int num_computed = 0;  // tokens whose KV is valid in the cache
  std::vector<int32_t> drafts;
  bool no_cache = false;  // the prompt's KV is not a function of its token ids alone: no prefix reuse, no commit
  int max_new_tokens = 16;
  bool ignore_eos = false;
  std::vector<int32_t> eos_ids;
  std::vector<int32_t> stop_ids;
  int64_t arrival_ms = 0;
  int state = SEQ_WAITING;
  int finish_reason = FINISH_NONE;
  int preempt_count = 0;
  int mb = -1;  // pipeline micro-batch this sequence belongs to (-1: none), fixed at admission
  // Held back from every queue's scheduling (it keeps its cache unless pre-empted): a beam that already has this
  // position's candidates waits here until the other beams of its request have theirs.
  bool paused = false;
  // in-flight step
  int sched_q_len = 0;
  int sched_drafts = 0;
  int sched_logits = 0;
  int num_generated() const { return static_cast<int>(tokens.size()) - prompt_len; }
};

struct StepEntry {
  int64_t seq_id;
  int q_start;     // tokens already in cache
  int q_len;       // tokens fed this step (real + drafts)
  int n_drafts;    // trailing draft tokens inside q_len
  int num_logits;  // rows that need logits: 0 (non-final chunk), 1, or 1 + n_drafts
  bool is_decode;
};

struct SeqEvent {
  int64_t seq_id;
  int finish_reason;
};

struct StepPlan {
  std::vector<StepEntry> entries;       // prefill entries first, then decode entries
  std::vector<CopyPair> swap_out;       // device -> host
  std::vector<CopyPair> swap_in;        // host -> device
  std::vector<CopyPair> block_copies;   // device -> device (fork copy-on-write)
  // flexible cache reuse, one row per token: (source slot, destination slot, source position, destination position);
  // executed before every other block operation of the step
  std::vector<int32_t> flexible;
  std::vector<SeqEvent> dropped;        // timed out / aborted before running
  int num_prefill = 0;
  int num_decode = 0;
  int total_tokens = 0;
  int total_logits = 0;
  int max_q_len = 0;
  int max_kv_len = 0;
  bool empty() const { return entries.empty(); }
};

struct StepResult {
  int64_t seq_id;
  std::vector<int32_t> new_tokens;
  int accepted_drafts;
  int finish_reason;  // FINISH_NONE while running
};

struct SchedStats {
  int64_t steps = 0;
  int64_t preempt_recompute = 0;
  int64_t preempt_swap = 0;
  int64_t swap_in = 0;
  int64_t mb_migrations = 0;  // sequences moved between pipeline micro-batches by the workload balancer
  int64_t draft_proposed = 0;
  int64_t draft_accepted = 0;
  int64_t timeouts = 0;
  int64_t finished = 0;
};

// Layout of the packed step buffer (int32 words). Every section starts on a 32-word boundary.
struct PackedLayout {
  int32_t num_seqs, num_prefill, num_decode, total_tokens, total_logits, max_q_len, max_kv_len, max_blocks;
  int32_t off_input_ids, off_positions, off_slot_mapping, off_cu_q, off_kv_lens, off_q_starts;
  int32_t off_logits_idx, off_block_tables, off_seq_of_token, total_words;
};

class Scheduler {
 public:
  Scheduler(const SchedulerConfig& cfg, std::shared_ptr<KVCacheManager> cache) : cfg_(cfg), cache_(std::move(cache)) {}

  const SchedulerConfig& config() const { return cfg_; }
  const SchedStats& stats() const { return stats_; }
  int num_waiting() const { return static_cast<int>(waiting_.size()); }
  int num_running() const { return static_cast<int>(running_.size()); }
  int num_swapped() const { return static_cast<int>(swapped_.size()); }
  bool has_unfinished() const { return !waiting_.empty() || !running_.empty() || !swapped_.empty(); }
  const Sequence* Get(int64_t id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? nullptr : it->second.get();
  }
  // Pending work of this scheduler in tokens (used for data-parallel balancing).
  int64_t Workload() const {
    int64_t w = 0;
    for (auto id : waiting_) {
      const Sequence& s = *seqs_.at(id);
      w += static_cast<int64_t>(s.tokens.size()) - s.num_computed;
    }
    for (auto id : running_) w += 1;
    for (auto id : swapped_) w += 1;
    return w;
  }

  int Enqueue(Sequence seq) {
    if (seq.tokens.empty() || seq.max_new_tokens < 0) return RET_INVALID_ARGUMENT;
    if (static_cast<int>(seq.tokens.size()) >= cfg_.max_token_len) return RET_INPUT_LENGTH_EXCEEDED;
    if (static_cast<int>(waiting_.size()) >= cfg_.max_waiting_queue_len) return RET_EXCEED_CAPACITY;
    if (seqs_.count(seq.id)) return RET_INVALID_ARGUMENT;
    // A sequence that can never fit in the cache would wait forever.
    int need = (static_cast<int>(seq.tokens.size()) + 1 + cfg_.block_size - 1) / cfg_.block_size;
    if (need > cache_->num_device_blocks()) return RET_OUT_OF_MEMORY;
    seq.prompt_len = static_cast<int>(seq.tokens.size());
    seq.state = SEQ_WAITING;
    int64_t id = seq.id;
    seqs_[id] = std::make_unique<Sequence>(std::move(seq));
    waiting_.push_back(id);
    return RET_SUCCESS;
  }

  // Marks a sequence aborted; it leaves the queues at the next Schedule()/Update().
  bool Abort(int64_t id) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return false;
    aborted_.insert(id);
    return true;
  }

  // Copy-on-write fork for parallel sampling / beam search. The child joins the running queue
  // right after its parent. The copies are attached to the next plan.
  bool Fork(int64_t parent, int64_t child) {
    auto it = seqs_.find(parent);
    if (it == seqs_.end() || seqs_.count(child)) return false;
    Sequence& p = *it->second;
    if (p.state != SEQ_RUNNING) return false;
    if (!cache_->Fork(parent, child, &pending_copies_)) return false;
    auto c = std::make_unique<Sequence>(p);
    c->id = child;
    c->drafts.clear();
    c->paused = false;
    seqs_[child] = std::move(c);
    auto pos = std::find(running_.begin(), running_.end(), parent);
    running_.insert(pos + 1, child);
    return true;
  }

  // Finishes a running sequence from outside (beam pruning, stop strings found by the detokenizer).
  bool Finish(int64_t id, int reason) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return false;
    RemoveFromQueues(id);
    Retire(*it->second, reason);
    return true;
  }

  // Replaces the tokens of a running sequence after `keep` tokens (beam search re-ranking keeps the
  // cache of the shared history and rewrites the last sampled token).
  bool ReplaceLastToken(int64_t id, int32_t token) {
    auto it = seqs_.find(id);
    if (it == seqs_.end() || it->second->tokens.empty()) return false;
    it->second->tokens.back() = token;
    return true;
  }

  void SetDrafts(int64_t id, const std::vector<int32_t>& drafts) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return;
    it->second->drafts = drafts;
    if (static_cast<int>(it->second->drafts.size()) > cfg_.max_draft_tokens)
      it->second->drafts.resize(cfg_.max_draft_tokens);
  }

  // Removes a finished sequence's record (the engine calls this after delivering the output).
  void Forget(int64_t id) {
    auto it = seqs_.find(id);
    if (it != seqs_.end() && it->second->state == SEQ_FINISHED) seqs_.erase(it);
  }

  // Pipeline micro-batches: with a filter set, Schedule() only touches the sequences of that micro-batch (and
  // assigns it to the sequences it admits), so that the other micro-batches' in-flight steps are left alone.
  // While set, Schedule() admits nothing from the waiting queue (running and swapped sequences go on). Attention
  // data parallelism uses it to line the ranks' prefills up (parallel/attn_dp.py ADPBalance).
  void SetHoldWaiting(bool hold) { hold_waiting_ = hold; }
  bool SetPaused(int64_t id, bool paused) {
    auto it = seqs_.find(id);
    if (it == seqs_.end()) return false;
    it->second->paused = paused;
    return true;
  }

  void SetMicroBatch(int mb, int count = 1) {
    mb_filter_ = mb;
    mb_count_ = count < 1 ? 1 : count;
  }

  int MicroBatchOf(int64_t id) const {
    auto it = seqs_.find(id);
    return it == seqs_.end() ? -1 : it->second->mb;
  }

  long SeqWorkload(const Sequence& s) const {
    long todo = std::max<long>(static_cast<long>(s.tokens.size()) - s.num_computed, 1);
    switch (cfg_.pp_wb_strategy) {
      case 3: return todo / 200 + 1;
      case 4: return todo;
      default: return 1;
    }
  }

  // Assigns unassigned waiting sequences to the least loaded micro-batch and, for the dynamic strategies, moves
  // work off the micro-batch about to be scheduled when it carries more than 1.2x the mean: waiting sequences
  // first, then running ones from the back of the queue. Only the micro-batch being scheduled gives work away (its
  // previous step has been collected, none of its sequences is in flight).
  void BalanceMicroBatches() {
    if (mb_filter_ < 0 || mb_count_ <= 1 || cfg_.pp_wb_strategy == 0) return;
    std::vector<long> load(mb_count_, 0);
    auto least = [&](int skip) {
      int best = -1;
      for (int m = 0; m < mb_count_; ++m)
        if (m != skip && (best < 0 || load[m] < load[best])) best = m;
      return best;
    };
    int mine = 0;
    for (auto* q : {&running_, &swapped_, &waiting_})
      for (int64_t id : *q) {
        Sequence& s = *seqs_.at(id);
        if (s.mb >= 0 && s.mb < mb_count_) {
          load[s.mb] += SeqWorkload(s);
          mine += s.mb == mb_filter_;
        }
      }
    for (int64_t id : waiting_) {
      Sequence& s = *seqs_.at(id);
      if (s.mb >= 0 && s.mb < mb_count_) continue;
      s.mb = least(-1);
      load[s.mb] += SeqWorkload(s);
      mine += s.mb == mb_filter_;
    }
    if (cfg_.pp_wb_strategy == 1 || mine < 5) return;
    long total = 0;
    for (long l : load) total += l;
    long ideal = (total + mb_count_ - 1) / mb_count_;
    if (load[mb_filter_] <= static_cast<long>(ideal * 1.2)) return;
    long to_move = load[mb_filter_] - ideal, moved = 0;
    auto give = [&](Sequence& s) {
      long w = SeqWorkload(s);
      if (moved + w > to_move) return false;
      load[mb_filter_] -= w;
      s.mb = least(mb_filter_);
      load[s.mb] += w;
      moved += w;
      ++stats_.mb_migrations;
      return true;
    };
    bool waiting_left = false;
    for (int64_t id : waiting_) {
      Sequence& s = *seqs_.at(id);
      if (s.mb != mb_filter_ || cache_->Has(id)) continue;
      if (moved >= to_move || !give(s)) {
        waiting_left = true;
        break;
      }
    }
    if (waiting_left) return;
    for (auto it = running_.rbegin(); it != running_.rend() && moved < to_move; ++it) {
      Sequence& s = *seqs_.at(*it);
      if (s.mb != mb_filter_) continue;
      if (!give(s)) break;
    }
  }

  StepPlan Schedule(int64_t now_ms) {
    StepPlan plan;
    ++stats_.steps;
    plan.block_copies.swap(pending_copies_);
    DropAbortedAndTimedOut(now_ms, &plan);
    BalanceMicroBatches();

    int token_budget = cfg_.max_step_tokens;
    int batch_budget = cfg_.max_batch_size;
    std::vector<StepEntry> prefill, decode;

    // ---- 1. running queue -------------------------------------------------------------------
    std::deque<int64_t> keep;
    while (!running_.empty()) {
      int64_t id = running_.front();
      Sequence& s = *seqs_.at(id);
      if ((mb_filter_ >= 0 && s.mb != mb_filter_) || s.paused) {
        running_.pop_front();
        keep.push_back(id);
        continue;
      }
      int remaining = static_cast<int>(s.tokens.size()) - s.num_computed;  // >= 1
      bool mid_prefill = remaining > 1;
      int n_drafts = mid_prefill ? 0 : std::min<int>(static_cast<int>(s.drafts.size()), cfg_.max_draft_tokens);
      int q_len = remaining;
      if (mid_prefill && cfg_.split_fuse_token_num > 0) q_len = std::min(q_len, cfg_.split_fuse_token_num);
      q_len = std::min(q_len, std::max(token_budget, 0));
      if (mid_prefill && cfg_.ptp_mode && q_len == remaining) {
        // the chunk reaches the sequence's end: the register tokens ride along if they still fit
        int want = std::min<int>(static_cast<int>(s.drafts.size()), cfg_.max_draft_tokens);
        if (remaining + want <= token_budget) n_drafts = want;
      }
      if (!mid_prefill || n_drafts > 0) q_len = remaining + n_drafts;
      if (batch_budget <= 0 || q_len <= 0 || q_len > token_budget) {
        // No room this step: the sequence simply waits in place (keeps its cache).
        running_.pop_front();
        keep.push_back(id);
        continue;
      }
      bool ok = cache_->EnsureCapacity(id, s.num_computed + q_len + cfg_.lookahead_slots);
      while (!ok) {
        // Pre-empt the most recently admitted sequence that is not yet planned this step.
        if (running_.size() <= 1) break;
        // (with a micro-batch filter only this micro-batch's sequences are candidates: the others may be in flight)
        auto vit = running_.end();
        for (auto it2 = running_.end(); it2 != running_.begin() + 1;) {
          --it2;
          if (mb_filter_ < 0 || seqs_.at(*it2)->mb == mb_filter_) {
            vit = it2;
            break;
          }
        }
        if (vit == running_.end()) break;
        int64_t victim = *vit;
        running_.erase(vit);
        Preempt(victim, &plan);
        ok = cache_->EnsureCapacity(id, s.num_computed + q_len + cfg_.lookahead_slots);
      }
      if (!ok) {
        running_.pop_front();
        const int need_blocks =
            (s.num_computed + q_len + cfg_.lookahead_slots + cfg_.block_size - 1) / cfg_.block_size;
        if (need_blocks > cache_->num_device_blocks()) {
          // It can never fit, not even with the whole pool to itself: pre-empting would only make it cycle
          // (recompute: re-admitted and thrown out again; swap: out, in, out). End it with what it has produced.
          Retire(s, FINISH_LENGTH);
          plan.dropped.push_back({id, FINISH_LENGTH});
          continue;
        }
        // Even alone it does not fit right now: pre-empt itself.
        Preempt(id, &plan);
        continue;
      }
      running_.pop_front();
      keep.push_back(id);
      bool final_chunk = (s.num_computed + q_len - n_drafts) == static_cast<int>(s.tokens.size());
      StepEntry e{id, s.num_computed, q_len, n_drafts, final_chunk ? 1 + n_drafts : 0,
                  !mid_prefill && q_len <= std::max(cfg_.decode_token_threshold, 1 + cfg_.max_draft_tokens)};
      (e.is_decode ? decode : prefill).push_back(e);
      token_budget -= q_len;
      --batch_budget;
    }
    running_.swap(keep);

    // ---- 2. swapped queue -------------------------------------------------------------------
    // (paused sequences move behind the others, in both queues, and end the scan when they are reached)
    auto not_paused = [&](int64_t q) { return !seqs_.at(q)->paused; };
    std::stable_partition(swapped_.begin(), swapped_.end(), not_paused);
    std::stable_partition(waiting_.begin(), waiting_.end(), not_paused);
    while (!swapped_.empty() && batch_budget > 0 && token_budget > 0 && plan.swap_out.empty()) {
      int64_t id = swapped_.front();
      Sequence& s = *seqs_.at(id);
      if (s.paused) break;
      if (mb_filter_ >= 0 && s.mb != mb_filter_) break;
      int need_now = 1 + std::min<int>(static_cast<int>(s.drafts.size()), cfg_.max_draft_tokens);
      int blocks_after = (s.num_computed + need_now + cfg_.block_size - 1) / cfg_.block_size;
      int extra = blocks_after - cache_->NumBlocks(id);
      int headroom = static_cast<int>(cfg_.swapin_block_threshold * (running_.size() + 1));
      if (cache_->NumHostBlocks(id) + std::max(extra, 0) + headroom > cache_->num_available_blocks() &&
          !running_.empty())
        break;
      if (!cache_->SwapIn(id, &plan.swap_in)) break;
      if (!cache_->EnsureCapacity(id, s.num_computed + need_now + cfg_.lookahead_slots)) {
        // Could not grow after coming back: stay resident, run next step.
        swapped_.pop_front();
        s.state = SEQ_RUNNING;
        running_.push_back(id);
        ++stats_.swap_in;
        continue;
      }
      swapped_.pop_front();
      s.state = SEQ_RUNNING;
      running_.push_back(id);
      ++stats_.swap_in;
      int n_drafts = need_now - 1;
      int remaining = static_cast<int>(s.tokens.size()) - s.num_computed;
      if (remaining == 1 && need_now <= token_budget) {
        StepEntry e{id, s.num_computed, need_now, n_drafts, 1 + n_drafts, true};
        decode.push_back(e);
        token_budget -= need_now;
        --batch_budget;
      }
    }

    // ---- 3. waiting queue -------------------------------------------------------------------
    bool preempted_now = !plan.swap_out.empty() || preempted_this_step_;
    preempted_this_step_ = false;
    // with micro-batches, one call admits its share of the queue so that the others get work too
    int admit_left = (mb_filter_ >= 0 && cfg_.pp_wb_strategy == 0)
                         ? std::max<int>(1, (static_cast<int>(waiting_.size()) + mb_count_ - 1) / mb_count_)
                         : (1 << 30);
    const bool swapped_ahead = !swapped_.empty() && !seqs_.at(swapped_.front())->paused;
    while (!hold_waiting_ && !waiting_.empty() && batch_budget > 0 && token_budget > 0 && !swapped_ahead &&
           !preempted_now && admit_left > 0) {
      if (seqs_.at(waiting_.front())->paused) break;
      --admit_left;
      if (mb_filter_ >= 0 && cfg_.pp_wb_strategy > 0) {
        // balanced micro-batches: admit this micro-batch's own waiting sequences, oldest first
        auto mine = std::find_if(waiting_.begin(), waiting_.end(),
                                 [&](int64_t w) { int m = seqs_.at(w)->mb; return (m == mb_filter_ || m < 0) && !seqs_.at(w)->paused; });
        if (mine == waiting_.end()) break;
        if (mine != waiting_.begin()) {
          int64_t w = *mine;
          waiting_.erase(mine);
          waiting_.push_front(w);
        }
      }
      int64_t id = waiting_.front();
      Sequence& s = *seqs_.at(id);
      size_t flex_mark = plan.flexible.size();
      if (!cache_->Has(id)) {
        int hit = s.no_cache ? 0 : cache_->MatchPrefix(s.tokens);
        int remaining = static_cast<int>(s.tokens.size()) - hit;
        int first = remaining;
        if (cfg_.split_fuse_token_num > 0) first = std::min(first, cfg_.split_fuse_token_num);
        first = std::min(first, token_budget);
        if (cfg_.split_fuse_token_num == 0 && first < remaining) {
          // Whole-prompt prefill does not fit what is left of this step's token budget. If it
          // fits a later step where it is first in line, wait for that step; otherwise it is
          // chunked by the budget.
          int fresh_budget = cfg_.max_step_tokens - static_cast<int>(decode.size());
          if (remaining <= fresh_budget && !prefill.empty()) break;
        }
        int blocks_needed = (hit + first + cfg_.block_size - 1) / cfg_.block_size - hit / cfg_.block_size;
        int headroom = static_cast<int>(cfg_.launch_block_threshold * running_.size());
        if (blocks_needed + headroom > cache_->num_available_blocks() && !running_.empty()) break;
        cache_->CreateSeq(id, s.tokens, !s.no_cache);
        s.num_computed = cache_->NumBlocks(id) * cfg_.block_size;
        flex_mark = plan.flexible.size();
        FlexibleRun run;
        if (cfg_.min_flexible_cache_num > 0 && !s.no_cache &&
            cache_->FlexibleReserve(id, s.tokens, s.num_computed, cfg_.min_flexible_cache_num, &run)) {
          for (int i = 0; i < run.size(); ++i) {
            plan.flexible.insert(plan.flexible.end(),
                                 {run.src_slots[i], run.dst_slots[i], run.src_pos[i], run.dst_begin + i});
          }
          s.num_computed += run.size();
        }
      }
      int remaining = static_cast<int>(s.tokens.size()) - s.num_computed;
      int q_len = remaining;
      if (cfg_.split_fuse_token_num > 0) q_len = std::min(q_len, cfg_.split_fuse_token_num);
      q_len = std::min(q_len, token_budget);
      if (q_len <= 0) break;
      if (!cache_->EnsureCapacity(id, s.num_computed + q_len + cfg_.lookahead_slots)) {
        if (running_.empty() && prefill.empty() && decode.empty()) {
          // Nothing else holds memory besides the cache itself; shrink the chunk to what fits.
          int fit = cache_->num_available_blocks() * cfg_.block_size;
          q_len = std::min(q_len, fit);
          if (q_len <= 0 || !cache_->EnsureCapacity(id, s.num_computed + q_len + cfg_.lookahead_slots)) {
            cache_->FreeSeq(id);
            s.num_computed = 0;
            plan.flexible.resize(flex_mark);
            break;
          }
        } else {
          cache_->FreeSeq(id);
          s.num_computed = 0;
          plan.flexible.resize(flex_mark);
          break;
        }
      }
      waiting_.pop_front();
      s.state = SEQ_RUNNING;
      if (mb_filter_ >= 0) s.mb = mb_filter_;
      running_.push_back(id);
      bool final_chunk = (s.num_computed + q_len) == static_cast<int>(s.tokens.size());
      bool as_decode = s.num_computed > 0 && q_len <= cfg_.decode_token_threshold;
      StepEntry e{id, s.num_computed, q_len, 0, final_chunk ? 1 : 0, as_decode};
      (as_decode ? decode : prefill).push_back(e);
      token_budget -= q_len;
      --batch_budget;
    }

    // Order: prefill by new-token count (desc), then decode by q_len (desc) — equal-q_len decode
    // entries are contiguous so one kernel launch covers each group.
    std::stable_sort(prefill.begin(), prefill.end(),
                     [](const StepEntry& a, const StepEntry& b) { return a.q_len > b.q_len; });
    std::stable_sort(decode.begin(), decode.end(),
                     [](const StepEntry& a, const StepEntry& b) { return a.q_len > b.q_len; });
    plan.num_prefill = static_cast<int>(prefill.size());
    plan.num_decode = static_cast<int>(decode.size());
    plan.entries = std::move(prefill);
    plan.entries.insert(plan.entries.end(), decode.begin(), decode.end());
    for (auto& e : plan.entries) {
      Sequence& s = *seqs_.at(e.seq_id);
      s.sched_q_len = e.q_len;
      s.sched_drafts = e.n_drafts;
      s.sched_logits = e.num_logits;
      plan.total_tokens += e.q_len;
      plan.total_logits += e.num_logits;
      plan.max_q_len = std::max(plan.max_q_len, e.q_len);
      plan.max_kv_len = std::max(plan.max_kv_len, e.q_start + e.q_len);
      stats_.draft_proposed += e.n_drafts;
    }
    return plan;
  }

  // Words needed by Pack() for this plan.
  int64_t PackedWords(const StepPlan& plan, int max_blocks) const {
    PackedLayout l;
    return ComputeLayout(plan, max_blocks, &l);
  }

  // Serialises the plan's device metadata into `buf` (capacity in words). Returns the layout;
  // total_words == -1 signals insufficient capacity.
  PackedLayout Pack(const StepPlan& plan, int32_t* buf, int64_t capacity, int max_blocks_hint) const {
    int max_blocks = std::max(1, max_blocks_hint);
    for (auto& e : plan.entries) max_blocks = std::max(max_blocks, cache_->NumBlocks(e.seq_id));
    PackedLayout l;
    int64_t words = ComputeLayout(plan, max_blocks, &l);
    if (words > capacity) {
      l.total_words = -1;
      return l;
    }
    int32_t* ids = buf + l.off_input_ids;
    int32_t* pos = buf + l.off_positions;
    int32_t* slot = buf + l.off_slot_mapping;
    int32_t* cu = buf + l.off_cu_q;
    int32_t* kvl = buf + l.off_kv_lens;
    int32_t* qs = buf + l.off_q_starts;
    int32_t* lg = buf + l.off_logits_idx;
    int32_t* bt = buf + l.off_block_tables;
    int32_t* sot = buf + l.off_seq_of_token;
    int t = 0, li = 0, b = 0;
    cu[0] = 0;
    const int bs = cfg_.block_size;
    for (auto& e : plan.entries) {
      const Sequence& s = *seqs_.at(e.seq_id);
      std::vector<BlockId> table = cache_->BlockTable(e.seq_id);
      int32_t* row = bt + static_cast<int64_t>(b) * max_blocks;
      for (int i = 0; i < max_blocks; ++i) row[i] = i < static_cast<int>(table.size()) ? table[i] : 0;
      int real = e.q_len - e.n_drafts;
      for (int i = 0; i < e.q_len; ++i) {
        int p = e.q_start + i;
        ids[t] = i < real ? s.tokens[p] : s.drafts[i - real];
        pos[t] = p;
        slot[t] = table[p / bs] * bs + p % bs;
        sot[t] = b;
        if (e.num_logits > 0 && i >= e.q_len - e.num_logits) lg[li++] = t;
        ++t;
      }
      cu[b + 1] = t;
      kvl[b] = e.q_start + e.q_len;
      qs[b] = e.q_start;
      ++b;
    }
    return l;
  }

  // Applies one step's sampled tokens. `sampled` holds plan.total_logits tokens in plan order.
  // `extra_stop` lets the caller veto acceptance (grammar): tokens after a vetoed one are dropped.
  std::vector<StepResult> Update(const StepPlan& plan, const std::vector<int32_t>& sampled, int64_t now_ms) {
    std::vector<StepResult> out;
    size_t cursor = 0;
    for (auto& e : plan.entries) {
      auto it = seqs_.find(e.seq_id);
      size_t base = cursor;
      cursor += e.num_logits;
      if (it == seqs_.end()) continue;
      Sequence& s = *it->second;
      if (s.state != SEQ_RUNNING) continue;  // finished/aborted while in flight
      StepResult r{e.seq_id, {}, 0, FINISH_NONE};
      int real = e.q_len - e.n_drafts;
      if (e.num_logits == 0) {
        s.num_computed += e.q_len;
        cache_->CommitFilled(s.id, s.tokens, s.num_computed);
        if (aborted_.count(s.id)) {
          RemoveFromQueues(s.id);
          Retire(s, FINISH_ABORTED);
          r.finish_reason = FINISH_ABORTED;
          out.push_back(std::move(r));
        }
        continue;
      }
      // Draft verification: sampled[i] is the model's token after (real tokens + drafts[0..i)).
      int accepted = 0;
      while (!cfg_.ptp_mode && accepted < e.n_drafts && sampled[base + accepted] == s.drafts[accepted] &&
             !IsStop(s, sampled[base + accepted])) {
        ++accepted;
      }
      stats_.draft_accepted += accepted;
      r.accepted_drafts = accepted;
      s.num_computed += real + accepted;
      int reason = FINISH_NONE;
      // parallel token prediction keeps the token of every register position; their KV is recomputed from the real
      // tokens in the next step (num_computed did not advance over the registers)
      int keep_upto = cfg_.ptp_mode ? e.n_drafts : accepted;
      for (int i = 0; i <= keep_upto; ++i) {
        int32_t tok = sampled[base + i];
        s.tokens.push_back(tok);
        r.new_tokens.push_back(tok);
        reason = CheckFinish(s, tok);
        if (reason != FINISH_NONE) break;
      }
      s.drafts.clear();
      cache_->CommitFilled(s.id, s.tokens, s.num_computed);
      if (reason == FINISH_NONE && aborted_.count(s.id)) reason = FINISH_ABORTED;
      if (reason != FINISH_NONE) {
        RemoveFromQueues(s.id);
        Retire(s, reason);
      }
      r.finish_reason = reason;
      out.push_back(std::move(r));
    }
    (void)now_ms;
    return out;
  }

  // Asynchronous scheduling: Update() may be called with PLACEHOLDER tokens (negative values, -(1 + row) where row
  // is the token's position in the step's sampled vector) before the device has produced the real ones, so that the
  // next step can be planned while this one runs. Placeholders never match a stop token; length limits still apply.
  // Resolve() later patches the real tokens in and reports the sequences that turn out to have finished on an EOS /
  // stop token. Such a sequence may already be part of the following in-flight step: Update() of that step skips it
  // (it is no longer running) and its blocks were released here; the stray KV write of the in-flight step lands
  // before any later step can reuse the blocks (same stream).
  // Requires one logit per entry (no draft tokens). Returns (seq_id, real token, finish_reason) per sampled row.
  std::vector<StepResult> Resolve(const StepPlan& plan, const std::vector<int32_t>& real) {
    std::vector<StepResult> out;
    size_t cursor = 0;
    for (auto& e : plan.entries) {
      size_t base = cursor;
      cursor += e.num_logits;
      if (e.num_logits == 0) continue;
      auto it = seqs_.find(e.seq_id);
      if (it == seqs_.end()) continue;
      Sequence& s = *it->second;
      const int32_t want = -(1 + static_cast<int32_t>(base));
      // the placeholder is the last token of the sequence (nothing was appended since)
      if (s.tokens.empty() || s.tokens.back() != want) continue;
      const int32_t tok = real[base];
      s.tokens.back() = tok;
      StepResult r{e.seq_id, {tok}, 0, s.state == SEQ_FINISHED ? s.finish_reason : FINISH_NONE};
      if (s.state != SEQ_FINISHED && IsStop(s, tok)) {
        int reason = FINISH_STOP_TOKEN;
        if (!s.ignore_eos)
          for (auto x : s.eos_ids)
            if (x == tok) reason = FINISH_EOS;
        RemoveFromQueues(s.id);
        Retire(s, reason);
        r.finish_reason = reason;
      }
      out.push_back(std::move(r));
    }
    return out;
  }

 private:
  int64_t ComputeLayout(const StepPlan& plan, int max_blocks, PackedLayout* l) const {
    auto align = [](int64_t x) { return (x + 31) / 32 * 32; };
    int B = static_cast<int>(plan.entries.size());
    int T = plan.total_tokens;
    int64_t off = 0;
    l->num_seqs = B;
    l->num_prefill = plan.num_prefill;
    l->num_decode = plan.num_decode;
    l->total_tokens = T;
    l->total_logits = plan.total_logits;
    l->max_q_len = plan.max_q_len;
    l->max_kv_len = plan.max_kv_len;
    l->max_blocks = max_blocks;
    l->off_input_ids = static_cast<int32_t>(off);
    off = align(off + T);
    l->off_positions = static_cast<int32_t>(off);
    off = align(off + T);
    l->off_slot_mapping = static_cast<int32_t>(off);
    off = align(off + T);
    l->off_seq_of_token = static_cast<int32_t>(off);
    off = align(off + T);
    l->off_cu_q = static_cast<int32_t>(off);
    off = align(off + B + 1);
    l->off_kv_lens = static_cast<int32_t>(off);
    off = align(off + B);
    l->off_q_starts = static_cast<int32_t>(off);
    off = align(off + B);
    l->off_logits_idx = static_cast<int32_t>(off);
    off = align(off + plan.total_logits);
    l->off_block_tables = static_cast<int32_t>(off);
    off = align(off + static_cast<int64_t>(B) * max_blocks);
    l->total_words = static_cast<int32_t>(off);
    return off;
  }

  bool IsStop(const Sequence& s, int32_t tok) const {
    if (!s.ignore_eos)
      for (auto e : s.eos_ids)
        if (e == tok) return true;
    for (auto e : s.stop_ids)
      if (e == tok) return true;
    return false;
  }

  int CheckFinish(const Sequence& s, int32_t tok) const {
    if (!s.ignore_eos)
      for (auto e : s.eos_ids)
        if (e == tok) return FINISH_EOS;
    for (auto e : s.stop_ids)
      if (e == tok) return FINISH_STOP_TOKEN;
    if (s.num_generated() >= s.max_new_tokens) return FINISH_LENGTH;
    if (static_cast<int>(s.tokens.size()) >= cfg_.max_token_len) return FINISH_LENGTH;
    return FINISH_NONE;
  }

  void Retire(Sequence& s, int reason) {
    cache_->FreeSeq(s.id);
    s.state = SEQ_FINISHED;
    s.finish_reason = reason;
    aborted_.erase(s.id);
    ++stats_.finished;
  }

  void RemoveFromQueues(int64_t id) {
    auto rm = [id](std::deque<int64_t>& q) {
      auto it = std::find(q.begin(), q.end(), id);
      if (it != q.end()) q.erase(it);
    };
    rm(waiting_);
    rm(running_);
    rm(swapped_);
  }

  void Preempt(int64_t id, StepPlan* plan) {
    Sequence& s = *seqs_.at(id);
    ++s.preempt_count;
    s.drafts.clear();
    bool mid_prefill = static_cast<int>(s.tokens.size()) - s.num_computed > 1;
    if (cfg_.preempt_mode == 0 && !mid_prefill && cache_->SwapOut(id, &plan->swap_out)) {
      s.state = SEQ_SWAPPED;
      swapped_.push_back(id);
      ++stats_.preempt_swap;
      return;
    }
    // Recompute: everything computed so far is dropped (blocks committed to the prefix tree stay
    // cached and are re-matched on re-admission).
    cache_->FreeSeq(id);
    s.num_computed = 0;
    s.state = SEQ_WAITING;
    waiting_.push_front(id);
    ++stats_.preempt_recompute;
    preempted_this_step_ = true;
  }

  void DropAbortedAndTimedOut(int64_t now_ms, StepPlan* plan) {
    auto sweep = [&](std::deque<int64_t>& q, bool check_timeout) {
      for (auto it = q.begin(); it != q.end();) {
        Sequence& s = *seqs_.at(*it);
        int reason = FINISH_NONE;
        if (aborted_.count(s.id))
          reason = FINISH_ABORTED;
        else if (check_timeout && cfg_.waiting_timeout_ms > 0 && now_ms - s.arrival_ms > cfg_.waiting_timeout_ms)
          reason = FINISH_TIMEOUT;
        if (reason != FINISH_NONE) {
          if (reason == FINISH_TIMEOUT) ++stats_.timeouts;
          it = q.erase(it);
          Retire(s, reason);
          plan->dropped.push_back({s.id, reason});
        } else {
          ++it;
        }
      }
    };
    sweep(waiting_, true);
    sweep(swapped_, true);
    sweep(running_, false);
  }

  SchedulerConfig cfg_;
  std::shared_ptr<KVCacheManager> cache_;
  std::unordered_map<int64_t, std::unique_ptr<Sequence>> seqs_;
  std::deque<int64_t> waiting_, running_, swapped_;
  std::unordered_set<int64_t> aborted_;
  std::vector<CopyPair> pending_copies_;
  int mb_filter_ = -1, mb_count_ = 1;
  bool hold_waiting_ = false;
  bool preempted_this_step_ = false;
  SchedStats stats_;
};

// Longest-processing-time greedy assignment of request workloads to data-parallel groups
// (capability of the reference's BalanceReqsAlgo, batch_scheduler_balance_reqs_algo.cpp:11-55).
inline std::vector<int> BalanceWorkloads(const std::vector<int64_t>& req_workloads,
                                         const std::vector<int64_t>& group_workloads) {
  std::vector<int> order(req_workloads.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = static_cast<int>(i);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return req_workloads[a] > req_workloads[b]; });
  std::vector<int64_t> load = group_workloads;
  std::vector<int> assign(req_workloads.size(), 0);
  for (int idx : order) {
    int best = 0;
    for (size_t g = 1; g < load.size(); ++g)
      if (load[g] < load[best]) best = static_cast<int>(g);
    assign[idx] = best;
    load[best] += req_workloads[idx];
  }
  return assign;
}

}  // namespace ksana
